"""Shared pieces of the ALBERT example: the metrics record that trainers publish and the validators that guard it
(same record as the reference's examples/albert/utils.py:12-28)."""
from typing import Dict, List, Tuple

from pydantic.v1 import BaseModel, StrictFloat, confloat, conint

import hivemind_b200 as hivemind
from hivemind_b200.dht.crypto import RSASignatureValidator
from hivemind_b200.dht.schema import BytesWithPublicKey, SchemaValidator
from hivemind_b200.dht.validation import RecordValidatorBase


class LocalMetrics(BaseModel):
    step: conint(ge=0, strict=True)
    samples_per_second: confloat(ge=0.0, strict=True)
    samples_accumulated: conint(ge=0, strict=True)
    loss: StrictFloat
    mini_steps: conint(ge=0, strict=True)


class MetricSchema(BaseModel):
    metrics: Dict[BytesWithPublicKey, LocalMetrics]


def make_validators(run_id: str) -> Tuple[List[RecordValidatorBase], bytes]:
    """Records under ``{run_id}_metrics`` must match the schema and be signed by the peer whose key is the subkey."""
    signature_validator = RSASignatureValidator()
    validators = [SchemaValidator(MetricSchema, prefix=run_id), signature_validator]
    return validators, signature_validator.local_public_key


COMPRESSIONS = {
    "none": hivemind.NoCompression, "float16": hivemind.Float16Compression,
    "meanstd16": hivemind.ScaledFloat16Compression, "uniform8": hivemind.Uniform8BitQuantization,
    "quantile8": hivemind.Quantile8BitQuantization, "blockwise8": hivemind.BlockwiseQuantization,
}


def make_compression(name: str):
    """A codec by name; ``size_adaptive`` sends small tensors as fp16 and large ones as 8-bit uniform."""
    if name == "size_adaptive":
        return hivemind.SizeAdaptiveCompression(threshold=2 ** 16 + 1, less=hivemind.Float16Compression(),
                                                greater_equal=hivemind.Uniform8BitQuantization())
    return COMPRESSIONS[name]()
