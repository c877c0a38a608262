"""Shared pieces of the ALBERT example: the metrics record that trainers publish and the validators that guard it
(same record as the reference's examples/albert/utils.py:12-28)."""
from typing import Dict, List, Tuple

from pydantic.v1 import BaseModel, StrictFloat, confloat, conint

import hivemind_b200 as hivemind
from hivemind_b200.dht.crypto import RSASignatureValidator
from hivemind_b200.dht.schema import BytesWithPublicKey, SchemaValidator
from hivemind_b200.dht.validation import RecordValidatorBase


class LocalMetrics(BaseModel):
    """One trainer's progress report, published under ``{run_id}_metrics`` with the trainer's public key as subkey."""
    step: conint(ge=0, strict=True)  # collaborative step (epoch) this report belongs to
    samples_per_second: confloat(ge=0.0, strict=True)
    samples_accumulated: conint(ge=0, strict=True)
    loss: StrictFloat  # mean loss over mini_steps
    mini_steps: conint(ge=0, strict=True)  # forward/backward passes since the previous report


def metrics_schema():
    """The pydantic model that validates the whole ``metrics`` dictionary (field name = DHT key without prefix)."""

    class MetricSchema(BaseModel):
        metrics: Dict[BytesWithPublicKey, LocalMetrics]

    return MetricSchema


def make_validators(run_id: str) -> Tuple[List[RecordValidatorBase], bytes]:
    """Validators for a trainer's DHT: schema check of the metrics key plus RSA ownership of every subkey.
    Returns them together with this process's public key (the subkey to publish under)."""
    ownership = RSASignatureValidator()
    schema = SchemaValidator(metrics_schema(), prefix=run_id)
    return [schema, ownership], ownership.local_public_key


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
