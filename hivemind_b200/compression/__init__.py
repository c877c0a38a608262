"""Tensor compression codecs for averaging and expert RPCs."""
from hivemind_b200.compression.adaptive import PerTensorCompression, RoleAdaptiveCompression, SizeAdaptiveCompression
from hivemind_b200.compression.base import CompressionBase, CompressionInfo, NoCompression, TensorRole
from hivemind_b200.compression.floating import Float16Compression, ScaledFloat16Compression
from hivemind_b200.compression.quantization import (BlockwiseQuantization, Quantile8BitQuantization,
                                                    Uniform8BitQuantization)
from hivemind_b200.compression.serialization import (combine_from_streaming, deserialize_tensor_stream,
                                                     deserialize_torch_tensor, serialize_torch_tensor,
                                                     split_for_streaming)
