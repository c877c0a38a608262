"""Chunked streaming of serialized tensors (thin aliases of the implementations in ``compression.serialization``)."""
from hivemind_b200.compression.serialization import (STREAMING_CHUNK_SIZE_BYTES, combine_from_streaming,  # noqa: F401
                                                     split_for_streaming)
