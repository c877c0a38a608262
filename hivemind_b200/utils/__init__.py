from hivemind_b200.utils.asyncio import *  # noqa
from hivemind_b200.utils.limits import increase_file_limit
from hivemind_b200.utils.logging import get_logger, use_hivemind_log_handler
from hivemind_b200.utils.mpfuture import MPFuture
from hivemind_b200.utils.nested import nested_compare, nested_flatten, nested_map, nested_pack
from hivemind_b200.utils.performance_ema import PerformanceEMA
from hivemind_b200.utils.serializer import MSGPackSerializer, SerializerBase
from hivemind_b200.utils.tensor_descr import BatchTensorDescriptor, TensorDescriptor
from hivemind_b200.utils.timed_storage import (MAX_DHT_TIME_DISCREPANCY_SECONDS, DHTExpiration, TimedStorage,
                                               ValueWithExpiration, get_dht_time)
