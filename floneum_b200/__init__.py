"""floneum_b200: B200 (sm_100a) attention for fusor-ml behind the reference's own API.

Only the attention hot path lives here: `Tensor.flash_attention`, `MaskKind`,
`AttentionMask`, `MaskCache` and `KvCache` mirror the names, arguments and error
behaviour of fusor (fusor-ml/fusor/src/composite/flash_attention.rs,
fusor-ml/fusor/src/cache/*.rs); all arithmetic runs in libfusor_cuda.so
(include/fusor_cuda.h).  Importing the package loads that library and fails if it is
missing.
"""
from ._lib import FusorCudaError, load  # noqa: F401

load()

from .device import Device  # noqa: E402,F401
from .tensor import MaskKind, Tensor  # noqa: E402,F401
from .cache import AttentionMask, KvCache, LlamaCache, MaskCache, PagedKvCache  # noqa: E402,F401
from .rope import RopeCache, rope  # noqa: E402,F401
