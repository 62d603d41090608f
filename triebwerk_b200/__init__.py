"""triebwerk_b200: the TurboQuant KV-cache append and GQA decode attention of BY571/triebwerk, rebuilt for
B200 (sm_100a) behind the reference's own launcher / Engine interface.

Everything here is a thin host mirror over ``csrc/libtriebwerk_b200.so`` (C ABI in
``include/triebwerk_b200.h``).  PyTorch is used for device memory and streams only.
"""
from ._lib import LIB_PATH, SYMBOLS, TqError, lib  # noqa: F401
from .engine import Engine  # noqa: F401
from .partition import lpt_partition, contiguous_partition  # noqa: F401
from . import ops  # noqa: F401
