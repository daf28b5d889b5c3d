"""B200-native NVFP4 weight-GEMM path: ctypes binding of libq27b200.so plus the host-side layout helpers."""

from . import layouts, q27lib  # noqa: F401
from .q27lib import call, lib  # noqa: F401
