"""Host side of the B200 kernels: ctypes binding, tensor-level wrappers, sharding."""
from . import _lib  # noqa: F401
from ._lib import B200KError, device_status, launch_count  # noqa: F401
