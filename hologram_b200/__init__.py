"""hologram_b200 — B200 (sm_100a) CUDA backend for hologram's tensor engine.

Host-side mirror of the reference `hologram-compute` backend boundary
(`Backend::dispatch(&KernelCall, &mut Workspace)`) over the C ABI in include/hologram_b200.h.

The pure-Python parts (the `KernelCall` mirror, the archive writer, the decoder archive builder)
import without the native library. Everything that executes (`B200Backend`, `DeviceWorkspace`,
`InferenceSession`, `DevicePool` ...) loads `libhologram_b200.so` on first use and raises if it has
not been built: there is no CPU path.
"""
from . import kernel_call

_BACKEND = ("B200Backend", "BackendError", "DeviceWorkspace", "HostWorkspace", "EXPORTED_SYMBOLS", "LIB_PATH", "DevicePool")
_SESSION = ("InferenceSession", "archive_check", "WeightStore")

__all__ = ["kernel_call", *_BACKEND, *_SESSION]


def __getattr__(name):
    if name in _BACKEND:
        from . import backend
        return getattr(backend, name)
    if name in _SESSION:
        from . import session
        return getattr(session, name)
    raise AttributeError(f"module 'hologram_b200' has no attribute {name!r}")
