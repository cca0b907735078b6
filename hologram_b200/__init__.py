"""hologram_b200 — B200 (sm_100a) CUDA backend for hologram's tensor engine.

Host-side mirror of the reference `hologram-compute` backend boundary
(`Backend::dispatch(&KernelCall, &mut Workspace)`) over the C ABI in include/hologram_b200.h.
"""
from . import kernel_call
from .backend import B200Backend, BackendError, DeviceWorkspace, HostWorkspace, EXPORTED_SYMBOLS, LIB_PATH

from .session import InferenceSession, archive_check

__all__ = ["InferenceSession", "archive_check", "kernel_call", "B200Backend", "BackendError", "DeviceWorkspace", "HostWorkspace", "EXPORTED_SYMBOLS",
           "LIB_PATH"]
