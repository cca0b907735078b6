"""Host-side mirror of the reference's `Backend` / `Workspace` pair over the C ABI.

`B200Backend.dispatch(call, workspace)` is `Backend::dispatch(&KernelCall, &mut Workspace)`
(crates/hologram-compute/src/backend.rs:8-15); `DeviceWorkspace` is a device-resident
slot table (the role BufferArena plays in crates/hologram-exec/src/buffer.rs); `HostWorkspace`
is the reference tests' `TestWorkspace { slots: Vec<Vec<u8>> }` (tests/lut.rs:13-49) whose
dispatch stages operands through the device per call.

The CUDA library is mandatory: importing this module without the built
`libhologram_b200.so` raises; there is no CPU path.
"""
import ctypes as C
import os
import weakref

import numpy as np

from . import kernel_call as kc

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libhologram_b200.so")


class BackendError(RuntimeError):
    """A failed C-ABI call; `.code` is the negative status, `.variant` the BackendError variant name."""
    VARIANTS = {kc.ERR_SLOT_OUT_OF_RANGE: "SlotOutOfRange", kc.ERR_SHAPE_MISMATCH: "ShapeMismatch",
                kc.ERR_UNSUPPORTED_OP: "UnsupportedOp", kc.ERR_INIT: "Init", kc.ERR_DISPATCH: "Dispatch"}

    def __init__(self, code, message, slot=None):
        super().__init__(f"{self.VARIANTS.get(code, code)}: {message}")
        self.code = code
        self.variant = self.VARIANTS.get(code, str(code))
        self.slot = slot


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python hologram_b200/build.py` "
            "(the B200 backend has no CPU fallback)")
    lib = C.CDLL(LIB_PATH)
    vp, u32, u64, i32 = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int32
    sigs = {
        "holo_b200_last_error": (C.c_char_p, []),
        "holo_b200_last_error_slot": (u32, []),
        "holo_b200_version": (C.c_char_p, []),
        "holo_b200_ctx_create": (i32, [i32, C.POINTER(vp)]),
        "holo_b200_ctx_destroy": (None, [vp]),
        "holo_b200_ctx_stream": (vp, [vp]),
        "holo_b200_ctx_set_stream": (i32, [vp, vp]),
        "holo_b200_ctx_synchronize": (i32, [vp]),
        "holo_b200_ctx_launch_count": (u64, [vp]),
        "holo_b200_ctx_set_lut_table": (i32, [vp, C.c_uint8, C.c_uint8, vp]),
        "holo_b200_ctx_get_lut_table": (i32, [vp, C.c_uint8, C.c_uint8, vp]),
        "holo_b200_workspace_create": (i32, [vp, u32, C.POINTER(vp)]),
        "holo_b200_workspace_destroy": (None, [vp]),
        "holo_b200_workspace_alloc": (i32, [vp, u32, u64]),
        "holo_b200_workspace_bind": (i32, [vp, u32, vp, u64]),
        "holo_b200_workspace_slot": (i32, [vp, u32, C.POINTER(vp), C.POINTER(u64)]),
        "holo_b200_workspace_upload": (i32, [vp, kc.BufferRef, vp, u64]),
        "holo_b200_workspace_download": (i32, [vp, kc.BufferRef, vp, u64]),
        "holo_b200_dispatch": (i32, [vp, C.POINTER(kc.KernelCall), vp]),
        "holo_b200_dispatch_host": (i32, [vp, C.POINTER(kc.KernelCall), C.POINTER(kc.HostSlot), u32]),
        "holo_b200_nccl_unique_id": (i32, [vp]),
        "holo_b200_ctx_init_tp": (i32, [vp, vp, i32, i32]),
        "holo_b200_ctx_tp_transport": (i32, [vp]),
        "holo_b200_tp_emulate_all_reduce": (i32, [vp, i32, C.POINTER(vp), C.POINTER(vp), C.POINTER(vp), u64, C.c_uint8, i32]),
    }
    for name, (res, args) in sigs.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()
EXPORTED_SYMBOLS = [
    "holo_b200_last_error", "holo_b200_last_error_slot", "holo_b200_version", "holo_b200_ctx_create",
    "holo_b200_ctx_destroy", "holo_b200_ctx_stream", "holo_b200_ctx_set_stream", "holo_b200_ctx_synchronize",
    "holo_b200_ctx_launch_count", "holo_b200_ctx_set_lut_table", "holo_b200_ctx_get_lut_table",
    "holo_b200_workspace_create", "holo_b200_workspace_destroy", "holo_b200_workspace_alloc",
    "holo_b200_workspace_bind", "holo_b200_workspace_slot", "holo_b200_workspace_upload",
    "holo_b200_workspace_download", "holo_b200_dispatch", "holo_b200_dispatch_host", "holo_b200_nccl_unique_id",
    "holo_b200_ctx_init_tp", "holo_b200_ctx_tp_transport", "holo_b200_tp_emulate_all_reduce",
]


def _check(rc):
    if rc != kc.OK:
        slot = lib.holo_b200_last_error_slot() if rc == kc.ERR_SLOT_OUT_OF_RANGE else None
        raise BackendError(rc, lib.holo_b200_last_error().decode("utf-8", "replace"), slot)


def _host_ptr(arr):
    return arr.ctypes.data_as(C.c_void_p)


class B200Backend:
    """Per-GPU backend state: stream, LUT tables, scratch (the `Backend` implementor)."""

    def __init__(self, device=0):
        h = C.c_void_p()
        _check(lib.holo_b200_ctx_create(device, C.byref(h)))
        self._h = h
        self.device = device
        self._workspaces = weakref.WeakSet()

    def close(self):
        """Destroy the context; device workspaces created on it are destroyed first."""
        if getattr(self, "_h", None):
            for ws in list(self._workspaces):
                ws.close()
            lib.holo_b200_ctx_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def stream(self):
        return lib.holo_b200_ctx_stream(self._h)

    def set_stream(self, cuda_stream):
        _check(lib.holo_b200_ctx_set_stream(self._h, C.c_void_p(cuda_stream)))

    def synchronize(self):
        _check(lib.holo_b200_ctx_synchronize(self._h))

    @property
    def launch_count(self):
        return int(lib.holo_b200_ctx_launch_count(self._h))

    def lut_table(self, act, dtype):
        out = np.empty(65536, dtype=np.uint16)
        _check(lib.holo_b200_ctx_get_lut_table(self._h, act, dtype, _host_ptr(out)))
        return out

    def set_lut_table(self, act, dtype, table):
        t = np.ascontiguousarray(table, dtype=np.uint16)
        assert t.size == 65536
        _check(lib.holo_b200_ctx_set_lut_table(self._h, act, dtype, _host_ptr(t)))

    def init_tp(self, unique_id, rank, world):
        buf = (C.c_uint8 * 128).from_buffer_copy(bytes(unique_id))
        _check(lib.holo_b200_ctx_init_tp(self._h, buf, rank, world))

    @property
    def tp_transport(self):
        """0 = no tensor-parallel group, 1 = NCCL, 2 = the one-shot peer-memory kernel."""
        return int(lib.holo_b200_ctx_tp_transport(self._h))

    def emulate_all_reduce(self, workspace, partial_slots, out_slots, count, dtype, residual_slots=None, repeats=1):
        """The peer-memory all-reduce with every rank emulated on this GPU (one cooperative launch)."""
        w = len(partial_slots)
        arr = lambda slots: (C.c_void_p * w)(*[workspace.slot(s)[0] for s in slots])
        res = arr(residual_slots) if residual_slots is not None else None
        _check(lib.holo_b200_tp_emulate_all_reduce(self._h, w, arr(partial_slots), res, arr(out_slots), count, dtype, repeats))

    @staticmethod
    def nccl_unique_id():
        buf = (C.c_uint8 * 128)()
        _check(lib.holo_b200_nccl_unique_id(buf))
        return bytes(buf)

    def dispatch(self, call, workspace):
        """`Backend::dispatch`: enqueue `call` against `workspace` (device or host form)."""
        if isinstance(workspace, HostWorkspace):
            _check(lib.holo_b200_dispatch_host(self._h, C.byref(call), workspace._table, len(workspace.slots)))
        else:
            _check(lib.holo_b200_dispatch(self._h, C.byref(call), workspace._h))


class DeviceWorkspace:
    """Device-resident `Workspace`: slot -> (device pointer, bytes)."""

    def __init__(self, backend, n_slots):
        h = C.c_void_p()
        _check(lib.holo_b200_workspace_create(backend._h, n_slots, C.byref(h)))
        self._h = h
        self.backend = backend
        self.n_slots = n_slots
        backend._workspaces.add(self)

    def close(self):
        if getattr(self, "_h", None):
            lib.holo_b200_workspace_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def alloc(self, slot, nbytes):
        _check(lib.holo_b200_workspace_alloc(self._h, slot, nbytes))

    def bind(self, slot, device_ptr, nbytes):
        _check(lib.holo_b200_workspace_bind(self._h, slot, C.c_void_p(device_ptr), nbytes))

    def slot(self, slot):
        p, n = C.c_void_p(), C.c_uint64()
        _check(lib.holo_b200_workspace_slot(self._h, slot, C.byref(p), C.byref(n)))
        return p.value, n.value

    def write(self, buf, array):
        """Upload `array`'s bytes into the range `buf` (Workspace::write)."""
        if isinstance(buf, int):
            buf = kc.rb(buf)
        a = np.ascontiguousarray(array)
        _check(lib.holo_b200_workspace_upload(self._h, buf, _host_ptr(a), a.nbytes))

    def put(self, slot, array):
        """Allocate `slot` to fit `array` and upload it."""
        a = np.ascontiguousarray(array)
        self.alloc(slot, a.nbytes)
        self.write(slot, a)

    def read(self, buf, nbytes=None, dtype=np.uint8):
        """Download the range `buf` (Workspace::read); synchronises."""
        if isinstance(buf, int):
            buf = kc.rb(buf)
        if nbytes is None:
            nbytes = buf.length if buf.length else self.slot(buf.slot)[1] - buf.offset
        out = np.empty(nbytes, dtype=np.uint8)
        _check(lib.holo_b200_workspace_download(self._h, buf, _host_ptr(out), nbytes))
        return out.view(dtype)


class HostWorkspace:
    """`TestWorkspace { slots: Vec<Vec<u8>> }`: numpy byte buffers; dispatch stages them per call."""

    def __init__(self, slots):
        self.slots = [np.ascontiguousarray(s).view(np.uint8).reshape(-1) for s in slots]
        self._table = (kc.HostSlot * len(self.slots))()
        for i, s in enumerate(self.slots):
            self._table[i].ptr = s.ctypes.data
            self._table[i].bytes = s.nbytes
