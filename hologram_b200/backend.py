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
        "holo_b200_ctx_init_tp_timeout": (i32, [vp, vp, i32, i32, u32]),
        "holo_b200_ctx_tp_transport": (i32, [vp]),
        "holo_b200_tp_emulate_all_reduce": (i32, [vp, i32, C.POINTER(vp), C.POINTER(vp), C.POINTER(vp), u64, C.c_uint8, i32]),
        "holo_b200_tp_emulate_all_reduce_ex": (i32, [vp, i32, C.POINTER(vp), C.POINTER(vp), C.POINTER(vp), u64, C.c_uint8, i32, i32, u32]),
        "holo_b200_decode_attention_q8_static": (i32, [vp] * 12 + [u32] * 6 + [C.c_uint8]),
        "holo_b200_decode_attention_q8_static_status": (i32, [vp]),
        "holo_b200_pool_create": (i32, [vp, C.POINTER(vp)]),
        "holo_b200_pool_destroy": (None, [vp]),
        "holo_b200_pool_rebind_reset": (i32, [vp, u32]),
        "holo_b200_pool_store_unbound": (i32, [vp, vp, vp, u64]),
        "holo_b200_pool_pin_bytes": (i32, [vp, vp, vp, u64]),
        "holo_b200_pool_bind_fresh": (i32, [vp, u32, u64]),
        "holo_b200_pool_bind_resident": (i32, [vp, u32, vp]),
        "holo_b200_pool_retain": (i32, [vp, u32, vp]),
        "holo_b200_pool_steal_transient": (i32, [vp, vp, C.POINTER(u32), u32, u32]),
        "holo_b200_pool_lease": (i32, [vp, vp]),
        "holo_b200_pool_release": (i32, [vp, vp]),
        "holo_b200_pool_resident": (i32, [vp, vp]),
        "holo_b200_pool_bindable_input": (i32, [vp, vp]),
        "holo_b200_pool_resolve": (i32, [vp, vp, vp, u64, C.POINTER(u64)]),
        "holo_b200_pool_slot": (i32, [vp, u32, C.POINTER(vp), C.POINTER(u64)]),
        "holo_b200_pool_write_slot": (i32, [vp, u32, vp, u64]),
        "holo_b200_pool_set_lazy_budget": (i32, [vp, u64]),
        "holo_b200_pool_pin_lazy": (i32, [vp, vp, vp, u64]),
        "holo_b200_pool_page_and_bind": (i32, [vp, C.POINTER(u32), vp, u32, vp]),
        "holo_b200_pool_stats": (i32, [vp, vp]),
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
    "holo_b200_ctx_init_tp_timeout", "holo_b200_tp_emulate_all_reduce_ex", "holo_b200_decode_attention_q8_static",
    "holo_b200_decode_attention_q8_static_status", "holo_b200_pool_create", "holo_b200_pool_destroy",
    "holo_b200_pool_rebind_reset", "holo_b200_pool_store_unbound", "holo_b200_pool_pin_bytes", "holo_b200_pool_bind_fresh",
    "holo_b200_pool_bind_resident", "holo_b200_pool_retain", "holo_b200_pool_steal_transient", "holo_b200_pool_lease",
    "holo_b200_pool_release", "holo_b200_pool_resident", "holo_b200_pool_bindable_input", "holo_b200_pool_resolve",
    "holo_b200_pool_slot", "holo_b200_pool_write_slot", "holo_b200_pool_set_lazy_budget", "holo_b200_pool_pin_lazy",
    "holo_b200_pool_page_and_bind", "holo_b200_pool_stats",
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

    def init_tp(self, unique_id, rank, world, timeout_ms=None):
        """Join the tensor-parallel group. `timeout_ms`: host-side limit on the group's formation (a rank that never
        joins makes this raise `Init` instead of waiting for ever); None = HOLO_TP_INIT_TIMEOUT_MS or 120 s."""
        buf = (C.c_uint8 * 128).from_buffer_copy(bytes(unique_id))
        if timeout_ms is None:
            _check(lib.holo_b200_ctx_init_tp(self._h, buf, rank, world))
        else:
            _check(lib.holo_b200_ctx_init_tp_timeout(self._h, buf, rank, world, timeout_ms))

    @property
    def tp_transport(self):
        """0 = no tensor-parallel group, 1 = NCCL, 2 = the one-shot peer-memory kernel."""
        return int(lib.holo_b200_ctx_tp_transport(self._h))

    def emulate_all_reduce(self, workspace, partial_slots, out_slots, count, dtype, residual_slots=None, repeats=1,
                           withheld_rank=-1, poll_limit=0):
        """The peer-memory all-reduce with every rank emulated on this GPU (one cooperative launch). `withheld_rank`:
        that rank never sends, so the others' bounded polls run out after `poll_limit` polls and the call raises `Dispatch`."""
        w = len(partial_slots)
        arr = lambda slots: (C.c_void_p * w)(*[workspace.slot(s)[0] for s in slots])
        res = arr(residual_slots) if residual_slots is not None else None
        _check(lib.holo_b200_tp_emulate_all_reduce_ex(self._h, w, arr(partial_slots), res, arr(out_slots), count, dtype, repeats,
                                                      withheld_rank, poll_limit))

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


class PoolStats(C.Structure):
    _fields_ = [("owned_bytes", C.c_uint64), ("lazy_resident_bytes", C.c_uint64), ("pages_in", C.c_uint64),
                ("leased", C.c_uint32), ("transient", C.c_uint32), ("released", C.c_uint32)]


class WeightProviderStruct(C.Structure):
    """`HoloWeightProvider`: size / get_range callbacks over a host-side weight set."""
    SIZE_FN = C.CFUNCTYPE(C.c_int64, C.c_void_p, C.POINTER(C.c_uint8))
    RANGE_FN = C.CFUNCTYPE(C.c_void_p, C.c_void_p, C.POINTER(C.c_uint8), C.c_uint64, C.c_uint64)
    _fields_ = [("user", C.c_void_p), ("size", SIZE_FN), ("get_range", RANGE_FN)]


class WeightStore:
    """An in-memory weight set keyed by BLAKE3 fingerprint (the reference's `WeightStore` as a `WeightProvider`,
    crates/hologram-archive/src/weight.rs:53-78). Bodies are kept as numpy byte arrays (pin them for full speed)."""

    def __init__(self, bodies=None):
        self.bodies = {}
        self.calls = 0
        for fp, body in (bodies or {}).items():
            self.insert(fp, body)

        def size(_user, fp):
            b = self.bodies.get(bytes(fp[:32]))
            return -1 if b is None else b.nbytes

        def get_range(_user, fp, offset, length):
            b = self.bodies.get(bytes(fp[:32]))
            if b is None or offset + length > b.nbytes:
                return None
            self.calls += 1
            return b.ctypes.data + offset

        self.struct = WeightProviderStruct(None, WeightProviderStruct.SIZE_FN(size), WeightProviderStruct.RANGE_FN(get_range))

    def insert(self, fingerprint, body):
        self.bodies[bytes(fingerprint)] = np.frombuffer(bytes(body), dtype=np.uint8).copy()


class DevicePool:
    """The label-keyed buffer pool on its own (`BufferArena`, crates/hologram-exec/src/buffer.rs:273-952): slots are
    bindings to buffers held by 71-byte label. `backend=None` gives a pool over host memory (the same table logic
    with no device)."""

    def __init__(self, backend=None):
        h = C.c_void_p()
        _check(lib.holo_b200_pool_create(backend._h if backend is not None else None, C.byref(h)))
        self._h, self.backend = h, backend
        if backend is not None:
            backend._workspaces.add(self)

    def close(self):
        if getattr(self, "_h", None):
            lib.holo_b200_pool_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @staticmethod
    def _l(label):
        assert len(label) == 71
        return C.c_char_p(bytes(label))

    @staticmethod
    def _flag(rc):
        if rc < 0:
            _check(rc)
        return bool(rc)

    def rebind_reset(self, n_slots): _check(lib.holo_b200_pool_rebind_reset(self._h, n_slots))
    def store_unbound(self, label, data):
        a = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        _check(lib.holo_b200_pool_store_unbound(self._h, self._l(label), _host_ptr(a) if a.size else None, a.size))
    def pin_bytes(self, label, data):
        a = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        _check(lib.holo_b200_pool_pin_bytes(self._h, self._l(label), _host_ptr(a) if a.size else None, a.size))
    def bind_fresh(self, slot, nbytes): _check(lib.holo_b200_pool_bind_fresh(self._h, slot, nbytes))
    def bind_resident(self, slot, label): return self._flag(lib.holo_b200_pool_bind_resident(self._h, slot, self._l(label)))
    def retain(self, slot, label): _check(lib.holo_b200_pool_retain(self._h, slot, self._l(label)))
    def steal_transient(self, label, allowed_slots, out_slot):
        arr = (C.c_uint32 * max(1, len(allowed_slots)))(*allowed_slots)
        return self._flag(lib.holo_b200_pool_steal_transient(self._h, self._l(label), arr, len(allowed_slots), out_slot))
    def lease(self, label): return self._flag(lib.holo_b200_pool_lease(self._h, self._l(label)))
    def release(self, label): return self._flag(lib.holo_b200_pool_release(self._h, self._l(label)))
    def resident(self, label): return self._flag(lib.holo_b200_pool_resident(self._h, self._l(label)))
    def bindable_input(self, label): return self._flag(lib.holo_b200_pool_bindable_input(self._h, self._l(label)))

    def resolve(self, label):
        """The bytes of a resident label, or None."""
        n = C.c_uint64()
        if not self._flag(lib.holo_b200_pool_resolve(self._h, self._l(label), None, 0, C.byref(n))):
            return None
        out = np.empty(n.value, dtype=np.uint8)
        self._flag(lib.holo_b200_pool_resolve(self._h, self._l(label), _host_ptr(out) if out.size else None, out.size, C.byref(n)))
        return out

    def slot(self, slot):
        p, n = C.c_void_p(), C.c_uint64()
        if not self._flag(lib.holo_b200_pool_slot(self._h, slot, C.byref(p), C.byref(n))):
            return None
        return p.value, n.value

    def write_slot(self, slot, data):
        a = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        _check(lib.holo_b200_pool_write_slot(self._h, slot, _host_ptr(a), a.size))

    def set_lazy_budget(self, nbytes): _check(lib.holo_b200_pool_set_lazy_budget(self._h, nbytes))
    def pin_lazy(self, label, fingerprint, size):
        fp = (C.c_uint8 * 32).from_buffer_copy(bytes(fingerprint))
        _check(lib.holo_b200_pool_pin_lazy(self._h, self._l(label), fp, size))
    def page_and_bind(self, group, store):
        """group: [(slot, label)...]; store: a WeightStore."""
        slots = (C.c_uint32 * len(group))(*[g[0] for g in group])
        labels = np.frombuffer(b"".join(g[1] for g in group), dtype=np.uint8)
        return self._flag(lib.holo_b200_pool_page_and_bind(self._h, slots, _host_ptr(labels), len(group), C.byref(store.struct)))

    def stats(self):
        st = PoolStats()
        _check(lib.holo_b200_pool_stats(self._h, C.byref(st)))
        return st
