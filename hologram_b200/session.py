"""`InferenceSession` over the C ABI: load a `.holo` image onto the device and walk it
(crates/hologram-exec/src/session.rs `InferenceSession::{load, execute}`)."""
import ctypes as C

import numpy as np

from . import kernel_call as kc
from .backend import DeviceWorkspace, WeightStore, _check, _host_ptr, lib

vp, u32, u64, i32 = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int32
for _name, _res, _args in [
    ("holo_b200_session_load", i32, [vp, vp, u64, i32, C.POINTER(vp)]),
    ("holo_b200_session_destroy", None, [vp]),
    ("holo_b200_session_workspace", vp, [vp]),
    ("holo_b200_session_info", i32, [vp] + [C.POINTER(u32)] * 5 + [C.POINTER(u64)]),
    ("holo_b200_session_nodes", i32, [vp, C.POINTER(u32), C.POINTER(u32)]),
    ("holo_b200_session_port", i32, [vp, i32, u32, C.c_char_p, u32, C.POINTER(u32), C.POINTER(u64), C.POINTER(C.c_uint8)]),
    ("holo_b200_session_call", i32, [vp, u32, C.POINTER(kc.KernelCall)]),
    ("holo_b200_session_execute", i32, [vp]),
    ("holo_b200_session_capture", i32, [vp]),
    ("holo_b200_archive_check", i32, [vp, u64, i32] + [C.POINTER(u32)] * 4),
    ("holo_b200_session_execute_addressed", i32, [vp, vp, u32, vp, u32, vp]),
    ("holo_b200_label_bytes", i32, [vp, u64, vp]),
    ("holo_b200_label_derive", i32, [C.c_uint16, vp, u32, vp, u32, vp]),
    ("holo_b200_op_signature", i32, [C.POINTER(kc.KernelCall), C.POINTER(C.c_uint16), vp, C.POINTER(u32)]),
    ("holo_b200_label_derive_boundary", i32, [C.c_uint16, vp, u32, vp, u32, vp]),
    ("holo_b200_session_intern_input", i32, [vp, vp, u64, vp]),
    ("holo_b200_session_resolve", i32, [vp, vp, vp, u64, C.POINTER(u64), C.POINTER(i32)]),
    ("holo_b200_session_retain_label", i32, [vp, vp, C.POINTER(i32)]),
    ("holo_b200_session_release_label", i32, [vp, vp, C.POINTER(i32)]),
    ("holo_b200_session_leased_count", u32, [vp]),
    ("holo_b200_session_load_paged", i32, [vp, vp, u64, i32, vp, u64, C.POINTER(vp)]),
    ("holo_b200_session_tier_report", i32, [vp, i32, vp]),
]:
    _fn = getattr(lib, _name)
    _fn.restype, _fn.argtypes = _res, _args

SESSION_SYMBOLS = ["holo_b200_session_load", "holo_b200_session_destroy", "holo_b200_session_workspace",
                   "holo_b200_session_info", "holo_b200_session_nodes", "holo_b200_session_port", "holo_b200_session_call",
                   "holo_b200_session_execute", "holo_b200_session_capture", "holo_b200_archive_check",
                   "holo_b200_session_execute_addressed", "holo_b200_label_bytes", "holo_b200_label_derive",
                   "holo_b200_op_signature", "holo_b200_label_derive_boundary", "holo_b200_session_intern_input",
                   "holo_b200_session_resolve", "holo_b200_session_retain_label", "holo_b200_session_release_label",
                   "holo_b200_session_leased_count", "holo_b200_session_load_paged", "holo_b200_session_tier_report"]

LABEL_BYTES = 71


class AddressedStats(C.Structure):
    _fields_ = [("dispatched", u32), ("skipped", u32), ("memo_hit", u32), ("pool_bytes", u64), ("moved", u32), ("paged_in", u32)]


class TierReport(C.Structure):
    """`TierReport` (crates/hologram-exec/src/coherence.rs:78-93)."""
    _fields_ = [("cpu_l1_calls", u32), ("cpu_l2_calls", u32), ("cpu_main_calls", u32), ("device_calls", u32),
                ("total_migration_slots", u32), ("levels_with_migrations", u32)]


TIER_COMPILED, TIER_FORCE_ALL_CPU, TIER_FORCE_ALL_DEVICE = 0, 1, 2
SESSION_LABEL_RESIDUAL = 4


def label_bytes(data):
    """`address_bytes` (crates/hologram-archive/src/address.rs:83-86): the 71-byte label of a leaf value."""
    a = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
    out = np.empty(LABEL_BYTES, dtype=np.uint8)
    _check(lib.holo_b200_label_bytes(_host_ptr(a) if a.size else None, a.size, _host_ptr(out)))
    return out.tobytes()


def label_derive(opcode, params, labels):
    """`derive_label` (address.rs:108-116) over an opcode, parameter bytes and ordered operand labels."""
    pr = np.frombuffer(bytes(params), dtype=np.uint8)
    lb = np.frombuffer(b"".join(labels), dtype=np.uint8)
    out = np.empty(LABEL_BYTES, dtype=np.uint8)
    _check(lib.holo_b200_label_derive(opcode, _host_ptr(pr) if pr.size else None, pr.size, _host_ptr(lb) if lb.size else None,
                                      len(labels), _host_ptr(out)))
    return out.tobytes()


def label_derive_boundary(opcode, params, labels):
    """`derive_label_boundary` (address.rs:197-221): the label a graph output is retained and reported under."""
    pr = np.frombuffer(bytes(params), dtype=np.uint8)
    lb = np.frombuffer(b"".join(labels), dtype=np.uint8)
    out = np.empty(LABEL_BYTES, dtype=np.uint8)
    _check(lib.holo_b200_label_derive_boundary(opcode, _host_ptr(pr) if pr.size else None, pr.size, _host_ptr(lb) if lb.size else None,
                                               len(labels), _host_ptr(out)))
    return out.tobytes()


def op_signature(call):
    """`KernelCall::op_signature` (kernel_call.rs:1321-1516): (opcode, parameter bytes)."""
    op, n = C.c_uint16(), u32()
    buf = np.zeros(64, dtype=np.uint8)
    _check(lib.holo_b200_op_signature(C.byref(call), C.byref(op), _host_ptr(buf), C.byref(n)))
    return op.value, buf[:n.value].tobytes()


def archive_check(archive_bytes, verify=True):
    """Host-only parse of a `.holo` image; returns (calls, inputs, outputs, constants) counts."""
    buf = np.frombuffer(archive_bytes, dtype=np.uint8)
    vals = [u32() for _ in range(4)]
    _check(lib.holo_b200_archive_check(_host_ptr(buf), buf.size, 1 if verify else 0, *[C.byref(v) for v in vals]))
    return tuple(v.value for v in vals)


class Port:
    def __init__(self, name, slot, element_count, dtype):
        self.name, self.slot, self.element_count, self.dtype = name, slot, element_count, dtype

    @property
    def nbytes(self):
        return self.element_count * {0: 1, 1: 1, 2: 1, 3: 8, 4: 4, 5: 8, 6: 2, 7: 2, 8: 4, 9: 8}[self.dtype]


class InferenceSession:
    def __init__(self, backend, archive_bytes, verify=True, addressed=False, label_residual=False, weight_store=None, budget=0):
        """`weight_store` (a WeightStore) makes this `load_paged` (session.rs:417): by-reference constants page in from it
        within `budget` resident bytes (0 = never evict)."""
        h = vp()
        buf = np.frombuffer(archive_bytes, dtype=np.uint8)
        flags = (1 if verify else 0) | (2 if addressed else 0) | (SESSION_LABEL_RESIDUAL if label_residual else 0)
        if weight_store is not None:
            self._store = weight_store      # the provider must outlive the session
            addressed = True
            _check(lib.holo_b200_session_load_paged(backend._h, _host_ptr(buf), buf.size, flags, C.byref(weight_store.struct), budget, C.byref(h)))
        else:
            _check(lib.holo_b200_session_load(backend._h, _host_ptr(buf), buf.size, flags, C.byref(h)))
        self.addressed = addressed
        self._h = h
        self.backend = backend
        backend._workspaces.add(self)
        ws = DeviceWorkspace.__new__(DeviceWorkspace)
        ws._h, ws.backend, ws.n_slots = vp(lib.holo_b200_session_workspace(h)), backend, None
        ws.close = lambda: None          # owned by the session
        self.workspace = ws
        vals = [u32() for _ in range(5)]
        dev = u64()
        _check(lib.holo_b200_session_info(h, *[C.byref(v) for v in vals], C.byref(dev)))
        self.n_calls, self.fused_count, self.moved_in_place, n_in, n_out = (v.value for v in vals)
        self.device_bytes = dev.value
        nn, nm = u32(), u32()
        _check(lib.holo_b200_session_nodes(h, C.byref(nn), C.byref(nm)))
        self.n_nodes, self.merged_calls = nn.value, nm.value
        self.inputs = [self._port(0, i) for i in range(n_in)]
        self.outputs = [self._port(1, i) for i in range(n_out)]
        self._by_name = {p.name: p for p in self.inputs + self.outputs}

    def _port(self, is_output, i):
        name = C.create_string_buffer(256)
        slot, cnt, dt = u32(), u64(), C.c_uint8()
        _check(lib.holo_b200_session_port(self._h, is_output, i, name, 256, C.byref(slot), C.byref(cnt), C.byref(dt)))
        return Port(name.value.decode(), slot.value, cnt.value, dt.value)

    def execute_addressed(self, input_labels):
        """`execute_addressed` (session.rs:942-984): the inputs have been written; `input_labels` are their
        71-byte labels in port order. Returns (output labels, AddressedStats)."""
        assert len(input_labels) == len(self.inputs)
        ins = np.frombuffer(b"".join(input_labels), dtype=np.uint8)
        outs = np.zeros(LABEL_BYTES * len(self.outputs), dtype=np.uint8)
        st = AddressedStats()
        _check(lib.holo_b200_session_execute_addressed(self._h, _host_ptr(ins), len(self.inputs), _host_ptr(outs),
                                                       len(self.outputs), C.byref(st)))
        raw = outs.tobytes()
        return [raw[i * LABEL_BYTES:(i + 1) * LABEL_BYTES] for i in range(len(self.outputs))], st

    def intern_input(self, data):
        """`intern_input` (session.rs:1018-1022): store host bytes in the pool under the label of their content."""
        a = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        out = np.empty(LABEL_BYTES, dtype=np.uint8)
        _check(lib.holo_b200_session_intern_input(self._h, _host_ptr(a) if a.size else None, a.size, _host_ptr(out)))
        return out.tobytes()

    def resolve(self, label, dtype=np.uint8):
        """`resolve` (session.rs:1027-1029): the bytes of a resident label, or None."""
        n, here = u64(), i32()
        lb = C.c_char_p(bytes(label))
        _check(lib.holo_b200_session_resolve(self._h, lb, None, 0, C.byref(n), C.byref(here)))
        if not here.value:
            return None
        out = np.empty(n.value, dtype=np.uint8)
        _check(lib.holo_b200_session_resolve(self._h, lb, _host_ptr(out) if out.size else None, out.size, C.byref(n), C.byref(here)))
        return out.view(dtype)

    def retain_label(self, label):
        ok = i32()
        _check(lib.holo_b200_session_retain_label(self._h, C.c_char_p(bytes(label)), C.byref(ok)))
        return bool(ok.value)

    def release_label(self, label):
        ok = i32()
        _check(lib.holo_b200_session_release_label(self._h, C.c_char_p(bytes(label)), C.byref(ok)))
        return bool(ok.value)

    @property
    def leased_count(self):
        return int(lib.holo_b200_session_leased_count(self._h))

    def tier_report(self, policy=TIER_FORCE_ALL_DEVICE):
        """`tier_report` (session.rs:797) under a routing policy; this backend executes under TIER_FORCE_ALL_DEVICE."""
        rep = TierReport()
        _check(lib.holo_b200_session_tier_report(self._h, policy, C.byref(rep)))
        return rep

    def close(self):
        if getattr(self, "_h", None):
            lib.holo_b200_session_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def port(self, name):
        return self._by_name[name]

    def call(self, index):
        out = kc.KernelCall()
        _check(lib.holo_b200_session_call(self._h, index, C.byref(out)))
        return out

    def write(self, name, array):
        self.workspace.write(kc.rb(self.port(name).slot), array)

    def read(self, name, dtype=np.uint8):
        p = self.port(name)
        return self.workspace.read(kc.rb(p.slot), p.nbytes, dtype)

    def device_ptr(self, name):
        return self.workspace.slot(self.port(name).slot)

    def execute(self):
        _check(lib.holo_b200_session_execute(self._h))

    def capture(self):
        _check(lib.holo_b200_session_capture(self._h))
