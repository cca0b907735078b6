"""The C-ABI library loads and exports everything include/hologram_b200.h declares; the
ctypes mirror has the header's struct layout (no GPU, no compute calls)."""
import ctypes
import os
import re
import subprocess
import tempfile

import hologram_b200 as hb
from hologram_b200 import kernel_call as kc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "hologram_b200.h")


def declared_functions():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(holo_b200_\w+)\s*\(", src)))


def test_every_declared_symbol_is_exported():
    lib = ctypes.CDLL(hb.LIB_PATH)
    names = declared_functions()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
    assert set(hb.EXPORTED_SYMBOLS) <= set(names)


def test_struct_layout_matches_the_header():
    probe = r'''
    #include <stdio.h>
    #include <stddef.h>
    #include "hologram_b200.h"
    int main(void) {
        printf("%zu %zu %zu %zu %zu %zu %zu %zu %zu\n", sizeof(HoloBufferRef), sizeof(HoloUnaryCall), sizeof(HoloMatMulCall),
               sizeof(HoloMatMulAddCall), sizeof(HoloNormCall), sizeof(HoloDecodeAttentionValidQ8Call),
               sizeof(HoloKernelCall), offsetof(HoloKernelCall, u), sizeof(HoloHostSlot));
        return 0;
    }'''
    with tempfile.TemporaryDirectory() as d:
        c = os.path.join(d, "probe.c")
        open(c, "w").write(probe)
        exe = os.path.join(d, "probe")
        subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), c, "-o", exe])
        got = [int(v) for v in subprocess.check_output([exe]).split()]
    want = [ctypes.sizeof(kc.BufferRef), ctypes.sizeof(kc.UnaryCall), ctypes.sizeof(kc.MatMulCall),
            ctypes.sizeof(kc.MatMulAddCall), ctypes.sizeof(kc.NormCall), ctypes.sizeof(kc.DecodeAttentionValidQ8Call),
            ctypes.sizeof(kc.KernelCall), kc.KernelCall.u.offset, ctypes.sizeof(kc.HostSlot)]
    assert got == want


def test_no_device_is_a_loud_init_error():
    import torch
    if torch.cuda.is_available():
        return
    try:
        hb.B200Backend(0)
    except hb.BackendError as e:
        assert e.variant == "Init"
    else:
        raise AssertionError("context creation must fail without a GPU")


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "hologram_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower() or f == "NOTES", f"{f} mentions the oracle"
