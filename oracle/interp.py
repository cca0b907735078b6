"""CPU interpreter of a KernelCall list over numpy byte slots, built on the oracle kernels.

TEST INFRASTRUCTURE ONLY (see oracle/hologram_oracle.c). It plays the role the reference's
CpuBackend + slot-vector TestWorkspace play in crates/hologram-compute/tests: each call reads
and writes `slots[slot]` (numpy uint8 arrays). `all_reduce(array_f32) -> array_f32` supplies
the tensor-parallel sum when the list contains AllReduce calls.
"""
import numpy as np

from hologram_b200 import kernel_call as kc
from . import oracle as orc

_NP = {kc.DTYPE_F32: np.float32, kc.DTYPE_BF16: np.uint16, kc.DTYPE_F16: np.uint16, kc.DTYPE_I8: np.int8,
       kc.DTYPE_I32: np.int32, kc.DTYPE_I64: np.int64, kc.DTYPE_U8: np.uint8}
_LUT = {kc.K_SIGMOID: kc.LUT_SIGMOID, kc.K_TANH: kc.LUT_TANH, kc.K_GELU: kc.LUT_GELU, kc.K_SILU: kc.LUT_SILU,
        kc.K_EXP: kc.LUT_EXP, kc.K_ERF: kc.LUT_ERF}

_REDUCE = {kc.K_REDUCE_SUM: (0, False), kc.K_REDUCE_MEAN: (0, True), kc.K_REDUCE_PROD: (1, False), kc.K_REDUCE_MIN: (2, False),
           kc.K_REDUCE_MAX: (3, False)}


def _get(slots, ref, nbytes, dtype):
    buf = slots[ref.slot]
    assert ref.offset + nbytes <= buf.size, f"slot {ref.slot} too short"
    return buf[ref.offset:ref.offset + nbytes].view(_NP[dtype])


def _put(slots, ref, arr):
    raw = np.ascontiguousarray(arr).view(np.uint8).reshape(-1)
    if ref.slot not in slots or slots[ref.slot].size < ref.offset + raw.size:
        new = np.zeros(ref.offset + raw.size, dtype=np.uint8)
        if ref.slot in slots:
            new[:slots[ref.slot].size] = slots[ref.slot]
        slots[ref.slot] = new
    slots[ref.slot][ref.offset:ref.offset + raw.size] = raw


def run(calls, slots, all_reduce=None):
    es = lambda dt: np.dtype(_NP[dt]).itemsize
    for call in calls:
        k, u = call.kind, call.u
        if k in _LUT:
            c = u.unary
            _put(slots, c.output, orc.unary_lut(_LUT[k], c.dtype, _get(slots, c.input, c.element_count * 2, c.dtype)))
        elif k in (kc.K_ADD, kc.K_MUL):
            c = u.binary
            n = c.element_count * es(c.dtype)
            _put(slots, c.output, orc.binary(0 if k == kc.K_ADD else 1, _get(slots, c.a, n, c.dtype), _get(slots, c.b, n, c.dtype), c.dtype))
        elif k in (kc.K_MATMUL, kc.K_MATMUL_ACTIVATION, kc.K_MATMUL_ADD):
            mm = u.matmul
            a = _get(slots, mm.a, mm.m * mm.k * 2, mm.dtype)
            b = _get(slots, mm.b, mm.k * mm.n * 2, mm.dtype)
            act = u.matmul_activation.act if k == kc.K_MATMUL_ACTIVATION else 0
            res = _get(slots, u.matmul_add.residual, mm.m * mm.n * 2, mm.dtype) if k == kc.K_MATMUL_ADD else None
            _put(slots, mm.output, orc.matmul(a, b, mm.m, mm.k, mm.n, mm.dtype, act=act, residual=res))
        elif k == kc.K_RMS_NORM:
            c = u.norm
            x = _get(slots, c.x, c.batch * c.feature * es(c.dtype), c.dtype)
            g = _get(slots, c.gamma, c.feature * es(c.dtype), c.dtype) if c.gamma.slot != kc.NO_SLOT else None
            _put(slots, c.output, orc.rms_norm(x, g, c.batch, c.feature, c.epsilon_bits, c.dtype))
        elif k == kc.K_LAYER_NORM:
            c = u.norm
            row = c.feature * es(c.dtype)
            x = _get(slots, c.x, c.batch * row, c.dtype)
            g = _get(slots, c.gamma, row, c.dtype) if c.gamma.slot != kc.NO_SLOT else None
            b = _get(slots, c.beta, row, c.dtype) if c.beta.slot != kc.NO_SLOT else None
            _put(slots, c.output, orc.layer_norm(x, g, b, c.batch, c.feature, c.epsilon_bits, c.dtype))
        elif k == kc.K_SOFTMAX:
            c = u.softmax
            x = _get(slots, c.input, c.batch * c.feature * es(c.dtype), c.dtype)
            _put(slots, c.output, orc.softmax(x, c.batch, c.feature, c.dtype))
        elif k in _REDUCE:
            c = u.reduce
            dims = [c.dims[i] for i in range(c.rank)]
            kind, mean = _REDUCE[k]
            _put(slots, c.output, orc.reduce(_get(slots, c.input, c.element_count * es(c.dtype), c.dtype), dims, c.axes_mask, kind, mean, c.dtype))
        elif k in (kc.K_EXPAND, kc.K_BROADCAST_BINARY):
            c = u.expand if k == kc.K_EXPAND else u.broadcast_binary
            ind, outd = [c.in_dims[i] for i in range(c.rank)], [c.out_dims[i] for i in range(c.rank)]
            small = _get(slots, c.input if k == kc.K_EXPAND else c.small, int(np.prod(ind)) * es(c.dtype), c.dtype)
            if k == kc.K_EXPAND:
                _put(slots, c.output, orc.broadcast(small, None, ind, outd, es(c.dtype)))
            else:
                other = _get(slots, c.other, int(np.prod(outd)) * es(c.dtype), c.dtype)
                _put(slots, c.output, orc.broadcast(small, other, ind, outd, es(c.dtype), c.op, bool(c.small_is_lhs), c.dtype))
        elif k in kc.EXACT_UNARY:
            c = u.unary
            _put(slots, c.output, orc.elementwise(k, _get(slots, c.input, c.element_count * es(c.dtype), c.dtype), None, c.dtype))
        elif k in kc.EXACT_BINARY:
            c = u.binary
            n = c.element_count * es(c.dtype)
            _put(slots, c.output, orc.elementwise(k, _get(slots, c.a, n, c.dtype), _get(slots, c.b, n, c.dtype), c.dtype))
        elif k == kc.K_WHERE:
            c = u.where
            n = c.element_count * es(c.dtype)
            _put(slots, c.output, orc.where(_get(slots, c.cond, c.element_count, kc.DTYPE_U8), _get(slots, c.a, n, c.dtype), _get(slots, c.b, n, c.dtype), c.dtype))
        elif k == kc.K_ATTENTION:
            c = u.attention
            hkv = c.kv_heads or c.heads
            q = _get(slots, c.q, c.batch * c.heads * c.seq * c.head_dim * es(c.dtype), c.dtype)
            kk = _get(slots, c.k, c.batch * hkv * c.seq * c.head_dim * es(c.dtype), c.dtype)
            v = _get(slots, c.v, c.batch * hkv * c.seq * c.head_dim * es(c.dtype), c.dtype)
            _put(slots, c.output, orc.attention(q, kk, v, c.batch, c.heads, c.kv_heads, c.seq, c.head_dim, bool(c.causal), c.scale_bits, c.dtype))
        elif k == kc.K_CONCAT:
            c = u.binary
            a = slots[c.a.slot][c.a.offset:c.a.offset + c.a.length] if c.a.length else slots[c.a.slot][c.a.offset:]
            b = slots[c.b.slot][c.b.offset:c.b.offset + c.b.length] if c.b.length else slots[c.b.slot][c.b.offset:]
            _put(slots, c.output, np.concatenate([a, b]))
        elif k == kc.K_ADD_RMS_NORM:
            c = u.norm
            n = c.batch * c.feature * es(c.dtype)
            x = _get(slots, c.x, n, c.dtype)
            r = _get(slots, c.residual, n, c.dtype) if c.residual.slot != kc.NO_SLOT else None
            g = _get(slots, c.gamma, c.feature * es(c.dtype), c.dtype) if c.gamma.slot != kc.NO_SLOT else None
            _put(slots, c.output, orc.add_rms_norm(x, r, g, c.batch, c.feature, c.epsilon_bits, c.dtype))
        elif k == kc.K_TRANSPOSE:
            c = u.transpose
            dims = [c.dims[i] for i in range(c.rank)]
            total = int(np.prod(dims)) * es(c.dtype)
            _put(slots, c.output, orc.transpose(_get(slots, c.input, total, kc.DTYPE_U8), dims, [c.perm[i] for i in range(c.rank)], es(c.dtype)))
        elif k == kc.K_ROTARY:
            c = u.rope
            n = c.element_count * es(c.dtype)
            _put(slots, c.output, orc.rope(_get(slots, c.x, n, c.dtype), _get(slots, c.cos, n, c.dtype), _get(slots, c.sin, n, c.dtype), c.head_dim, c.dtype))
        elif k == kc.K_GATHER:
            c = u.gather
            data = _get(slots, c.data, c.outer * c.axis_dim * c.inner * es(c.dtype), c.dtype)
            idx = _get(slots, c.indices, c.num_indices * es(c.idx_dtype), c.idx_dtype)
            rc, out = orc.gather(data, idx, c.outer, c.axis_dim, c.inner, c.dtype)
            assert rc == 0
            _put(slots, c.output, out)
        elif k == kc.K_QUANTIZE_ROWS_I8:
            c = u.quantize_rows_i8
            x = _get(slots, c.input, c.rows * c.row_len * es(c.dtype), c.dtype)
            codes, scales = orc.quantize_rows_i8(x, c.dtype, c.rows, c.row_len)
            _put(slots, c.codes, codes)
            _put(slots, c.scales, scales)
        elif k == kc.K_DECODE_ATTENTION_VALID_Q8:
            c = u.decode_attention_valid_q8
            hkv = c.kv_heads or c.heads
            prow, nrow = c.batch * hkv * c.past_len, c.batch * hkv * c.new_len
            q = _get(slots, c.q, c.batch * c.heads * c.q_rows * c.head_dim * es(c.dtype), c.dtype)
            g8 = lambda r, n: _get(slots, r, n * c.head_dim, kc.DTYPE_I8)
            gs = lambda r, n: _get(slots, r, n * 4, kc.DTYPE_F32)
            vl = int(_get(slots, c.valid_len, 4, kc.DTYPE_I32).view(np.uint32)[0])
            rc, out = orc.decode_attention_valid_q8(q, c.dtype, g8(c.k_past, prow), gs(c.k_past_scales, prow), g8(c.v_past, prow),
                                                    gs(c.v_past_scales, prow), g8(c.k_new, nrow), gs(c.k_new_scales, nrow),
                                                    g8(c.v_new, nrow), gs(c.v_new_scales, nrow), vl, c.batch, c.heads, c.kv_heads,
                                                    c.q_rows, c.past_len, c.new_len, c.head_dim, c.scale_bits)
            assert rc == 0
            _put(slots, c.output, out)
        elif k == kc.K_KV_CACHE_WRITE:
            c = u.kv_cache_write
            total = c.planes * c.bucket_rows * c.row_bytes
            cache = _get(slots, c.cache, total, kc.DTYPE_U8)
            new = _get(slots, c.new, c.planes * c.new_rows * c.row_bytes, kc.DTYPE_U8)
            pos = int(_get(slots, c.pos, 4, kc.DTYPE_I32).view(np.uint32)[0])
            rc, out = orc.kv_cache_write(cache, new, pos, c.planes, c.bucket_rows, c.new_rows, c.row_bytes)
            assert rc == 0
            _put(slots, c.output, out)
        elif k == kc.K_ALL_REDUCE:
            c = u.all_reduce
            assert c.dtype == kc.DTYPE_BF16
            part = orc.bf16_to_f32(_get(slots, c.buffer, c.element_count * 2, c.dtype))
            total = all_reduce(part) if all_reduce else part
            _put(slots, c.buffer, orc.f32_to_bf16_rne(total))
        else:
            raise NotImplementedError(f"oracle interpreter: KernelCall kind {k}")
    return slots
