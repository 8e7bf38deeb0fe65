"""ctypes/numpy doorway onto the CPU oracle (test infrastructure only).

`liboracle.so` is this repository's restatement of the RAFTInfer CPU reference
operators (oracle/oracle.cpp); `_ref/libraftinfer_ref.so` is the reference's own
cpp/reference library compiled unmodified (present when it was built where the
reference checkout exists).  Only tests, the smoke check and the benchmark's
CPU-baseline leg may import this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_u16p = np.ctypeslib.ndpointer(dtype=np.uint16, flags="C_CONTIGUOUS")
_f64p = np.ctypeslib.ndpointer(dtype=np.float64, flags="C_CONTIGUOUS")
_sz = C.c_size_t


def build(force: bool = False) -> None:
    """Compile the oracle (and the reference library when its checkout is present)."""
    need = force or not os.path.exists(os.path.join(_HERE, "liboracle.so"))
    src = os.path.join(_HERE, "oracle.cpp")
    lib = os.path.join(_HERE, "liboracle.so")
    if not need and os.path.getmtime(src) > os.path.getmtime(lib):
        need = True
    if need or not os.path.exists(os.path.join(_HERE, "_ref", "libraftinfer_ref.so")):
        subprocess.run(["make", "-C", _HERE, "-s"] + (["-B"] if force else []), check=True)


_lib = None
_ref = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(os.path.join(_HERE, "liboracle.so"))
        L.orc_round_to_bf16.argtypes = [_f32p, _f32p, _sz]
        L.orc_float_to_bf16_bits.argtypes = [_f32p, _u16p, _sz]
        L.orc_bf16_bits_to_float.argtypes = [_u16p, _f32p, _sz]
        L.orc_attention_core_f32.argtypes = [_f32p, _f32p, _f32p, _f32p, _f32p] + [_sz] * 5 + [C.c_int]
        L.orc_attention_core_cache.argtypes = [_f32p, _f32p, _f32p, _u16p] + [_sz] * 6 + [C.c_int]
        L.orc_decode_partials.argtypes = [_f32p, _u16p, _f32p, _f32p, _f32p] + [_sz] * 6 + [C.c_int]
        L.orc_full_attention_layer.argtypes = [_f32p] * 5 + [_sz] * 7 + [C.c_float, C.c_float, C.c_int]
        L.orc_qk_norm_rope.argtypes = [_f32p, _f32p] + [_sz] * 5 + [C.c_float, C.c_float]
        L.orc_gdn_core.argtypes = [_f32p] * 7 + [_sz] * 5 + [C.c_int]
        L.orc_gated_delta_layer.argtypes = [_f32p] * 8 + [_sz] * 7 + [C.c_float, C.c_int]
        L.orc_compare.argtypes = [_f32p, _f32p, _sz, C.c_double, _f64p]
        for name in ("orc_round_to_bf16", "orc_float_to_bf16_bits", "orc_bf16_bits_to_float",
                     "orc_attention_core_f32", "orc_attention_core_cache", "orc_decode_partials",
                     "orc_full_attention_layer", "orc_qk_norm_rope", "orc_gdn_core",
                     "orc_gated_delta_layer", "orc_compare"):
            getattr(L, name).restype = None
        _lib = L
    return _lib


def ref():
    """The unmodified reference library, or None when it was never built."""
    global _ref
    if _ref is None:
        path = os.path.join(_HERE, "_ref", "libraftinfer_ref.so")
        if not os.path.exists(path):
            return None
        R = C.CDLL(path)
        R.ref_full_attention.argtypes = [_f32p] * 5 + [_sz] * 7 + [C.c_float, C.c_float]
        R.ref_full_attention.restype = C.c_int
        R.ref_gated_delta.argtypes = [_f32p] * 8 + [_sz] * 7 + [C.c_float, C.c_int]
        R.ref_gated_delta.restype = C.c_int
        R.ref_compare.argtypes = [_f32p, _f32p, _sz, C.c_double, _f64p]
        R.ref_compare.restype = C.c_int
        _ref = R
    return _ref


def _f(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def cpu_threads() -> int:
    return max(1, len(os.sched_getaffinity(0)))


# ---- bf16 codec -----------------------------------------------------------------------------
def round_bf16(a):
    a = _f(a)
    out = np.empty_like(a)
    lib().orc_round_to_bf16(a.reshape(-1), out.reshape(-1), a.size)
    return out


def to_bf16_bits(a):
    a = _f(a)
    out = np.empty(a.shape, dtype=np.uint16)
    lib().orc_float_to_bf16_bits(a.reshape(-1), out.reshape(-1), a.size)
    return out


def from_bf16_bits(a):
    a = np.ascontiguousarray(a, dtype=np.uint16)
    out = np.empty(a.shape, dtype=np.float32)
    lib().orc_bf16_bits_to_float(a.reshape(-1), out.reshape(-1), a.size)
    return out


# ---- attention ------------------------------------------------------------------------------
def attention_core(q, k, v, gate, past=0, threads=None):
    """q, gate [T][Hq][D]; k, v [past+T][Hkv][D] float -> out [T][Hq][D]."""
    q, k, v, gate = _f(q), _f(k), _f(v), _f(gate)
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    assert k.shape[0] == past + T and v.shape == k.shape
    out = np.empty_like(q)
    lib().orc_attention_core_f32(q, k, v, gate, out, T, Hq, Hkv, D, past, threads or cpu_threads())
    return out


def attention_core_cache(q, gate, cache_bits, max_ctx, past, threads=None):
    """Keys/values from the BF16 head-major cache [2][Hkv][max_ctx][D] (uint16 bit patterns)."""
    q, gate = _f(q), _f(gate)
    T, Hq, D = q.shape
    cache_bits = np.ascontiguousarray(cache_bits, dtype=np.uint16)
    Hkv = cache_bits.size // (2 * max_ctx * D)
    out = np.empty_like(q)
    lib().orc_attention_core_cache(q, gate, out, cache_bits.reshape(-1), T, Hq, Hkv, D, max_ctx, past,
                                   threads or cpu_threads())
    return out


def decode_partials(q, cache_bits, max_ctx, ctx, part_tokens, threads=None):
    q = _f(q)
    Hq, D = q.shape
    cache_bits = np.ascontiguousarray(cache_bits, dtype=np.uint16)
    Hkv = cache_bits.size // (2 * max_ctx * D)
    max_parts = -(-max_ctx // part_tokens)
    pmax = np.full(Hq * max_parts, np.nan, dtype=np.float32)
    psum = np.full(Hq * max_parts, np.nan, dtype=np.float32)
    pval = np.full(Hq * max_parts * D, np.nan, dtype=np.float32)
    lib().orc_decode_partials(q, cache_bits.reshape(-1), pmax, psum, pval, Hq, Hkv, D, max_ctx, ctx,
                              part_tokens, threads or cpu_threads())
    return pmax.reshape(Hq, max_parts), psum.reshape(Hq, max_parts), pval.reshape(Hq, max_parts, D)


def full_attention_layer(inp, q_norm_w, k_norm_w, out_w, *, tokens, hidden, q_heads, kv_heads, head_dim,
                         rotary, pos_offset, rope_base, eps, threads=None):
    out = np.empty(tokens * hidden, dtype=np.float32)
    lib().orc_full_attention_layer(_f(inp).reshape(-1), out, _f(q_norm_w), _f(k_norm_w), _f(out_w).reshape(-1),
                                   tokens, hidden, q_heads, kv_heads, head_dim, rotary, pos_offset,
                                   rope_base, eps, threads or cpu_threads())
    return out.reshape(tokens, hidden)


def ref_full_attention_layer(inp, q_norm_w, k_norm_w, out_w, *, tokens, hidden, q_heads, kv_heads, head_dim,
                             rotary, pos_offset, rope_base, eps):
    out = np.empty(tokens * hidden, dtype=np.float32)
    rc = ref().ref_full_attention(_f(inp).reshape(-1), out, _f(q_norm_w), _f(k_norm_w), _f(out_w).reshape(-1),
                                  tokens, hidden, q_heads, kv_heads, head_dim, rotary, pos_offset, rope_base, eps)
    if rc != 0:
        raise ValueError("reference rejected the arguments")
    return out.reshape(tokens, hidden)


def qk_norm_rope(x, norm_w, rotary, pos_offset, rope_base, eps):
    x = _f(x).copy()
    T, H, D = x.shape
    lib().orc_qk_norm_rope(x, _f(norm_w), T, H, D, rotary, pos_offset, rope_base, eps)
    return x


# ---- gated delta ----------------------------------------------------------------------------
def gdn_core(q, k, v, beta, decay, state, threads=None):
    """q,k [T][Hk][dk] (q pre-scaled, k normalised), v [T][Hv][dv], beta/decay [T][Hv].
    Returns (out [T][Hv][dv], new_state [Hv][dk][dv])."""
    q, k, v, beta, decay = _f(q), _f(k), _f(v), _f(beta), _f(decay)
    T, Hk, dk = q.shape
    Hv, dv = v.shape[1], v.shape[2]
    st = _f(state).copy()
    out = np.empty((T, Hv, dv), dtype=np.float32)
    lib().orc_gdn_core(q, k, v, beta, decay, st.reshape(-1), out.reshape(-1), T, Hk, Hv, dk, dv,
                       threads or cpu_threads())
    return out, st


def _delta_call(fn, inp, conv_w, rec_a, dt_bias, out_norm_w, conv_state, rec_state, shape, last):
    T, hidden, Hk, Hv, dk, dv, W, eps = shape
    out = np.empty(T * hidden, dtype=np.float32)
    cs = _f(conv_state).copy().reshape(-1)
    rs = _f(rec_state).copy().reshape(-1)
    if cs.size == 0:
        cs = np.zeros(1, dtype=np.float32)
    rc = fn(_f(inp).reshape(-1), out, _f(conv_w).reshape(-1), _f(rec_a), _f(dt_bias), _f(out_norm_w), cs, rs,
            T, hidden, Hk, Hv, dk, dv, W, eps, last)
    if rc not in (None, 0):
        raise ValueError("reference rejected the arguments")
    return out.reshape(T, hidden), cs, rs


def gated_delta_layer(inp, conv_w, rec_a, dt_bias, out_norm_w, conv_state, rec_state, shape, threads=None):
    """shape = (tokens, hidden, Hk, Hv, dk, dv, conv_width, eps). Returns (out, conv_state, rec_state)."""
    return _delta_call(lib().orc_gated_delta_layer, inp, conv_w, rec_a, dt_bias, out_norm_w, conv_state,
                       rec_state, shape, threads or cpu_threads())


def ref_gated_delta_layer(inp, conv_w, rec_a, dt_bias, out_norm_w, conv_state, rec_state, shape, per_step=False):
    return _delta_call(ref().ref_gated_delta, inp, conv_w, rec_a, dt_bias, out_norm_w, conv_state, rec_state,
                       shape, 1 if per_step else 0)


# ---- metrics --------------------------------------------------------------------------------
def compare(cand, reference, rel_floor=1e-12):
    """dict(max_abs, max_rel, cosine, nonfinite, rel_l2) as cpp/reference/correctness.cpp:18-75."""
    c, r = _f(cand).reshape(-1), _f(reference).reshape(-1)
    assert c.size == r.size
    out = np.zeros(5, dtype=np.float64)
    lib().orc_compare(c, r, c.size, rel_floor, out)
    return dict(max_abs=out[0], max_rel=out[1], cosine=out[2], nonfinite=int(out[3]), rel_l2=out[4])
