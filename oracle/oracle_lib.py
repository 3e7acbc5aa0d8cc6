"""numpy-facing binding of the CPU oracle (oracle/libds4oracle.so).

Test infrastructure: the oracle is the checker for the CUDA kernels.  Only
tests, the smoke check and the benchmark's CPU-baseline legs import this.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

ORACLE_DIR = Path(__file__).resolve().parent
LIB_PATH = ORACLE_DIR / "libds4oracle.so"

TABLE_F16, TABLE_Q8_0 = 0, 1
FP8_BLOCK64_POW2, FP8_ROW_AMAX = 0, 1
GLU_PLAIN, GLU_CLAMP_REF, GLU_CLAMP_SYM = 0, 1, 2


class RopeParams(C.Structure):
    _fields_ = [("freq_base", C.c_float), ("theta_scale", C.c_float), ("freq_scale", C.c_float),
                ("ext_factor", C.c_float), ("attn_factor", C.c_float), ("corr_low", C.c_float),
                ("corr_high", C.c_float)]


_lib = None


def build() -> Path:
    src = [ORACLE_DIR / "ds4_oracle.c", ORACLE_DIR / "ds4_oracle.h"]
    if not LIB_PATH.exists() or any(s.stat().st_mtime > LIB_PATH.stat().st_mtime for s in src):
        subprocess.run(["make", "-C", str(ORACLE_DIR), "libds4oracle.so"], check=True,
                       capture_output=True)
    return LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(str(build()))
        _lib.ds4o_f16_to_f32.restype = C.c_float
        _lib.ds4o_f16_to_f32.argtypes = [C.c_uint16]
        _lib.ds4o_f32_to_f16.restype = C.c_uint16
        _lib.ds4o_f32_to_f16.argtypes = [C.c_float]
        _lib.ds4o_f32_to_bf16.restype = C.c_uint16
        _lib.ds4o_f32_to_bf16.argtypes = [C.c_float]
        _lib.ds4o_bf16_to_f32.restype = C.c_float
        _lib.ds4o_bf16_to_f32.argtypes = [C.c_uint16]
        _lib.ds4o_e4m3_value.restype = C.c_float
        _lib.ds4o_e4m3_value.argtypes = [C.c_int]
        _lib.ds4o_e4m3_nearest_index.restype = C.c_int
        _lib.ds4o_e4m3_nearest_index.argtypes = [C.c_float]
        _lib.ds4o_e4m3_encode.restype = C.c_uint8
        _lib.ds4o_e4m3_encode.argtypes = [C.c_float]
        _lib.ds4o_e4m3_decode.restype = C.c_float
        _lib.ds4o_e4m3_decode.argtypes = [C.c_uint8]
    return _lib


def _p(a):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be C-contiguous"
    return a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _call(name, *args):
    fn = getattr(lib(), name)
    fn.restype = None
    conv = []
    for a in args:
        if isinstance(a, np.ndarray) or a is None:
            conv.append(_p(a))
        elif isinstance(a, float):
            conv.append(C.c_float(a))
        elif isinstance(a, (int, np.integer)):
            conv.append(C.c_int64(int(a)))
        else:
            conv.append(a)
    fn(*conv)


def _i(v):
    return C.c_int(int(v))


# ---- parameter helpers -----------------------------------------------------

def rope_params_for_layer(il: int, n_rot: int = 64) -> RopeParams:
    p = RopeParams()
    _call("ds4o_rope_params_for_layer", _i(il), _i(n_rot), C.byref(p))
    return p


def rope_params_explicit(freq_base, yarn_factor, n_ctx_orig, n_rot=64) -> RopeParams:
    p = RopeParams()
    _call("ds4o_rope_params_explicit", C.c_float(freq_base), C.c_float(yarn_factor), _i(n_ctx_orig),
          _i(n_rot), C.byref(p))
    return p


# ---- ops ----------------------------------------------------------------------

def add(a, b):
    a, b = _f32(a), _f32(b)
    y = np.empty_like(a)
    _call("ds4o_add", a, b, y, a.size)
    return y


def rms_norm_rows(x, w=None, residual=None, eps=1e-6, want_bf16=False, want_residual=False):
    x = _f32(x)
    rows, n = x.shape
    w = None if w is None else _f32(w)
    residual = None if residual is None else _f32(residual)
    y = np.empty_like(x)
    yb = np.empty(x.shape, dtype=np.uint16) if want_bf16 else None
    ro = np.empty_like(x) if want_residual else None
    _call("ds4o_rms_norm_rows", x, residual, w, 0 if w is None else w.size, y, yb, ro, rows, _i(n),
          float(eps))
    return y, yb, ro


def rope_rows(x, pos, params, n_rot=64, inverse=False, unit_rms=False, eps=1e-6):
    x = _f32(x)
    T, H, D = x.shape
    out = np.empty_like(x)
    _call("ds4o_rope_rows", x, out, T, _i(H), _i(D), _i(n_rot), _i32(pos), C.byref(params),
          _i(inverse), _i(unit_rms), float(eps))
    return out


def fp8_kv_round_trip_rows(kv, n_rot=64):
    kv = _f32(kv)
    out = np.empty_like(kv)
    _call("ds4o_fp8_kv_round_trip_rows", kv, out, kv.shape[0], _i(kv.shape[1]), _i(n_rot))
    return out


def n_scales(head_dim, n_rot, scale_mode):
    return (head_dim - n_rot) // 64 if scale_mode == FP8_BLOCK64_POW2 else 1


def fp8_encode_rows(rows, n_rot, scale_mode, n_slots=None, slots=None):
    rows = _f32(rows)
    R, D = rows.shape
    n_slots = R if n_slots is None else n_slots
    ns = n_scales(D, n_rot, scale_mode)
    codes = np.zeros((n_slots, D), dtype=np.uint8)
    scales = np.zeros((n_slots, ns), dtype=np.float32)
    tail = np.zeros((n_slots, n_rot), dtype=np.float32)
    _call("ds4o_fp8_encode_rows", rows, R, _i(D), _i(n_rot), _i(scale_mode),
          None if slots is None else _i32(slots), codes, scales, tail)
    return codes, scales, tail


def rope_fp8_store_rows(kv, pos, params, n_rot, scale_mode, n_slots=None, slots=None, norm_w=None,
                        eps=1e-6):
    kv = _f32(kv)
    R, D = kv.shape
    n_slots = R if n_slots is None else n_slots
    ns = n_scales(D, n_rot, scale_mode)
    codes = np.zeros((n_slots, D), dtype=np.uint8)
    scales = np.zeros((n_slots, ns), dtype=np.float32)
    tail = np.zeros((n_slots, n_rot), dtype=np.float32)
    rope_out = np.empty_like(kv)
    _call("ds4o_rope_fp8_store_rows", kv, R, _i(D), _i(n_rot), _i32(pos), C.byref(params),
          None if norm_w is None else _f32(norm_w), float(eps), _i(scale_mode),
          None if slots is None else _i32(slots), codes, scales, tail, rope_out)
    return codes, scales, tail, rope_out


def f16_round(x):
    x = _f32(x)
    y = np.empty_like(x)
    _call("ds4o_f16_round", x, y, x.size)
    return y


def kv_rows_to_raw(kv, pos, params, n_rot=64, norm_w=None, eps=1e-6):
    """The reference's KV row chain: kv_norm -> RoPE -> FP8 round trip -> f16 round."""
    kv = _f32(kv)
    x = rms_norm_rows(kv, norm_w, eps=eps)[0] if norm_w is not None else kv
    x = rope_rows(x[:, None, :], pos, params, n_rot=n_rot)[:, 0, :]
    return f16_round(fp8_kv_round_trip_rows(x, n_rot=n_rot))


def swa_window_push(window, n_raw, new_rows):
    """One row at a time, as cuda/forward_layer.cu:941-972 does; returns (window, n_raw)."""
    window = window.copy()
    cap = window.shape[0]
    for row in f16_round(new_rows):
        if n_raw < cap:
            window[n_raw] = row
            n_raw += 1
        else:
            window[:-1] = f16_round(window[1:])
            window[-1] = row
    return window, n_raw


def quantize_q8_0_rows(x):
    x = _f32(x).ravel()
    nb = x.size // 32
    xq, xs = np.empty(nb * 32, dtype=np.int8), np.empty(nb, dtype=np.float32)
    _call("ds4o_quantize_q8_0_rows", x, xq, xs, nb)
    return xq, xs


def quantize_q8_K_rows(x):
    x = _f32(x).ravel()
    nb = x.size // 256
    xq, xs, bs = np.empty(nb * 256, dtype=np.int8), np.empty(nb, dtype=np.float32), np.empty(nb * 16, dtype=np.int16)
    _call("ds4o_quantize_q8_K_rows", x, xq, xs, bs, nb)
    return xq, xs, bs


def swiglu_rows(gate, up, weights=None, mode=GLU_PLAIN, clamp=0.0, combine=False):
    gate, up = _f32(gate), _f32(up)
    T, k, n = gate.shape
    out = np.empty((T, n) if combine else (T, k, n), dtype=np.float32)
    _call("ds4o_swiglu_rows", gate, up, None if weights is None else _f32(weights), out, T, _i(k),
          _i(n), _i(mode), float(clamp), _i(combine))
    return out


def embed_gather_rows(table, table_dtype, ids, n_embd, residual=None, norm_w=None, eps=1e-6,
                      n_replicas=1, want_bf16=False):
    ids = _i32(ids)
    T = ids.size
    rows = np.empty((T, n_replicas, n_embd), dtype=np.float32)
    nf = np.empty((T, n_embd), dtype=np.float32) if norm_w is not None else None
    nb = np.empty((T, n_embd), dtype=np.uint16) if (norm_w is not None and want_bf16) else None
    _call("ds4o_embed_gather_rows", np.ascontiguousarray(table), _i(table_dtype), ids, T, _i(n_embd),
          None if residual is None else _f32(residual), None if norm_w is None else _f32(norm_w),
          float(eps), rows, _i(n_replicas), nf, nb)
    return rows, nf, nb


def sinkhorn_4x4(v, iters=20, eps=1e-6):
    v = _f32(v).reshape(16)
    c = np.empty(16, dtype=np.float32)
    _call("ds4o_sinkhorn_4x4", v, _i(iters), float(eps), c)
    return c


def hc_pre_rows(resid, fn_f16, scale3, base24, iters=20, eps=1e-6):
    resid = _f32(resid)
    T, _, n = resid.shape
    post = np.empty((T, 4), dtype=np.float32)
    comb = np.empty((T, 16), dtype=np.float32)
    out = np.empty((T, n), dtype=np.float32)
    mix = np.empty((T, 24), dtype=np.float32)
    _call("ds4o_hc_pre_rows", resid, np.ascontiguousarray(fn_f16).view(np.uint16), _f32(scale3),
          _f32(base24), post, comb, out, mix, T, _i(n), _i(iters), float(eps))
    return post, comb, out, mix


def output_hc_head_rows(resid, fn_f16, scale1, base4, norm_w=None, eps=1e-6):
    resid = _f32(resid)
    T, _, n = resid.shape
    out = np.empty((T, n), dtype=np.float32)
    normed = np.empty((T, n), dtype=np.float32) if norm_w is not None else None
    _call("ds4o_output_hc_head_rows", resid, np.ascontiguousarray(fn_f16).view(np.uint16), _f32(scale1),
          _f32(base4), None if norm_w is None else _f32(norm_w), out, normed, T, _i(n), float(eps))
    return out, normed


def hc_post_rows(block_out, resid, post, comb, block_out2=None):
    resid = _f32(resid)
    T, _, n = resid.shape
    out = np.empty_like(resid)
    _call("ds4o_hc_post_rows", None if block_out is None else _f32(block_out),
          None if block_out2 is None else _f32(block_out2), resid,
          None if post is None else _f32(post), _f32(comb), out, T, _i(n))
    return out


def hc_sinkhorn_mix_rows(logits, resid, iters=20, eps=1e-6):
    resid = _f32(resid)
    T, _, n = resid.shape
    out = np.empty_like(resid)
    comb = np.empty((T, 16), dtype=np.float32)
    _call("ds4o_hc_sinkhorn_mix_rows", _f32(logits), resid, out, comb, T, _i(n), _i(iters), float(eps))
    return out, comb


def compressor_step(is_attn, kv_cur, sc_cur, ape_f16, norm_w, head_dim, ratio, pos, params,
                    state_kv, state_score, n_rot=64, eps=1e-6):
    """One step; sc_cur, state_kv, state_score are updated in place.  Returns emit [head_dim] or None."""
    assert kv_cur.dtype == np.float32 and sc_cur.dtype == np.float32 and ape_f16.dtype == np.uint16
    assert state_kv.dtype == np.float32 and state_score.dtype == np.float32
    emit = np.zeros(head_dim, dtype=np.float32)
    fn = lib().ds4o_compressor_step
    fn.restype = C.c_int
    rc = fn(_i(is_attn), _p(kv_cur), _p(sc_cur), _p(ape_f16), _p(_f32(norm_w)), _i(head_dim), _i(ratio), _i(pos),
            C.byref(params), _i(n_rot), C.c_float(eps), _p(state_kv), _p(state_score), _p(emit))
    return emit if rc else None


def e4m3_encode(x):
    x = _f32(x).ravel()
    f = lib().ds4o_e4m3_encode
    return np.array([f(float(v)) for v in x], dtype=np.uint8)


def e4m3_decode(codes):
    f = lib().ds4o_e4m3_decode
    return np.array([f(int(c)) for c in np.asarray(codes).ravel()], dtype=np.float32)
