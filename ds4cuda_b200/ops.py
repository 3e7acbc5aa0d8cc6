"""Host-side mirror of the C ABI on torch CUDA tensors.

Every function here only allocates outputs (torch) and forwards device
pointers plus torch's current stream to libds4b200.so; the arithmetic lives in
the CUDA kernels.  Tensors must be contiguous CUDA tensors; nothing runs on CPU.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from ._lib import (FP8_BLOCK64_POW2, FP8_ROW_AMAX, GLU_CLAMP_REF, GLU_CLAMP_SYM, GLU_PLAIN,
                   TABLE_F16, TABLE_Q8_0, RopeParams, check)

__all__ = [
    "FP8_BLOCK64_POW2", "FP8_ROW_AMAX", "GLU_CLAMP_REF", "GLU_CLAMP_SYM", "GLU_PLAIN",
    "TABLE_F16", "TABLE_Q8_0", "RopeParams", "rope_params_for_layer", "rope_params_explicit",
    "add", "rms_norm_rows", "rms_norm_q8_0_rows", "quantize_q8_0_rows", "quantize_q8_K_rows", "embed_gather_rows", "rope_rows", "rope_table_rows", "rope_q8_0_rows", "fp8_kv_round_trip_rows",
    "rope_fp8_store_rows", "fp8_cache_load_rows", "kv_rows_to_raw", "swa_window_push_rows", "swiglu_rows", "hc_pre_rows", "hc_pre_norm_rows", "output_hc_head_rows", "hc_post_rows", "hc_sinkhorn_rows", "hc_sinkhorn_mix_rows",
    "e4m3_encode", "e4m3_decode", "e4m3_selfcheck", "div_selfcheck", "device_status", "compressor_step", "compressor_chunk", "swiglu_q8_K_rows",
]


def _p(t):
    if t is None:
        return None
    if not t.is_cuda:
        raise ValueError("ds4cuda_b200 ops take CUDA tensors only")
    if not t.is_contiguous():
        raise ValueError("ds4cuda_b200 ops take contiguous tensors")
    return C.c_void_p(t.data_ptr())


def _s():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def rope_params_for_layer(il: int, n_rot: int = 64) -> RopeParams:
    """Per-layer routing of the reference launcher (cuda/rope.cu:214-250)."""
    p = RopeParams()
    _lib.load().ds4b200_rope_params_for_layer(il, n_rot, C.byref(p))
    return p


def rope_params_explicit(freq_base: float, yarn_factor: float, n_ctx_orig: int,
                         n_rot: int = 64) -> RopeParams:
    p = RopeParams()
    _lib.load().ds4b200_rope_params_explicit(freq_base, yarn_factor, n_ctx_orig, n_rot, C.byref(p))
    return p


def device_status() -> int:
    return _lib.load().ds4b200_device_status()


def add(a, b):
    y = torch.empty_like(a)
    check(_lib.load().ds4b200_add_f32(_p(a), _p(b), _p(y), a.numel(), _s()))
    return y


def rms_norm_rows(x, w=None, residual=None, eps=1e-6, want_f32=True, want_bf16=False,
                  want_residual=False):
    """x [rows, n]; w None | [n] | [rows, n].  Returns (y_f32, y_bf16, residual_out)."""
    rows, n = x.shape
    weight_dim = 0 if w is None else w.numel()
    y = torch.empty_like(x) if want_f32 else None
    yb = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device) if want_bf16 else None
    ro = torch.empty_like(x) if want_residual else None
    check(_lib.load().ds4b200_rms_norm_rows_f32(_p(x), _p(residual), _p(w), weight_dim, _p(y),
                                                _p(yb), _p(ro), rows, n, eps, _s()))
    return y, yb, ro


def rms_norm_q8_0_rows(x, w=None, residual=None, eps=1e-6, want_f32=True, want_residual=False):
    """RMSNorm + Q8_0 activation quantiser.  Returns (y_f32, residual_out, xq int8 [rows, n], xscale [rows, n/32])."""
    rows, n = x.shape
    y = torch.empty_like(x) if want_f32 else None
    ro = torch.empty_like(x) if want_residual else None
    xq = torch.empty((rows, n), dtype=torch.int8, device=x.device)
    xs = torch.empty((rows, n // 32), dtype=torch.float32, device=x.device)
    check(_lib.load().ds4b200_rms_norm_q8_0_rows_f32(_p(x), _p(residual), _p(w), 0 if w is None else w.numel(), _p(y),
                                                     _p(ro), _p(xq), _p(xs), rows, n, eps, _s()))
    return y, ro, xq, xs


def rms_norm_q8_K_rows(x, w=None, residual=None, eps=1e-6, want_f32=True, want_residual=False, want_q8_0=False):
    """RMSNorm + Q8_K activation quantiser (and optionally the Q8_0 one on the same row).  Returns
    (y_f32, residual_out, (xq, xscale) or None, (kq int8 [rows, n], kscale [rows, n/256], kbsums int16 [rows, n/16]))."""
    rows, n = x.shape
    y = torch.empty_like(x) if want_f32 else None
    ro = torch.empty_like(x) if want_residual else None
    xq = torch.empty((rows, n), dtype=torch.int8, device=x.device) if want_q8_0 else None
    xs = torch.empty((rows, n // 32), dtype=torch.float32, device=x.device) if want_q8_0 else None
    kq = torch.empty((rows, n), dtype=torch.int8, device=x.device)
    ks = torch.empty((rows, n // 256), dtype=torch.float32, device=x.device)
    kb = torch.empty((rows, n // 16), dtype=torch.int16, device=x.device)
    check(_lib.load().ds4b200_rms_norm_q8_K_rows_f32(_p(x), _p(residual), _p(w), 0 if w is None else w.numel(), _p(y),
                                                     _p(ro), _p(xq), _p(xs), _p(kq), _p(ks), _p(kb), rows, n, eps,
                                                     _s()))
    return y, ro, ((xq, xs) if want_q8_0 else None), (kq, ks, kb)


def quantize_q8_0_rows(x):
    """x with numel % 32 == 0 -> (int8 like x, f32 scales [numel/32])."""
    xq = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    xs = torch.empty(x.numel() // 32, dtype=torch.float32, device=x.device)
    check(_lib.load().ds4b200_quantize_q8_0_rows_f32(_p(x), _p(xq), _p(xs), x.numel() // 32, _s()))
    return xq, xs


def quantize_q8_K_rows(x):
    """x with numel % 256 == 0 -> (int8 like x, f32 scales [numel/256], int16 sums [numel/16])."""
    nb = x.numel() // 256
    xq = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    xs = torch.empty(nb, dtype=torch.float32, device=x.device)
    bs = torch.empty(nb * 16, dtype=torch.int16, device=x.device)
    check(_lib.load().ds4b200_quantize_q8_K_rows_f32(_p(x), _p(xq), _p(xs), _p(bs), nb, _s()))
    return xq, xs, bs


def embed_gather_rows(table, table_dtype, ids, n_embd, residual=None, norm_w=None, eps=1e-6,
                      n_replicas=1, want_rows=True, want_f32=False, want_bf16=False):
    """Returns (rows [T, n_replicas, n_embd] f32, normed_f32, normed_bf16)."""
    T = ids.numel()
    dev = ids.device
    rows = torch.empty((T, n_replicas, n_embd), dtype=torch.float32, device=dev) if want_rows else None
    nf = torch.empty((T, n_embd), dtype=torch.float32, device=dev) if want_f32 else None
    nb = torch.empty((T, n_embd), dtype=torch.bfloat16, device=dev) if want_bf16 else None
    check(_lib.load().ds4b200_embed_gather_rows(_p(table), table_dtype, _p(ids), T, n_embd,
                                                _p(residual), _p(norm_w), eps, _p(rows), n_replicas,
                                                _p(nf), _p(nb), _s()))
    return rows, nf, nb


def rope_rows(x, pos, params, n_rot=64, inverse=False, unit_rms=False, eps=1e-6, out=None, table=None):
    """x [T, H, D], pos [T] int32; table: rope_table_rows(pos, params), in place of pos + params."""
    T, H, D = x.shape
    out = torch.empty_like(x) if out is None else out
    if table is not None:
        check(_lib.load().ds4b200_rope_rows_table_f32(_p(x), _p(out), T, H, D, n_rot, _p(table), int(inverse),
                                                      int(unit_rms), eps, _s()))
        return out
    check(_lib.load().ds4b200_rope_rows_f32(_p(x), _p(out), T, H, D, n_rot, _p(pos),
                                            C.byref(params), int(inverse), int(unit_rms), eps, _s()))
    return out


def rope_table_rows(pos, params, n_rot=64):
    """(cos, sin) multipliers of the n_rot/2 tail pairs at every position: [T, n_rot/2, 2]."""
    T = pos.numel()
    cs = torch.empty((T, n_rot // 2, 2), dtype=torch.float32, device=pos.device)
    check(_lib.load().ds4b200_rope_table_rows(_p(pos), C.byref(params), T, n_rot, _p(cs), _s()))
    return cs


def rope_q8_0_rows(x, pos, params, n_rot=64, inverse=False, unit_rms=False, eps=1e-6, want_f32=False, table=None):
    """rope_rows whose result leaves as Q8_0 blocks: (out f32 or None, xq int8 [T, H, D], xscale [T, H, D/32]).
    table: rope_table_rows(pos, params), in place of pos + params."""
    T, H, D = x.shape
    out = torch.empty_like(x) if want_f32 else None
    xq = torch.empty((T, H, D), dtype=torch.int8, device=x.device)
    xs = torch.empty((T, H, D // 32), dtype=torch.float32, device=x.device)
    check(_lib.load().ds4b200_rope_q8_0_rows_f32(_p(x), _p(out), _p(xq), _p(xs), T, H, D, n_rot, _p(pos),
                                                 None if params is None else C.byref(params), _p(table),
                                                 int(inverse), int(unit_rms), eps, _s()))
    return out, xq, xs


def fp8_kv_round_trip_rows(kv, n_rot=64, out=None):
    rows, D = kv.shape
    out = torch.empty_like(kv) if out is None else out
    check(_lib.load().ds4b200_fp8_kv_round_trip_rows_f32(_p(kv), _p(out), rows, D, n_rot, _s()))
    return out


def rope_fp8_store_rows(kv, pos, params, n_rot, scale_mode, codes, scales, slots=None,
                        norm_w=None, eps=1e-6, tail_out=None, rope_out=None, table=None):
    """Writes into the caller's cache tensors `codes` (uint8) and `scales` (f32).  `table` (rope_table_rows,
    one row per kv row) replaces pos + params."""
    rows, D = kv.shape
    if table is not None:
        check(_lib.load().ds4b200_rope_fp8_store_rows_table(
            _p(kv), rows, D, n_rot, _p(table), _p(norm_w), eps, scale_mode, _p(slots), _p(codes), _p(scales),
            _p(tail_out), _p(rope_out), _s()))
        return
    check(_lib.load().ds4b200_rope_fp8_store_rows(
        _p(kv), rows, D, n_rot, _p(pos), None if params is None else C.byref(params), _p(norm_w),
        eps, scale_mode, _p(slots), _p(codes), _p(scales), _p(tail_out), _p(rope_out), _s()))


def fp8_cache_load_rows(codes, scales, slots, n_rot, scale_mode, tail=None, f16_round=False):
    """Rows at `slots` of the byte cache -> f32 [len(slots), head_dim]."""
    D = codes.shape[1]
    out = torch.empty((slots.numel(), D), dtype=torch.float32, device=codes.device)
    check(_lib.load().ds4b200_fp8_cache_load_rows(_p(codes), _p(scales), _p(tail), _p(slots), slots.numel(), D, n_rot,
                                                  scale_mode, int(f16_round), _p(out), _s()))
    return out


def kv_rows_to_raw(kv, pos, params, raw_out, n_rot=64, slots=None, norm_w=None, eps=1e-6, table=None, table_out=None):
    """norm -> RoPE -> FP8 round trip -> f16 round, written to raw_out[slot] (f32 rows).  `table`
    (rope_table_rows, one row per kv row) replaces pos + params; `table_out` [rows, n_rot/2, 2] receives the
    angles this launch evaluates (the chunk's table, for the RoPE launches that follow)."""
    rows, D = kv.shape
    if table_out is not None:
        check(_lib.load().ds4b200_kv_rows_to_raw_table_out_f32(_p(kv), rows, D, n_rot, _p(pos), C.byref(params),
                                                               _p(norm_w), eps, _p(slots), _p(raw_out), _p(table_out), _s()))
        return raw_out
    if table is not None:
        check(_lib.load().ds4b200_kv_rows_to_raw_table_f32(_p(kv), rows, D, n_rot, _p(table), _p(norm_w), eps,
                                                           _p(slots), _p(raw_out), _s()))
        return raw_out
    check(_lib.load().ds4b200_kv_rows_to_raw_f32(_p(kv), rows, D, n_rot, _p(pos),
                                                 None if params is None else C.byref(params), _p(norm_w), eps,
                                                 _p(slots), _p(raw_out), _s()))
    return raw_out


def swa_window_push_rows(raw_kv, n_raw, new_rows):
    """raw_kv [cap, D] window with n_raw rows; pushes new_rows [n, D]; returns the new row count."""
    cap, D = raw_kv.shape
    after = C.c_int()
    check(_lib.load().ds4b200_swa_window_push_rows_f32(_p(raw_kv), cap, n_raw, _p(new_rows), new_rows.shape[0], D,
                                                       C.byref(after), _s()))
    return after.value


def compressor_chunk(is_attn, kv_cur, sc_cur, ape_f16, norm_w, head_dim, ratio, pos0, il, state_kv, state_score):
    """A window-aligned chunk of compressor steps at once; returns emits [T / ratio, head_dim]."""
    T = kv_cur.shape[0]
    emits = torch.empty((T // ratio, head_dim), dtype=torch.float32, device=kv_cur.device)
    check(_lib.load().ds4b200_compressor_chunk_f32(int(is_attn), _p(kv_cur), _p(sc_cur), _p(ape_f16), _p(norm_w),
                                                   head_dim, ratio, pos0, T, il, _p(state_kv), _p(state_score),
                                                   _p(emits), _s()))
    return emits


def swiglu_q8_K_rows(gate, up, weights=None, mode=GLU_PLAIN, clamp=0.0, fast_exp=False, want_f32=False):
    """gate/up [T, k, n] -> Q8_K blocks of the [T, k, n] SwiGLU rows: (xq int8 [T,k,n], scales [T,k,n/256],
    bsums int16 [T,k,n/256,16], mid f32 or None)."""
    T, k, n = gate.shape
    dev = gate.device
    xq = torch.empty((T, k, n), dtype=torch.int8, device=dev)
    xs = torch.empty((T, k, n // 256), dtype=torch.float32, device=dev)
    bs = torch.empty((T, k, n // 256, 16), dtype=torch.int16, device=dev)
    mid = torch.empty((T, k, n), dtype=torch.float32, device=dev) if want_f32 else None
    check(_lib.load().ds4b200_swiglu_q8_K_rows_f32(_p(gate), _p(up), _p(weights), _p(xq), _p(xs), _p(bs), _p(mid),
                                                   T, k, n, mode, clamp, int(fast_exp), _s()))
    return xq, xs, bs, mid


def compressor_step(is_attn, kv_cur, sc_cur, ape_f16, norm_w, head_dim, ratio, pos, il, state_kv, state_score,
                    emit_out):
    """One streaming-compressor step after its projections, in place; True when emit_out was written."""
    emitted = C.c_int()
    check(_lib.load().ds4b200_compressor_step_f32(int(is_attn), _p(kv_cur), _p(sc_cur), _p(ape_f16), _p(norm_w),
                                                  head_dim, ratio, pos, il, _p(state_kv), _p(state_score),
                                                  _p(emit_out), C.byref(emitted), _s()))
    return bool(emitted.value)


def swiglu_rows(gate, up, weights=None, mode=GLU_PLAIN, clamp=0.0, combine=False, fast_exp=False):
    """gate/up [T, k, n]; returns [T, n] when combine else [T, k, n]."""
    T, k, n = gate.shape
    out = torch.empty((T, n) if combine else (T, k, n), dtype=torch.float32, device=gate.device)
    check(_lib.load().ds4b200_swiglu_rows_f32(_p(gate), _p(up), _p(weights), _p(out), T, k, n, mode,
                                              clamp, int(combine), int(fast_exp), _s()))
    return out


def swiglu_q8_0_rows(gate, up, weights=None, mode=GLU_PLAIN, clamp=0.0, fast_exp=False, want_f32=False):
    """gate/up [T, k, n] -> (xq int8 [T, k, n], xscale [T, k, n/32], mid f32 or None): the SwiGLU rows as Q8_0 blocks."""
    T, k, n = gate.shape
    xq = torch.empty((T, k, n), dtype=torch.int8, device=gate.device)
    xs = torch.empty((T, k, n // 32), dtype=torch.float32, device=gate.device)
    mid = torch.empty((T, k, n), dtype=torch.float32, device=gate.device) if want_f32 else None
    check(_lib.load().ds4b200_swiglu_q8_0_rows_f32(_p(gate), _p(up), _p(weights), _p(xq), _p(xs), _p(mid), T, k, n, mode,
                                                   clamp, int(fast_exp), _s()))
    return xq, xs, mid


def hc_pre_rows(resid, fn_f16, scale3, base24, iters=20, eps=1e-6):
    """resid [T, 4, n]; fn_f16 [24, 4n] float16.  Returns (post [T,4], comb [T,16], out [T,n])."""
    T, _, n = resid.shape
    dev = resid.device
    post = torch.empty((T, 4), dtype=torch.float32, device=dev)
    comb = torch.empty((T, 16), dtype=torch.float32, device=dev)
    out = torch.empty((T, n), dtype=torch.float32, device=dev)
    check(_lib.load().ds4b200_hc_pre_rows_f32(_p(resid), _p(fn_f16), _p(scale3), _p(base24), _p(post),
                                              _p(comb), _p(out), T, n, iters, eps, _s()))
    return post, comb, out


def hc_pre_norm_rows(resid, fn_f16, scale3, base24, norm_w, iters=20, eps=1e-6, want_normed=True, want_q8=True):
    """hc_pre_rows followed by RMSNorm(out) * norm_w and its Q8_0 blocks.
    Returns (post, comb, out, normed or None, xq int8 [T, n] or None, xscale [T, n/32] or None)."""
    T, _, n = resid.shape
    dev = resid.device
    post = torch.empty((T, 4), dtype=torch.float32, device=dev)
    comb = torch.empty((T, 16), dtype=torch.float32, device=dev)
    out = torch.empty((T, n), dtype=torch.float32, device=dev)
    normed = torch.empty((T, n), dtype=torch.float32, device=dev) if want_normed else None
    xq = torch.empty((T, n), dtype=torch.int8, device=dev) if want_q8 else None
    xscale = torch.empty((T, n // 32), dtype=torch.float32, device=dev) if want_q8 else None
    check(_lib.load().ds4b200_hc_pre_norm_rows_f32(_p(resid), _p(fn_f16), _p(scale3), _p(base24), _p(norm_w), _p(post),
                                                   _p(comb), _p(out), _p(normed), _p(xq), _p(xscale), T, n, iters,
                                                   eps, _s()))
    return post, comb, out, normed, xq, xscale


def output_hc_head_rows(resid, fn_f16, scale1, base4, norm_w=None, eps=1e-6, want_out=True):
    """resid [T, 4, n]; fn_f16 [4, 4n].  Returns (out [T, n], normed [T, n] or None)."""
    T, _, n = resid.shape
    out = torch.empty((T, n), dtype=torch.float32, device=resid.device) if want_out else None
    normed = torch.empty((T, n), dtype=torch.float32, device=resid.device) if norm_w is not None else None
    check(_lib.load().ds4b200_output_hc_head_rows_f32(_p(resid), _p(fn_f16), _p(scale1), _p(base4), _p(norm_w),
                                                      _p(out), _p(normed), T, n, eps, _s()))
    return out, normed


def hc_post_rows(block_out, resid, post, comb, block_out2=None):
    T, _, n = resid.shape
    out = torch.empty_like(resid)
    check(_lib.load().ds4b200_hc_post_rows_f32(_p(block_out), _p(block_out2), _p(resid), _p(post),
                                               _p(comb), _p(out), T, n, _s()))
    return out


def hc_post_pre_rows(block_out, resid, post, comb, fn_f16, scale3, base24, block_out2=None, iters=20, eps=1e-6):
    """hc_post_rows then hc_pre_rows of its result.  Returns (out_hc [T,4,n], post [T,4], comb [T,16], out [T,n])."""
    T, _, n = resid.shape
    dev = resid.device
    out_hc = torch.empty_like(resid)
    post2 = torch.empty((T, 4), dtype=torch.float32, device=dev)
    comb2 = torch.empty((T, 16), dtype=torch.float32, device=dev)
    out = torch.empty((T, n), dtype=torch.float32, device=dev)
    check(_lib.load().ds4b200_hc_post_pre_rows_f32(_p(block_out), _p(block_out2), _p(resid), _p(post), _p(comb),
                                                   _p(fn_f16), _p(scale3), _p(base24), _p(out_hc), _p(post2), _p(comb2),
                                                   _p(out), T, n, iters, eps, _s()))
    return out_hc, post2, comb2, out


def hc_sinkhorn_rows(logits, iters=20, eps=1e-6):
    """logits [T, 16] -> comb [T, 16]."""
    comb = torch.empty_like(logits)
    check(_lib.load().ds4b200_hc_sinkhorn_rows_f32(_p(logits), _p(comb), logits.shape[0], iters, eps, _s()))
    return comb


def hc_sinkhorn_mix_rows(logits, resid, iters=20, eps=1e-6, want_comb=False):
    T, _, n = resid.shape
    out = torch.empty_like(resid)
    comb = torch.empty((T, 16), dtype=torch.float32, device=resid.device) if want_comb else None
    check(_lib.load().ds4b200_hc_sinkhorn_mix_rows_f32(_p(logits), _p(resid), _p(out), _p(comb), T, n,
                                                       iters, eps, _s()))
    return (out, comb) if want_comb else out


def e4m3_encode(x):
    codes = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    check(_lib.load().ds4b200_e4m3_encode_f32(_p(x), _p(codes), x.numel(), _s()))
    return codes


def e4m3_decode(codes):
    x = torch.empty(codes.shape, dtype=torch.float32, device=codes.device)
    check(_lib.load().ds4b200_e4m3_decode_f32(_p(codes), _p(x), codes.numel(), _s()))
    return x


def e4m3_selfcheck(first_bits: int, count: int) -> int:
    """Number of f32 bit patterns in the range whose hardware code differs from the table rule."""
    bad = torch.zeros(1, dtype=torch.int64, device="cuda")
    check(_lib.load().ds4b200_e4m3_selfcheck(first_bits, count, _p(bad), _s()))
    return int(bad.item())


def div_selfcheck(first: int, count: int) -> int:
    """Pairs (n, d in [1, 2]) for which the kernels' branch-free division differs from n / d."""
    bad = torch.zeros(1, dtype=torch.int64, device="cuda")
    check(_lib.load().ds4b200_div_selfcheck(first, count, _p(bad), _s()))
    return int(bad.item())
