"""ctypes binding of libds4b200.so (the C ABI declared in include/ds4b200.h).

The library is the product: if it is missing this module raises, there is no
Python or CPU fallback for any op.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libds4b200.so"


class RopeParams(C.Structure):
    """Mirror of `ds4b200_rope_params`."""
    _fields_ = [("freq_base", C.c_float), ("theta_scale", C.c_float), ("freq_scale", C.c_float),
                ("ext_factor", C.c_float), ("attn_factor", C.c_float), ("corr_low", C.c_float),
                ("corr_high", C.c_float)]


class PathConfig(C.Structure):
    """Mirror of `ds4b200_path_config`."""
    _fields_ = [(n, C.c_int32) for n in (
        "n_tokens", "n_embd", "vocab", "table_dtype", "kv_dim", "n_rot", "n_slots", "ff_dim",
        "top_k", "max_layers", "sinkhorn_iters", "fp8_scale_mode", "glu_mode", "glu_fast_exp",
        "use_graph")] + [("eps", C.c_float), ("clamp", C.c_float), ("rope", RopeParams)]


class PathIO(C.Structure):
    """Mirror of `ds4b200_path_io` (host pointers; None = skip)."""
    INPUTS = ("ids", "pos", "residual", "norm_w", "kv", "gate", "up", "router_w", "hc_logits",
              "hc_resid")
    OUTPUTS = ("residual_out", "normed_bf16", "kv_codes", "kv_scales", "kv_tail", "ffn_out",
               "hc_out")
    _fields_ = [(n, C.c_void_p) for n in INPUTS + OUTPUTS]


class LayerDims(C.Structure):
    """Mirror of `ds4b200_layer_dims` (include/ds4b200_layer.h)."""
    _fields_ = [(n, C.c_int32) for n in ("n_embd", "n_heads", "head_dim", "n_rot", "q_lora", "ff_dim", "top_k",
                                         "sinkhorn_iters", "il", "glu_fast_exp")] + [("eps", C.c_float),
                                                                                      ("clamp", C.c_float)]


class LayerWeights(C.Structure):
    """Mirror of `ds4b200_layer_weights` (device pointers)."""
    NAMES = ("hc_attn_fn", "hc_attn_scale", "hc_attn_base", "attn_norm", "q_a_norm", "kv_a_norm", "hc_ffn_fn",
             "hc_ffn_scale", "hc_ffn_base", "ffn_norm")
    _fields_ = [(n, C.c_void_p) for n in NAMES]


class LayerBuffers(C.Structure):
    """Mirror of `ds4b200_layer_buffers` (device pointers)."""
    NAMES = ("x", "x_norm", "xq", "xscale", "q_lora", "q_lora_norm", "kv_raw", "raw_rows", "q", "kqv", "attn_out",
             "post", "comb", "resid_mid", "sh_gate", "sh_up", "sh_mid", "gate", "up", "router_w", "mid_q",
             "mid_scale", "mid_bsums", "moe_out", "shexp_out")
    OPTIONAL = ("kqv_q", "kqv_scale", "rope_cs", "ffn_kq", "ffn_kscale", "ffn_kbsums", "sh_q", "sh_scale", "ql_q", "ql_scale")
    _fields_ = [(n, C.c_void_p) for n in NAMES + OPTIONAL]


STAGE_QKV_A, STAGE_Q_B, STAGE_ATTENTION, STAGE_ATTN_OUT, STAGE_FFN_UP, STAGE_FFN_DOWN = range(6)
StageHook = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_int, C.c_int64, C.c_void_p)
ChunkHook = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int64, C.c_void_p)

TABLE_F16, TABLE_Q8_0 = 0, 1
FP8_BLOCK64_POW2, FP8_ROW_AMAX = 0, 1
GLU_PLAIN, GLU_CLAMP_REF, GLU_CLAMP_SYM = 0, 1, 2

_P, _I, _L, _F = C.c_void_p, C.c_int, C.c_int64, C.c_float
_RP = C.POINTER(RopeParams)

# name -> (restype, argtypes); one entry per function in include/ds4b200.h
SIGNATURES = {
    "ds4b200_version": (C.c_char_p, []),
    "ds4b200_last_error": (C.c_char_p, []),
    "ds4b200_device_status": (_I, []),
    "ds4b200_selftest_bounded_wait": (_I, [_I, _P, _P]),
    "ds4b200_rope_params_for_layer": (None, [_I, _I, _RP]),
    "ds4b200_rope_params_explicit": (None, [_F, _F, _I, _I, _RP]),
    # drop-in launchers
    "ds4b200_launch_rms_norm_f32": (None, [_P, _P, _P, _I, _F, _P]),
    "ds4b200_launch_rms_norm_batch_f32": (None, [_P, _P, _I, _P, _I, _I, _F, _P]),
    "ds4b200_launch_add_f32": (None, [_P, _P, _P, _I, _P]),
    "ds4b200_launch_tail_rope_yarn_f32": (None, [_P, _P, _I, _I, _I, _I, _I, _P]),
    "ds4b200_launch_tail_rope_yarn_inverse_f32": (None, [_P, _P, _I, _I, _I, _I, _I, _P]),
    "ds4b200_launch_fp8_kv_quantize_round_trip_f32": (None, [_P, _P, _I, _I, _I, _P]),
    "ds4b200_launch_silu_mul_f32": (None, [_P, _P, _P, _I, _P]),
    "ds4b200_launch_embed_token_f16_to_f32": (None, [_P, _I, _I, _P, _P]),
    "ds4b200_launch_hc_attn_pre_f32": (None, [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _F, _P]),
    "ds4b200_launch_hc_attn_pre_v2_f32": (None, [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _F, _P, _P, _P]),
    "ds4b200_launch_hc_post_f32": (None, [_P, _P, _P, _P, _P, _I, _I, _P]),
    "ds4b200_launch_output_hc_head_f32": (None, [_P, _P, _P, _P, _P, _I, _I, _F, _P]),
    # batched siblings
    "ds4b200_add_f32": (_I, [_P, _P, _P, _L, _P]),
    "ds4b200_rms_norm_rows_f32": (_I, [_P, _P, _P, _L, _P, _P, _P, _L, _I, _F, _P]),
    "ds4b200_rms_norm_q8_0_rows_f32": (_I, [_P, _P, _P, _L, _P, _P, _P, _P, _L, _I, _F, _P]),
    "ds4b200_rms_norm_q8_K_rows_f32": (_I, [_P, _P, _P, _L, _P, _P, _P, _P, _P, _P, _P, _L, _I, _F, _P]),
    "ds4b200_quantize_q8_0_rows_f32": (_I, [_P, _P, _P, _L, _P]),
    "ds4b200_quantize_q8_K_rows_f32": (_I, [_P, _P, _P, _P, _L, _P]),
    "ds4b200_embed_gather_rows": (_I, [_P, _I, _P, _L, _I, _P, _P, _F, _P, _I, _P, _P, _P]),
    "ds4b200_rope_rows_f32": (_I, [_P, _P, _L, _I, _I, _I, _P, _RP, _I, _I, _F, _P]),
    "ds4b200_rope_q8_0_rows_f32": (_I, [_P, _P, _P, _P, _L, _I, _I, _I, _P, _RP, _P, _I, _I, _F, _P]),
    "ds4b200_rope_table_rows": (_I, [_P, _RP, _L, _I, _P, _P]),
    "ds4b200_rope_rows_table_f32": (_I, [_P, _P, _L, _I, _I, _I, _P, _I, _I, _F, _P]),
    "ds4b200_fp8_kv_round_trip_rows_f32": (_I, [_P, _P, _L, _I, _I, _P]),
    "ds4b200_rope_fp8_store_rows": (_I, [_P, _L, _I, _I, _P, _RP, _P, _F, _I, _P, _P, _P, _P, _P, _P]),
    "ds4b200_fp8_cache_load_rows": (_I, [_P, _P, _P, _P, _L, _I, _I, _I, _I, _P, _P]),
    "ds4b200_kv_rows_to_raw_f32": (_I, [_P, _L, _I, _I, _P, _RP, _P, _F, _P, _P, _P]),
    "ds4b200_rope_fp8_store_rows_table": (_I, [_P, _L, _I, _I, _P, _P, _F, _I, _P, _P, _P, _P, _P, _P]),
    "ds4b200_kv_rows_to_raw_table_f32": (_I, [_P, _L, _I, _I, _P, _P, _F, _P, _P, _P]),
    "ds4b200_kv_rows_to_raw_table_out_f32": (_I, [_P, _L, _I, _I, _P, _RP, _P, _F, _P, _P, _P, _P]),
    "ds4b200_swa_window_push_rows_f32": (_I, [_P, _I, _I, _P, _I, _I, C.POINTER(C.c_int), _P]),
    "ds4b200_swiglu_rows_f32": (_I, [_P, _P, _P, _P, _L, _I, _I, _I, _F, _I, _I, _P]),
    "ds4b200_hc_pre_rows_f32": (_I, [_P, _P, _P, _P, _P, _P, _P, _L, _I, _I, _F, _P]),
    "ds4b200_hc_pre_norm_rows_f32": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _L, _I, _I, _F, _P]),
    "ds4b200_output_hc_head_rows_f32": (_I, [_P, _P, _P, _P, _P, _P, _P, _L, _I, _F, _P]),
    "ds4b200_hc_post_rows_f32": (_I, [_P, _P, _P, _P, _P, _P, _L, _I, _P]),
    "ds4b200_hc_post_pre_rows_f32": (_I, [_P] * 12 + [_L, _I, _I, _F, _P]),
    "ds4b200_hc_sinkhorn_rows_f32": (_I, [_P, _P, _L, _I, _F, _P]),
    "ds4b200_hc_sinkhorn_mix_rows_f32": (_I, [_P, _P, _P, _P, _L, _I, _I, _F, _P]),
    "ds4b200_hc_sinkhorn_mix_rows_static_f32": (_I, [_P, _P, _P, _L, _I, _I, _F, _P]),
    "ds4b200_e4m3_encode_f32": (_I, [_P, _P, _L, _P]),
    "ds4b200_e4m3_decode_f32": (_I, [_P, _P, _L, _P]),
    "ds4b200_e4m3_selfcheck": (_I, [C.c_uint32, C.c_uint64, _P, _P]),
    "ds4b200_layer_rows_f32": (_I, [C.POINTER(LayerDims), C.POINTER(LayerWeights), C.POINTER(LayerBuffers), _P, _P, _L, _P,
                               StageHook, _P, _P]),
    "ds4b200_chunk_rows_f32": (_I, [C.POINTER(LayerDims), C.POINTER(LayerWeights), _I, _I, C.POINTER(LayerBuffers), _P, _P, _P,
                               _L, ChunkHook, _P, _P, C.POINTER(C.c_void_p)]),
    "ds4b200_swiglu_q8_K_rows_f32": (_I, [_P, _P, _P, _P, _P, _P, _P, _L, _I, _I, _I, C.c_float, _I, _P]),
    "ds4b200_swiglu_q8_0_rows_f32": (_I, [_P, _P, _P, _P, _P, _P, _L, _I, _I, _I, _F, _I, _P]),
    "ds4b200_compressor_chunk_f32": (_I, [_I, _P, _P, _P, _P, _I, _I, _I, _L, _I, _P, _P, _P, _P]),
    "ds4b200_compressor_step_f32": (_I, [_I, _P, _P, _P, _P, _I, _I, _I, _I, _P, _P, _P, C.POINTER(C.c_int), _P]),
    "ds4b200_div_selfcheck": (_I, [C.c_uint64, C.c_uint64, _P, _P]),
    # prefill path object (include/ds4b200_path.h)
    "ds4b200_path_create": (_P, [_P]),
    "ds4b200_path_destroy": (None, [_P]),
    "ds4b200_path_upload_table": (_I, [_P, _P, C.c_size_t]),
    "ds4b200_path_check_io": (_I, [_P, _P]),
    "ds4b200_path_upload": (_I, [_P, _P]),
    "ds4b200_path_buffer": (_P, [_P, C.c_char_p, C.POINTER(C.c_int64)]),
    "ds4b200_path_stream": (_P, [_P]),
    "ds4b200_path_run_device": (_I, [_P, _I]),
    "ds4b200_path_run_host": (_I, [_P, _P, _I, C.POINTER(C.c_float)]),
    "ds4b200_path_run_host_chunked": (_I, [_P, _P, _I, _I, C.POINTER(C.c_float)]),
    "ds4b200_path_time_device": (_I, [_P, _I, _I, _I, C.POINTER(C.c_float)]),
    "ds4b200_path_profile_ops": (_I, [_P, _I, C.POINTER(C.c_float)]),
    "ds4b200_path_launches_per_run": (_I, [_P, _I]),
    "ds4b200_path_op_bytes": (_L, [_P, _I]),
}

_lib = None


def load() -> C.CDLL:
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m ds4cuda_b200.build` "
            "(there is no fallback implementation)")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError if the symbol is not exported
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib


class Ds4Error(RuntimeError):
    pass


def check(rc: int) -> None:
    if rc != 0:
        raise Ds4Error(f"ds4b200 error {rc}: {load().ds4b200_last_error().decode()}")
