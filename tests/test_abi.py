"""CPU tests of the drop-in boundary: the shared library loads, exports every
symbol the headers declare (C names and the reference's mangled C++ names), and
the checked entry points reject bad arguments before touching the GPU."""
import ctypes as C
import re
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    from ds4cuda_b200 import _lib, build
    build.build()
    return _lib.load()


def _declared(header: str):
    text = (ROOT / "include" / header).read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ds4b200_[A-Za-z0-9_]+)\s*\(", text)))


def test_every_declared_c_symbol_is_exported_and_bound(lib):
    from ds4cuda_b200 import _lib
    names = _declared("ds4b200.h") + _declared("ds4b200_path.h") + _declared("ds4b200_layer.h")
    assert len(names) > 40
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/ but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert set(_lib.SIGNATURES) <= set(names)


def test_reference_cxx_launchers_are_exported_with_reference_signatures():
    """The mangled names the reference's forward_layer.o / forward_token.o import."""
    from ds4cuda_b200 import _lib
    out = subprocess.run(["nm", "-D", "--defined-only", "-C", str(_lib.LIB_PATH)], capture_output=True,
                         text=True, check=True).stdout
    want = [
        "ds4cuda::launch_rms_norm_f32(float const*, float const*, float*, int, float, CUstream_st*)",
        "ds4cuda::launch_rms_norm_batch_f32(float const*, float const*, int, float*, int, int, float, CUstream_st*)",
        "ds4cuda::launch_add_f32(float const*, float const*, float*, int, CUstream_st*)",
        "ds4cuda::launch_tail_rope_yarn_f32(float const*, float*, int, int, int, int, int, CUstream_st*)",
        "ds4cuda::launch_tail_rope_yarn_inverse_f32(float const*, float*, int, int, int, int, int, CUstream_st*)",
        "ds4cuda::launch_fp8_kv_quantize_round_trip_f32(float const*, float*, int, int, int, CUstream_st*)",
        "ds4cuda::launch_silu_mul_f32(float const*, float const*, float*, int, CUstream_st*)",
        "ds4cuda::launch_embed_token_f16_to_f32(unsigned short const*, int, int, float*, CUstream_st*)",
        "ds4cuda::launch_hc_attn_pre_f32(float const*, unsigned short const*, float const*, float const*, float*, float*, float*, int, int, int, float, CUstream_st*)",
        "ds4cuda::launch_hc_attn_pre_v2_f32(float const*, unsigned short const*, float const*, float const*, float*, float*, float*, int, int, int, float, float*, float*, CUstream_st*)",
        "ds4cuda::launch_hc_ffn_pre_v2_f32(float const*, unsigned short const*, float const*, float const*, float*, float*, float*, int, int, int, float, float*, float*, CUstream_st*)",
        "ds4cuda::launch_hc_post_f32(float const*, float const*, float const*, float const*, float*, int, int, CUstream_st*)",
        "ds4cuda::launch_output_hc_head_f32(float const*, unsigned short const*, float const*, float const*, float*, int, int, float, CUstream_st*)",
    ]
    for sig in want:
        assert sig in out, f"missing drop-in symbol: {sig}"


def test_rope_routing_matches_oracle(lib, oracle):
    from ds4cuda_b200 import _lib
    for il in (0, 1, 2, 3, 42):
        a = _lib.RopeParams()
        lib.ds4b200_rope_params_for_layer(il, 64, C.byref(a))
        b = oracle.rope_params_for_layer(il)
        assert a.theta_scale == 0.0                      # evaluated on the device, as the reference does
        for f in ("freq_base", "freq_scale", "ext_factor", "attn_factor", "corr_low", "corr_high"):
            assert getattr(a, f) == getattr(b, f), (il, f)
    a = _lib.RopeParams()
    lib.ds4b200_rope_params_explicit(10000.0, 16.0, 4096, 64, C.byref(a))
    assert bytes(a) == bytes(oracle.rope_params_explicit(10000.0, 16.0, 4096))


def test_path_rejects_out_of_range_ids_and_positions_on_the_host(lib):
    """The prefill path indexes the embedding table with ids and the KV cache with pos; both are
    range-checked while still in host memory, before any copy or launch."""
    import numpy as np
    from ds4cuda_b200._lib import PathConfig, PathIO
    EINVAL = -22
    cfg = PathConfig(n_tokens=8, vocab=100, n_slots=64)
    ids = np.arange(8, dtype=np.int32)
    pos = np.arange(8, dtype=np.int32)
    io = PathIO(ids=ids.ctypes.data, pos=pos.ctypes.data)
    assert lib.ds4b200_path_check_io(C.byref(cfg), C.byref(io)) == 0
    ids[5] = 100
    assert lib.ds4b200_path_check_io(C.byref(cfg), C.byref(io)) == EINVAL
    assert b"ids[5] = 100" in lib.ds4b200_last_error()
    ids[5] = -1
    assert lib.ds4b200_path_check_io(C.byref(cfg), C.byref(io)) == EINVAL
    ids[5] = 99
    pos[7] = 64
    assert lib.ds4b200_path_check_io(C.byref(cfg), C.byref(io)) == EINVAL
    assert b"pos[7] = 64" in lib.ds4b200_last_error()
    pos[7] = 63
    assert lib.ds4b200_path_check_io(C.byref(cfg), C.byref(io)) == 0
    assert lib.ds4b200_path_check_io(C.byref(cfg), C.byref(PathIO())) == 0      # absent arrays: nothing to check
    assert lib.ds4b200_path_check_io(None, C.byref(io)) == EINVAL


def test_checked_entry_points_reject_bad_arguments_without_a_gpu(lib):
    EINVAL = -22
    p = C.c_void_p(0x1000)       # never dereferenced: every call below fails validation first
    assert lib.ds4b200_add_f32(None, p, p, 8, None) == EINVAL
    assert b"null" in lib.ds4b200_last_error()
    assert lib.ds4b200_add_f32(p, p, p, -1, None) == EINVAL
    assert lib.ds4b200_add_f32(None, None, None, 0, None) == 0          # empty input is a no-op
    assert lib.ds4b200_rms_norm_rows_f32(p, None, None, 7, p, None, None, 4, 16, 1e-6, None) == EINVAL
    assert lib.ds4b200_rms_norm_rows_f32(p, None, None, 0, None, None, None, 4, 16, 1e-6, None) == EINVAL
    assert lib.ds4b200_rms_norm_rows_f32(p, None, None, 0, p, None, p, 4, 16, 1e-6, None) == EINVAL
    assert lib.ds4b200_rms_norm_rows_f32(None, None, None, 0, None, None, None, 0, 16, 1e-6, None) == 0
    q = C.c_void_p(0x1000)
    assert lib.ds4b200_rms_norm_q8_K_rows_f32(q, None, None, 0, None, None, None, None, q, q, q, 4, 4000, 1e-6, None) == EINVAL
    assert lib.ds4b200_rms_norm_q8_K_rows_f32(q, None, None, 0, None, None, q, None, q, q, q, 4, 4096, 1e-6, None) == EINVAL
    assert lib.ds4b200_rms_norm_q8_K_rows_f32(q, None, None, 0, None, None, None, None, q, None, q, 4, 4096, 1e-6, None) == EINVAL
    assert lib.ds4b200_rms_norm_q8_K_rows_f32(q, None, None, 0, None, None, None, None, q, q, q, 0, 4096, 1e-6, None) == 0
    assert lib.ds4b200_embed_gather_rows(p, 7, p, 4, 64, None, None, 1e-6, p, 1, None, None, None) == EINVAL
    assert lib.ds4b200_embed_gather_rows(p, 1, p, 4, 48, None, None, 1e-6, p, 1, None, None, None) == EINVAL
    assert lib.ds4b200_embed_gather_rows(p, 0, p, 4, 64, None, None, 1e-6, None, 1, None, None, None) == EINVAL
    from ds4cuda_b200._lib import RopeParams
    rp = RopeParams(10000.0, 0.75, 1.0, 0.0, 1.0, 0.0, 0.0)
    assert lib.ds4b200_rope_rows_f32(p, p, 2, 2, 64, 63, p, C.byref(rp), 0, 0, 1e-6, None) == EINVAL
    assert lib.ds4b200_rope_rows_f32(p, p, 2, 2, 64, 128, p, C.byref(rp), 0, 0, 1e-6, None) == EINVAL
    assert lib.ds4b200_rope_rows_f32(p, p, 2, 2, 64, 32, p, None, 0, 0, 1e-6, None) == EINVAL
    assert lib.ds4b200_fp8_kv_round_trip_rows_f32(p, p, 2, 500, 64, None) == EINVAL
    assert lib.ds4b200_rope_fp8_store_rows(p, 2, 512, 64, p, C.byref(rp), None, 1e-6, 9, None, p, p,
                                           None, None, None) == EINVAL
    assert lib.ds4b200_rope_fp8_store_rows(p, 2, 2048, 64, p, C.byref(rp), None, 1e-6, 1, None, p, p,
                                           None, None, None) == EINVAL
    assert lib.ds4b200_rope_fp8_store_rows(C.c_void_p(0x1004), 2, 512, 64, p, C.byref(rp), None, 1e-6, 1,
                                           None, p, p, None, None, None) == EINVAL
    assert b"alignment" in lib.ds4b200_last_error()
    # the entry points that take the chunk's angle table in place of pos + params
    assert lib.ds4b200_rope_table_rows(None, C.byref(rp), 4, 64, p, None) == EINVAL
    assert lib.ds4b200_rope_rows_table_f32(p, p, 4, 64, 512, 64, None, 0, 0, 1e-6, None) == EINVAL
    assert lib.ds4b200_rope_q8_0_rows_f32(p, None, p, p, 4, 64, 512, 64, None, None, None, 1, 0, 1e-6, None) == EINVAL
    assert lib.ds4b200_rope_fp8_store_rows_table(p, 2, 512, 64, None, None, 1e-6, 1, None, p, p, None, None, None) == EINVAL
    assert lib.ds4b200_rope_fp8_store_rows_table(p, 2, 512, 128, p, None, 1e-6, 1, None, p, p, None, None, None) == EINVAL
    assert b"at most 64" in lib.ds4b200_last_error()
    assert lib.ds4b200_rope_fp8_store_rows_table(p, 2, 512, 64, C.c_void_p(0x1004), None, 1e-6, 1, None, p, p, None, None,
                                                 None) == EINVAL
    assert b"alignment" in lib.ds4b200_last_error()
    assert lib.ds4b200_kv_rows_to_raw_table_f32(p, 2, 512, 64, None, None, 1e-6, None, p, None) == EINVAL
    assert lib.ds4b200_kv_rows_to_raw_table_f32(p, 2, 500, 64, p, None, 1e-6, None, p, None) == EINVAL
    assert lib.ds4b200_kv_rows_to_raw_table_f32(None, 0, 512, 64, None, None, 1e-6, None, None, None) == 0
    assert lib.ds4b200_swiglu_rows_f32(p, p, None, p, 2, 6, 64, 5, 10.0, 1, 0, None) == EINVAL
    assert lib.ds4b200_hc_pre_rows_f32(p, p, p, p, p, p, p, 2, 4098, 20, 1e-6, None) == EINVAL
    assert lib.ds4b200_hc_pre_rows_f32(p, p, p, p, p, p, p, 2, 4096, 0, 1e-6, None) == EINVAL
    assert lib.ds4b200_hc_post_rows_f32(p, None, p, None, p, p, 2, 4096, None) == EINVAL
    assert lib.ds4b200_hc_post_rows_f32(None, p, p, None, p, p, 2, 4096, None) == EINVAL
    assert lib.ds4b200_hc_post_pre_rows_f32(p, None, p, p, p, p, p, p, p, p, p, p, 2, 4096, 20, 1e-6, None) == EINVAL   # out_hc aliases the input
    q2 = C.c_void_p(0x2000)
    assert lib.ds4b200_hc_post_pre_rows_f32(p, None, p, None, p, p, p, p, q2, p, p, q2, 2, 4096, 20, 1e-6, None) == EINVAL   # block without post
    assert lib.ds4b200_hc_post_pre_rows_f32(None, None, p, None, p, p, p, p, q2, p, p, q2, 2, 4096, 0, 1e-6, None) == EINVAL   # iters
    assert lib.ds4b200_hc_post_pre_rows_f32(None, None, p, None, p, p, p, p, q2, p, p, q2, 0, 4096, 20, 1e-6, None) == 0
    assert lib.ds4b200_hc_sinkhorn_mix_rows_f32(None, p, p, None, 2, 4096, 20, 1e-6, None) == EINVAL
    assert lib.ds4b200_swiglu_q8_0_rows_f32(p, p, None, p, p, None, 2, 1, 2000, 0, 0.0, 0, None) == EINVAL   # n % 32
    assert lib.ds4b200_swiglu_q8_0_rows_f32(p, p, None, None, p, None, 2, 1, 2048, 0, 0.0, 0, None) == EINVAL
    assert lib.ds4b200_swiglu_q8_0_rows_f32(p, p, None, p, p, None, 2, 1, 2048, 9, 0.0, 0, None) == EINVAL   # mode
    assert lib.ds4b200_swiglu_q8_0_rows_f32(p, p, None, p, p, None, 0, 1, 2048, 0, 0.0, 0, None) == 0
    assert lib.ds4b200_swiglu_q8_K_rows_f32(p, p, None, p, p, p, None, 2, 6, 2000, 1, 10.0, 1, None) == EINVAL
    assert b"256" in lib.ds4b200_last_error()
    assert lib.ds4b200_swiglu_q8_K_rows_f32(p, p, None, None, p, p, None, 2, 6, 2048, 1, 10.0, 1, None) == EINVAL
    emitted = C.c_int(-1)
    assert lib.ds4b200_compressor_step_f32(1, p, p, p, p, 500, 4, 3, 2, p, p, p, C.byref(emitted), None) == EINVAL
    assert lib.ds4b200_compressor_step_f32(1, p, p, p, p, 512, 4, -1, 2, p, p, p, C.byref(emitted), None) == EINVAL
    assert lib.ds4b200_compressor_step_f32(1, p, None, p, p, 512, 4, 3, 2, p, p, p, C.byref(emitted), None) == EINVAL
    assert emitted.value == -1                                # untouched on a rejected call
    assert lib.ds4b200_compressor_chunk_f32(1, p, p, p, p, 512, 4, 6, 64, 2, p, p, p, None) == EINVAL      # pos0 % 4
    assert b"window boundaries" in lib.ds4b200_last_error()
    assert lib.ds4b200_compressor_chunk_f32(1, p, p, p, p, 512, 4, 8, 62, 2, p, p, p, None) == EINVAL      # T % 4
    assert lib.ds4b200_compressor_chunk_f32(1, p, p, p, p, 512, 4, 8, 0, 2, p, p, p, None) == 0            # empty chunk
    from ds4cuda_b200._lib import LayerBuffers, LayerDims, LayerWeights, StageHook
    hook = StageHook(lambda user, stage, n, stream: 0)
    dims = LayerDims(4096, 64, 512, 64, 1024, 2048, 6, 20, 2, 1, 1e-6, 10.0)
    wts, bufs = LayerWeights(), LayerBuffers()                 # all null
    assert lib.ds4b200_layer_rows_f32(C.byref(dims), C.byref(wts), C.byref(bufs), p, p, 4, p, hook, None, None) == EINVAL
    assert b"null weight or buffer" in lib.ds4b200_last_error()
    assert lib.ds4b200_layer_rows_f32(None, C.byref(wts), C.byref(bufs), p, p, 4, p, hook, None, None) == EINVAL
    bad_dims = LayerDims(4096, 64, 500, 64, 1024, 2048, 6, 20, 2, 1, 1e-6, 10.0)
    assert lib.ds4b200_layer_rows_f32(C.byref(bad_dims), C.byref(wts), C.byref(bufs), p, p, 4, p, hook, None, None) == EINVAL
    assert b"geometry" in lib.ds4b200_last_error()
    from ds4cuda_b200._lib import ChunkHook
    chook = ChunkHook(lambda user, il, stage, n, stream: 0)
    final = C.c_void_p()
    assert lib.ds4b200_chunk_rows_f32(C.byref(dims), C.byref(wts), 2, 0, C.byref(bufs), p, p, p, 4, chook, None, None, C.byref(final)) == EINVAL
    assert b"same buffer" in lib.ds4b200_last_error()
    other = C.c_void_p(0x2000)
    assert lib.ds4b200_chunk_rows_f32(C.byref(dims), C.byref(wts), -1, 0, C.byref(bufs), p, other, p, 4, chook, None, None, None) == EINVAL
    assert lib.ds4b200_chunk_rows_f32(C.byref(dims), C.byref(wts), 2, 0, C.byref(bufs), p, other, p, 4, chook, None, None, None) == EINVAL
    assert b"null weight or buffer" in lib.ds4b200_last_error()          # the first layer's own check
    assert lib.ds4b200_chunk_rows_f32(C.byref(dims), C.byref(wts), 0, 0, C.byref(bufs), p, other, p, 4, chook, None, None, C.byref(final)) == 0
    assert final.value == p.value                                        # no layer: the streams stay where they were
    # optional buffers come in groups: kqv_q with kqv_scale; ffn_kq with ffn_kscale and ffn_kbsums
    a = 0x1000
    full = {n: a for n in LayerBuffers.NAMES}
    all_w = LayerWeights(*[a] * len(LayerWeights.NAMES))
    half = LayerBuffers(**full, kqv_q=a)
    assert lib.ds4b200_layer_rows_f32(C.byref(dims), C.byref(all_w), C.byref(half), p, p, 4, p, hook, None, None) == EINVAL
    assert b"go together" in lib.ds4b200_last_error()
    two_of_three = LayerBuffers(**full, ffn_kq=a, ffn_kbsums=a)
    assert lib.ds4b200_layer_rows_f32(C.byref(dims), C.byref(all_w), C.byref(two_of_three), p, p, 4, p, hook, None, None) == EINVAL
    assert b"ffn_kq, ffn_kscale and ffn_kbsums go together" in lib.ds4b200_last_error()
    lone = LayerBuffers(**full, sh_q=a)
    assert lib.ds4b200_layer_rows_f32(C.byref(dims), C.byref(all_w), C.byref(lone), p, p, 4, p, hook, None, None) == EINVAL
    assert b"sh_q and sh_scale go together" in lib.ds4b200_last_error()
    lone = LayerBuffers(**full, ql_scale=a)
    assert lib.ds4b200_layer_rows_f32(C.byref(dims), C.byref(all_w), C.byref(lone), p, p, 4, p, hook, None, None) == EINVAL
    assert b"ql_q and ql_scale go together" in lib.ds4b200_last_error()
    skewed = LayerBuffers(**{**full, "x_norm": a + 4})
    assert lib.ds4b200_layer_rows_f32(C.byref(dims), C.byref(all_w), C.byref(skewed), p, p, 4, p, hook, None, None) == EINVAL
    assert b"16-byte alignment" in lib.ds4b200_last_error()
    narrow = LayerDims(4096 + 32, 64, 512, 64, 1024, 2048, 6, 20, 2, 1, 1e-6, 10.0)      # not a multiple of 256
    q8k = LayerBuffers(**full, ffn_kq=a, ffn_kscale=a, ffn_kbsums=a)
    assert lib.ds4b200_layer_rows_f32(C.byref(narrow), C.byref(all_w), C.byref(q8k), p, p, 4, p, hook, None, None) == EINVAL
    assert b"Q8_K form of the ffn norm" in lib.ds4b200_last_error()
    assert lib.ds4b200_path_create(None) is None
    from ds4cuda_b200._lib import PathConfig
    bad = PathConfig(n_tokens=0)
    assert lib.ds4b200_path_create(C.byref(bad)) is None
    assert b"geometry" in lib.ds4b200_last_error()


def test_path_create_reports_allocation_or_device_failure_instead_of_crashing(lib):
    """Host-side failure path: without a usable device (this CPU box) or with a request no
    device can hold, path_create returns NULL and says which step failed."""
    from ds4cuda_b200._lib import PathConfig, RopeParams
    cfg = PathConfig(n_tokens=1 << 30, n_embd=8192, vocab=1 << 30, table_dtype=0, kv_dim=1024, n_rot=64,
                     n_slots=1 << 30, ff_dim=4096, top_k=8, max_layers=64, sinkhorn_iters=20, fp8_scale_mode=1,
                     glu_mode=1, glu_fast_exp=0, use_graph=0, eps=1e-6, clamp=10.0,
                     rope=RopeParams(10000.0, 0.75, 1.0, 0.0, 1.0, 0.0, 0.0))
    assert lib.ds4b200_path_create(C.byref(cfg)) is None
    msg = lib.ds4b200_last_error()
    assert b"path_create" in msg and (b"cudaMalloc" in msg or b"cudaStreamCreate" in msg)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from ds4cuda_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(RuntimeError, match="no fallback"):
        _lib.load()


def test_ops_refuse_cpu_tensors():
    import torch
    from ds4cuda_b200 import ops
    with pytest.raises(ValueError, match="CUDA tensors only"):
        ops.add(torch.zeros(4), torch.zeros(4))


import ref_lib  # noqa: E402  (oracle/ is on sys.path through conftest)

REFERENCE = ref_lib.reference_tree() or Path("reference-tree-not-reachable")
CALLERS = ["forward_layer.cu", "forward_token.cu", "forward_batch.cu", "compressor.cu"]
STAR = ("launch_rms_norm_f32", "launch_rms_norm_batch_f32", "launch_add_f32", "launch_tail_rope_yarn_f32",
        "launch_tail_rope_yarn_inverse_f32", "launch_fp8_kv_quantize_round_trip_f32", "launch_silu_mul_f32",
        "launch_embed_token_f16_to_f32", "launch_hc_attn_pre_f32", "launch_hc_attn_pre_v2_f32",
        "launch_hc_ffn_pre_v2_f32", "launch_hc_post_f32", "launch_output_hc_head_f32")


@pytest.mark.skipif(not (REFERENCE / "cuda" / "forward_layer.cu").exists(), reason="reference tree not mounted")
def test_reference_callers_resolve_their_launchers_in_our_library(tmp_path):
    """Compile the reference's own callers (unchanged) and check that every launcher of the
    path they import, by mangled name, is defined by libds4b200.so: the drop-in is link-compatible."""
    from ds4cuda_b200 import _lib, build
    defined = set(subprocess.run(["nm", "-D", "--defined-only", str(_lib.LIB_PATH)], capture_output=True,
                                 text=True, check=True).stdout.split())
    wanted = set()
    for src in CALLERS:
        obj = tmp_path / (src + ".o")
        subprocess.run([build.nvcc(), "-O1", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a",
                        f"-I{REFERENCE}/include", f"-I{REFERENCE}/cuda", "-c", str(REFERENCE / "cuda" / src),
                        "-o", str(obj)], check=True, capture_output=True)
        for line in subprocess.run(["nm", "-u", str(obj)], capture_output=True, text=True, check=True).stdout.split():
            if line.startswith("_ZN7ds4cuda") and any(f"{len(n)}{n}E" in line for n in STAR):
                wanted.add(line)
    assert len(wanted) >= 12, wanted          # every launcher of the path is imported by some caller
    missing = sorted(w for w in wanted if w not in defined)
    assert not missing, f"reference callers import launchers we do not define: {missing}"
