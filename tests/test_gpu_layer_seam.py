"""The batched layer (`ds4b200_layer_rows_f32`) carrying real work at its six hook points, against the
reference's own single-token layer.

Reference side: `ds4_forward_layer` itself (cuda/forward_layer.cu:334-1461), unmodified, called once per
token over a synthetic layer 0 (dense raw-SWA attention, hash router) whose quantised weights live in one
device blob.  Product side: ONE call of `ds4b200_layer_rows_f32` for all T tokens; its hook loops the
reference's single-token launchers per token at the points where the reference calls them — the Q8_0
matvecs (cuda/dense_q8.cu), the raw-SWA flash attention over the growing window (cuda/flash_attn.cu), the
grouped out-projection (cuda/attn_out.cu), the router (cuda/router.cu) and the routed down-projection
(cuda/moe_q2k_sum6.cu).  The routed gate / up dot products exist in the reference only fused with the SwiGLU
tail (cuda/moe_iq2_pair.cu:264-373); the test library restates the dots alone with the same operation order,
and this file first checks that restatement against the fused launcher.

What can be equal and what cannot: the row stages of the product differ from the reference's kernels in the
last bits (other reduction orders); behind seven of them the reference quantises the row to int8 for the next
matvec, so a last-bit difference now and then moves one int8 value by one step, which changes that matvec's
output by a few 1e-4 of its scale and everything behind it for that token.  The test makes that visible
instead of hiding it in a loose tolerance: after every reference token it keeps a copy of the reference's
activation arena, so every intermediate of every token can be compared; at each of the seven quantisation
points it quantises both sides' rows with the product's (bit-exact) quantiser and marks a token whose int8
values differ.  Until a token is marked, every one of its stages must meet the f32 bar (1e-5 of the stage's
largest value); after that only a loose bound holds.  At least half of the tokens must reach the end of the
layer unmarked.  (The first token is marked by construction: its attention sees one KV row, so its output is
a multiple of E4M3 grid values, and `127 * x / amax` of such values is often exactly k + 0.5, a tie that any
last-bit difference in the scale decides the other way.)  Byte-equality is checked where the product promises it (the raw KV rows of unmarked tokens,
the Q8_K blocks of the routed mid rows against the blocks the reference's down-projection quantised for
itself from the same f32 rows).
"""
import ctypes as C

import numpy as np
import pytest
import torch

import inputs

pytestmark = pytest.mark.gpu

N, H, HD, QL, FF, K, NEXP, LOW = 4096, 64, 512, 1024, 2048, 6, 256, 8192
N_EXP_BACKED = 8            # experts with weights behind them; the hash table only names these
VOCAB = 32


def q8_0_blocks(g, n_rows, n_cols):
    """[n_rows][n_cols/32] blocks of {f16 d, int8 qs[32]}; weights ~ unit-variance rows / sqrt(n_cols)."""
    nb = n_cols // 32
    a = np.empty((n_rows, nb), dtype=np.dtype([("d", "<f2"), ("qs", "i1", 32)]))
    a["qs"] = g.integers(-127, 128, (n_rows, nb, 32), dtype=np.int8)
    a["d"] = (g.uniform(0.5, 1.5, (n_rows, nb)) / (73.0 * np.sqrt(n_cols))).astype(np.float16)
    return a


def iq2_xxs_blocks(g, n_exp, n_rows, n_cols):
    """{f16 d, u16 qs[32]}: every bit pattern of qs is a valid code (grid indices, signs, 4-bit scales)."""
    nb = n_cols // 256
    a = np.empty((n_exp, n_rows, nb), dtype=np.dtype([("d", "<f2"), ("qs", "<u2", 32)]))
    a["qs"] = g.integers(0, 65536, (n_exp, n_rows, nb, 32), dtype=np.uint16)
    a["d"] = (g.uniform(0.5, 1.5, (n_exp, n_rows, nb)) * 4e-4).astype(np.float16)
    return a


def q2_k_blocks(g, n_exp, n_rows, n_cols):
    """{u8 scales[16], u8 qs[64], f16 d, f16 dmin}: any bytes are valid codes."""
    nb = n_cols // 256
    a = np.empty((n_exp, n_rows, nb), dtype=np.dtype([("scales", "u1", 16), ("qs", "u1", 64), ("d", "<f2"), ("dmin", "<f2")]))
    a["scales"] = g.integers(0, 256, (n_exp, n_rows, nb, 16), dtype=np.uint8)
    a["qs"] = g.integers(0, 256, (n_exp, n_rows, nb, 64), dtype=np.uint8)
    a["d"] = (g.uniform(0.5, 1.5, (n_exp, n_rows, nb)) * 6e-4).astype(np.float16)
    a["dmin"] = (g.uniform(0.5, 1.5, (n_exp, n_rows, nb)) * 6e-4).astype(np.float16)
    return a


def synthetic_layer(il, seed):
    """name -> numpy array for every tensor ds4_forward_layer looks up on a ratio-0 layer
    (cuda/forward_layer.cu:383-460)."""
    g = inputs.rng(seed)
    wa, wf = inputs.hc_pre_weights(seed + 1, N), inputs.hc_pre_weights(seed + 2, N)
    w = {
        "hc_attn_fn.weight": wa["fn"], "hc_attn_scale.weight": wa["scale"], "hc_attn_base.weight": wa["base"],
        "attn_norm.weight": inputs.uniform(g, (N,), 0.5, 1.5),
        "attn_q_a.weight": q8_0_blocks(g, QL, N),
        "attn_q_a_norm.weight": inputs.uniform(g, (QL,), 0.5, 1.5),
        "attn_kv.weight": q8_0_blocks(g, HD, N),
        "attn_kv_a_norm.weight": inputs.uniform(g, (HD,), 0.5, 1.5),
        "attn_q_b.weight": q8_0_blocks(g, H * HD, QL),
        "attn_sinks.weight": inputs.normal(g, (H,), 0.5),
        "attn_output_a.weight": q8_0_blocks(g, LOW, N),          # 8 groups x 1024 rows, 4096 columns each
        "attn_output_b.weight": q8_0_blocks(g, N, LOW),
        "hc_ffn_fn.weight": wf["fn"], "hc_ffn_scale.weight": wf["scale"], "hc_ffn_base.weight": wf["base"],
        "ffn_norm.weight": inputs.uniform(g, (N,), 0.5, 1.5),
        "ffn_gate_shexp.weight": q8_0_blocks(g, FF, N),
        "ffn_up_shexp.weight": q8_0_blocks(g, FF, N),
        "ffn_down_shexp.weight": q8_0_blocks(g, N, FF),
        "ffn_gate_inp.weight": (g.standard_normal((NEXP, N), dtype=np.float32) / 64.0).astype(np.float16),
        "ffn_gate_tid2eid.weight": np.stack([g.permutation(N_EXP_BACKED)[:K] for _ in range(VOCAB)]).astype(np.int32),
        "ffn_gate_exps.weight": iq2_xxs_blocks(g, N_EXP_BACKED, FF, N),
        "ffn_up_exps.weight": iq2_xxs_blocks(g, N_EXP_BACKED, FF, N),
        "ffn_down_exps.weight": q2_k_blocks(g, N_EXP_BACKED, N, FF),
    }
    return {f"blk.{il}.{k}": np.ascontiguousarray(v) for k, v in w.items()}


class Blob:
    """All tensors in one device buffer at 256-byte aligned offsets; `self[name]` is the device view."""

    def __init__(self, tensors):
        self.names, self.offsets, self.sizes, cur = list(tensors), [], [], 0
        for nm in self.names:
            self.offsets.append(cur)
            self.sizes.append(tensors[nm].nbytes)
            cur += (tensors[nm].nbytes + 255) & ~255
        host = np.zeros(cur, dtype=np.uint8)
        for nm, off in zip(self.names, self.offsets):
            host[off:off + tensors[nm].nbytes] = tensors[nm].reshape(-1).view(np.uint8)
        self.dev = torch.from_numpy(host).cuda()
        self.total = cur

    def __getitem__(self, suffix):
        i = next(i for i, nm in enumerate(self.names) if nm.endswith("." + suffix))
        return self.dev[self.offsets[i]:self.offsets[i] + self.sizes[i]]


def arena_layout():
    """Offsets (in floats) of the intermediates ds4_forward_layer carves from its activation arena on a
    ratio-0 layer, in carve order (cuda/forward_layer.cu:616-797; every carve rounded up to 256 bytes)."""
    order = [("hc_attn_post_w", 4), ("hc_attn_comb", 16), ("hc_attn_pre", N), ("hc_attn_rms", 1), ("hc_attn_mix", 24),
             ("attn_norm", N), ("q_lora", QL), ("q_lora_norm", QL), ("kv_raw", HD), ("kv_norm", HD), ("kv_rope", HD),
             ("kv_cur", HD), ("q_raw", H * HD), ("q_norm", H * HD), ("q_cur", H * HD), ("kqv_out", H * HD),
             ("kqv_back", H * HD), ("attn_low", LOW), ("attn_out", N), ("resid_hc_attn", 4 * N),
             ("hc_ffn_post_w", 4), ("hc_ffn_comb", 16), ("hc_ffn_pre", N), ("hc_ffn_rms", 1), ("hc_ffn_mix", 24),
             ("ffn_norm", N), ("shared_gate", FF), ("shared_up", FF), ("shared_silu", FF), ("ffn_shexp", N),
             ("router_logits", NEXP), ("router_probs", NEXP), ("router_topk_ids", K), ("router_topk_w", K),
             ("routed_mid", K * FF), ("ffn_moe_out", N), ("ffn_out", N)]
    out, cur = {}, 0
    for name, n in order:
        out[name] = (cur // 4, n)
        cur += (4 * n + 255) & ~255
    return out


def rel_err(got, want):
    got, want = got.double().flatten(), want.double().flatten()
    return float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))


@pytest.mark.parametrize("T", [8])
def test_batched_layer_with_reference_matvecs_in_the_hook_against_the_reference_layer(ops, ref, T):
    from ds4cuda_b200 import _lib
    L, R = _lib.load(), ref.lib()
    il = 0
    blob = Blob(synthetic_layer(il, seed=4100))
    g = inputs.rng(4200)
    resid_in = torch.from_numpy(inputs.normal(g, (T, 4, N))).cuda()
    token_ids = [int(v) for v in g.integers(0, VOCAB, T)]
    positions = [100 + t for t in range(T)]
    pos = torch.tensor(positions, dtype=torch.int32, device="cuda")
    f32 = lambda *shape: torch.zeros(*shape, device="cuda")
    i8 = lambda *shape: torch.zeros(*shape, dtype=torch.int8, device="cuda")

    # ------------------------------------------------------------ reference: its own layer, token by token
    R.ds4ref_model_create.restype = C.c_void_p
    R.ds4ref_session_create.restype = C.c_void_p
    R.ds4ref_session_arena.restype = C.c_void_p
    R.ds4ref_session_raw_kv.restype = C.c_void_p
    names = (C.c_char_p * len(blob.names))(*[nm.encode() for nm in blob.names])
    offs = (C.c_uint64 * len(blob.names))(*blob.offsets)
    sizes = (C.c_uint64 * len(blob.names))(*blob.sizes)
    model = C.c_void_p(R.ds4ref_model_create(names, offs, sizes, len(blob.names), C.c_void_p(blob.dev.data_ptr()),
                                             C.c_uint64(blob.total)))
    session = C.c_void_p(R.ds4ref_session_create(256))
    assert model.value and session.value
    want = f32(T, 4, N)
    lay = arena_layout()
    arena = f32(T, sum(((4 * n + 255) & ~255) for _, n in lay.values()) // 4)
    for t in range(T):
        rc = R.ds4ref_forward_layer(model, session, il, token_ids[t], positions[t], C.c_void_p(resid_in[t].data_ptr()),
                                    C.c_void_p(want[t].data_ptr()), None)
        assert rc == 0, f"ds4_forward_layer failed at token {t}"
        # the layer's intermediates for this token, before the next call reuses the arena
        assert R.ds4ref_copy_bytes(C.c_void_p(arena[t].data_ptr()), C.c_void_p(R.ds4ref_session_arena(session)),
                                   C.c_uint64(arena.shape[1] * 4), None) == 0
    torch.cuda.synchronize()
    assert R.ds4ref_session_n_raw(session, il) == T
    ref_window = f32(T, HD)
    assert R.ds4ref_copy_bytes(C.c_void_p(ref_window.data_ptr()), C.c_void_p(R.ds4ref_session_raw_kv(session, il)),
                               C.c_uint64(T * HD * 4), None) == 0
    torch.cuda.synchronize()
    refv = {name: arena[:, o:o + n] for name, (o, n) in lay.items()}       # [T, n] per intermediate

    # ------------------------------------------------------------ product: one batched call, reference launchers in the hook
    B = dict(x=f32(T, N), x_norm=f32(T, N), xq=i8(T, N), xscale=f32(T, N // 32), q_lora=f32(T, QL), q_lora_norm=f32(T, QL),
             kv_raw=f32(T, HD), raw_rows=f32(T, HD), q=f32(T, H, HD), kqv=f32(T, H, HD), attn_out=f32(T, N),
             post=f32(T, 4), comb=f32(T, 16), resid_mid=f32(T, 4, N), sh_gate=f32(T, 1, FF), sh_up=f32(T, 1, FF),
             sh_mid=f32(T, 1, FF), gate=f32(T, K, FF), up=f32(T, K, FF), router_w=f32(T, K), mid_q=i8(T, K, FF),
             mid_scale=f32(T, K, FF // 256), mid_bsums=torch.zeros(T, K, FF // 256, 16, dtype=torch.int16, device="cuda"),
             moe_out=f32(T, N), shexp_out=f32(T, N))
    ffn_kq, ffn_ks = i8(T, N), f32(T, N // 256)                            # the ffn norm's row as Q8_K blocks
    ffn_kb = torch.zeros(T, N // 16, dtype=torch.int16, device="cuda")
    ql_q, ql_s = i8(T, QL), f32(T, QL // 32)                               # the q_a norm's row as Q8_0 blocks
    ref_ffn_k = []                                                         # what the reference's quantiser made of each row
    ref_ql_q = []                                                          # ... for the q_a norm's row (q_b projection)
    ref_sh_q = []                                                          # the same for the shared expert's silu(gate) * up
    sxq, sxs = i8(H * HD), f32(H * HD // 32)                               # Q8_0 scratch of the matvec launchers
    kxq, kxs, kxb = i8(K * FF), f32(K * FF // 256), torch.zeros(K * FF // 256 * 16, dtype=torch.int16, device="cuda")
    window, attn_low = f32(128, HD), f32(T, LOW)
    logits, probs = f32(NEXP), f32(NEXP)
    ids = torch.zeros(T, K, dtype=torch.int32, device="cuda")
    snap = {}

    def matvec(wname, x, y, n_rows, n_cols):
        ref.call("mul_mv_q8_0_q8_0_f32_prealloc", blob[wname], x, y, n_rows, n_cols, sxq, sxs)

    failure = []

    def hook(user, stage, n_tokens, stream):
        try:                       # an exception must not unwind through the C caller
            return stages_of_the_caller(stage, n_tokens)
        except Exception as e:     # noqa: BLE001
            failure.append(e)
            return -5

    def stages_of_the_caller(stage, n_tokens):
        assert n_tokens == T
        if stage == _lib.STAGE_QKV_A:                                      # forward_layer.cu:833, :856
            snap["hc_attn_pre"], snap["attn_norm"] = B["x"].clone(), B["x_norm"].clone()
            snap["post_a"], snap["comb_a"] = B["post"].clone(), B["comb"].clone()
            for t in range(T):
                matvec("attn_q_a.weight", B["x_norm"][t], B["q_lora"][t], QL, N)
                matvec("attn_kv.weight", B["x_norm"][t], B["kv_raw"][t], HD, N)
        elif stage == _lib.STAGE_Q_B:                                      # :879
            for t in range(T):
                matvec("attn_q_b.weight", B["q_lora_norm"][t], B["q"][t], H * HD, QL)
                ref_ql_q.append((sxq[:QL].clone(), sxs[:QL // 32].clone()))     # what its quantiser made of the row
        elif stage == _lib.STAGE_ATTENTION:                                # :950 (push), :1166 (raw-SWA attention)
            snap["q_cur"] = B["q"].clone()
            for t in range(T):
                window[t].copy_(B["raw_rows"][t])
                ref.call("flash_attn_decode_raw_f32", B["q"][t], window, window, blob["attn_sinks.weight"], B["kqv"][t],
                         H, t + 1, HD)
            snap["kqv_out"] = B["kqv"].clone()
        elif stage == _lib.STAGE_ATTN_OUT:                                 # :1190, :1205
            for t in range(T):
                ref.call("mul_mv_q8_0_q8_0_grouped_f32_prealloc", blob["attn_output_a.weight"], B["kqv"][t], attn_low[t],
                         8, N, 1024, sxq, sxs)
                matvec("attn_output_b.weight", attn_low[t], B["attn_out"][t], N, LOW)
        elif stage == _lib.STAGE_FFN_UP:                                   # :1260-1350
            snap["hc_ffn_pre"], snap["ffn_norm"] = B["x"].clone(), B["x_norm"].clone()
            for t in range(T):
                matvec("ffn_gate_shexp.weight", B["x_norm"][t], B["sh_gate"][t], FF, N)
                matvec("ffn_up_shexp.weight", B["x_norm"][t], B["sh_up"][t], FF, N)
                ref.call("mul_mv_f16_f32", blob["ffn_gate_inp.weight"], B["x_norm"][t], logits, NEXP, N)
                ref.call("sqrt_softplus_f32", logits, probs, NEXP)
                ref.call("hash_router_topk_ids_i32", blob["ffn_gate_tid2eid.weight"], token_ids[t], ids[t], K)
                ref.call("hash_router_topk_w_f32", probs, ids[t], B["router_w"][t], K, 1.5, 6.103515625e-5)
                ref.call("test_iq2_pair_dots", blob["ffn_gate_exps.weight"], blob["ffn_up_exps.weight"], B["x_norm"][t],
                         ids[t], B["gate"][t], B["up"][t], K, FF, N, NEXP, kxq, kxs, kxb)
                ref_ffn_k.append((kxq[:N].clone(), kxs[:N // 256].clone(), kxb[:N // 16].clone()))
        elif stage == _lib.STAGE_FFN_DOWN:                                 # :1296, :1416
            # the reference's down-projection takes the f32 mid rows and quantises them itself
            snap["mid"] = ops.swiglu_rows(B["gate"], B["up"], B["router_w"], ops.GLU_CLAMP_REF, 10.0, fast_exp=True)
            for t in range(T):
                matvec("ffn_down_shexp.weight", B["sh_mid"][t], B["shexp_out"][t], N, FF)
                ref_sh_q.append((sxq[:FF].clone(), sxs[:FF // 32].clone()))    # what its quantiser made of the row
                ref.call("routed_moe_q2k_sum6_full_f32_prealloc", blob["ffn_down_exps.weight"], snap["mid"][t], ids[t],
                         B["moe_out"][t], K, N, FF, NEXP, kxq, kxs, kxb)
        return 0

    w_names = dict(hc_attn_fn="hc_attn_fn.weight", hc_attn_scale="hc_attn_scale.weight", hc_attn_base="hc_attn_base.weight",
                   attn_norm="attn_norm.weight", q_a_norm="attn_q_a_norm.weight", kv_a_norm="attn_kv_a_norm.weight",
                   hc_ffn_fn="hc_ffn_fn.weight", hc_ffn_scale="hc_ffn_scale.weight", hc_ffn_base="hc_ffn_base.weight",
                   ffn_norm="ffn_norm.weight")
    dims = _lib.LayerDims(N, H, HD, 64, QL, FF, K, 20, il, 1, 1e-6, 10.0)
    weights = _lib.LayerWeights(*[blob[w_names[nm]].data_ptr() for nm in _lib.LayerWeights.NAMES])
    buffers = _lib.LayerBuffers(*[B[nm].data_ptr() for nm in _lib.LayerBuffers.NAMES], None, None, None,
                                ffn_kq.data_ptr(), ffn_ks.data_ptr(), ffn_kb.data_ptr(), None, None,
                                ql_q.data_ptr(), ql_s.data_ptr())
    got = f32(T, 4, N)
    cb = _lib.StageHook(hook)
    rc = L.ds4b200_layer_rows_f32(C.byref(dims), C.byref(weights), C.byref(buffers), resid_in.data_ptr(), pos.data_ptr(),
                                  T, got.data_ptr(), cb, None, None)
    assert rc == 0, (L.ds4b200_last_error(), failure)
    torch.cuda.synchronize()
    assert ops.device_status() == 0

    # ------------------------------------------------------------ the ffn norm's Q8_K blocks == what the reference's
    # quantiser (inside its routed gate / up launcher) made of the same normalised row, token by token
    for t in range(T):
        rq, rs, rb = ref_ffn_k[t]
        assert torch.equal(ffn_kq[t], rq) and torch.equal(ffn_ks[t], rs) and torch.equal(ffn_kb[t], rb), t

    # ------------------------------------------------------------ the q_a norm's Q8_0 blocks == what the reference's q_b
    # projection quantised for itself from the same row, token by token
    for t in range(T):
        rq, rs = ref_ql_q[t]
        assert torch.equal(ql_q[t], rq) and torch.equal(ql_s[t], rs), t

    # ------------------------------------------------------------ the shared expert's rows as Q8_0 blocks (the fused
    # form of silu(gate) * up) == what the reference's down projection quantised for itself, token by token
    shq, shs, _ = ops.swiglu_q8_0_rows(B["sh_gate"], B["sh_up"])
    for t in range(T):
        rq, rs = ref_sh_q[t]
        assert torch.equal(shq[t, 0], rq) and torch.equal(shs[t, 0], rs), t

    # ------------------------------------------------------------ the routed epilogue's Q8_K blocks == what the reference's
    # down-projection quantised for itself from the same f32 rows (its scratch still holds the last token's)
    t = T - 1
    assert torch.equal(B["mid_q"][t].flatten(), kxq) and torch.equal(B["mid_scale"][t].flatten(), kxs)
    assert torch.equal(B["mid_bsums"][t].flatten(), kxb)

    # ------------------------------------------------------------ the restated dots against the fused reference launcher
    fused_mid = f32(K, FF)
    ref.call("routed_moe_pair_swiglu_full_f32_prealloc", blob["ffn_gate_exps.weight"], blob["ffn_up_exps.weight"],
             B["x_norm"][t], ids[t], B["router_w"][t], fused_mid, K, FF, N, NEXP, 10.0, kxq, kxs, kxb)
    torch.cuda.synchronize()
    dots_err = rel_err(snap["mid"][t], fused_mid)
    n_diff = int((snap["mid"][t] != fused_mid).sum())
    print(f"dots + separate SwiGLU tail vs the reference's fused launcher: {n_diff} of {fused_mid.numel()} values differ, "
          f"max-abs / max {dots_err:.2e}")
    assert n_diff == 0, f"dots + separate SwiGLU tail vs the fused launcher: {n_diff} values differ, {dots_err:.3e}"

    # ------------------------------------------------------------ every stage of every token against the reference's arena
    F32_BAR, LOOSE = 1e-5, 5e-2
    marked = [False] * T                 # token t has had an int8 value move at a quantisation point (its own, or for the
    report, flips = [], []               # attention an earlier token's KV row)

    def stage(name, ours, also_marked=None):
        worst_clean, worst_marked = 0.0, 0.0
        for u in range(T):
            err = rel_err(ours[u], refv[name][u])
            m = marked[u] or (also_marked is not None and also_marked[u])
            if m:
                worst_marked = max(worst_marked, err)
                assert err <= LOOSE, f"{name}, token {u} (behind a moved int8 value): {err:.3e}"
            else:
                worst_clean = max(worst_clean, err)
                assert err <= F32_BAR, f"{name}, token {u}: {err:.3e} > {F32_BAR:.0e}   [{'; '.join(report)}]"
        report.append(f"{name} {worst_clean:.1e}" + (f" ({worst_marked:.1e} marked)" if worst_marked else ""))

    def quantisation_point(name, ours, quantise):
        for u in range(T):
            mine, theirs = quantise(ours[u].contiguous())[0], quantise(refv[name][u].contiguous())[0]
            n_moved = int((mine.flatten() != theirs.flatten()).sum())
            if n_moved:
                flips.append(f"{name}[{u}]: {n_moved}")
                marked[u] = True

    stage("hc_attn_pre", snap["hc_attn_pre"]); stage("attn_norm", snap["attn_norm"])
    quantisation_point("attn_norm", snap["attn_norm"], ops.quantize_q8_0_rows)
    stage("q_lora", B["q_lora"]); stage("q_lora_norm", B["q_lora_norm"]); stage("kv_raw", B["kv_raw"])
    kv_marked = list(marked)
    for u in range(T):                   # the KV rows: byte-equal for unmarked tokens up to single f16 grid steps
        if not kv_marked[u]:
            same = float((window[u] == ref_window[u]).float().mean())
            assert same >= 0.99 and rel_err(window[u], ref_window[u]) <= 2e-3, f"raw KV row {u}: {same:.4f} equal"
    quantisation_point("q_lora_norm", B["q_lora_norm"], ops.quantize_q8_0_rows)
    stage("q_cur", snap["q_cur"])
    window_marked = [any(kv_marked[:u + 1]) for u in range(T)]          # attention reads the rows of earlier tokens
    stage("kqv_out", snap["kqv_out"], window_marked); stage("kqv_back", B["kqv"], window_marked)
    for u in range(T):
        marked[u] = marked[u] or window_marked[u]
    quantisation_point("kqv_back", B["kqv"], ops.quantize_q8_0_rows)
    stage("attn_low", attn_low)
    quantisation_point("attn_low", attn_low, ops.quantize_q8_0_rows)
    stage("attn_out", B["attn_out"]); stage("resid_hc_attn", B["resid_mid"])
    stage("hc_ffn_pre", snap["hc_ffn_pre"]); stage("ffn_norm", snap["ffn_norm"])
    quantisation_point("ffn_norm", snap["ffn_norm"], ops.quantize_q8_0_rows)
    quantisation_point("ffn_norm", snap["ffn_norm"], ops.quantize_q8_K_rows)
    stage("shared_gate", B["sh_gate"]); stage("shared_up", B["sh_up"]); stage("shared_silu", B["sh_mid"])
    stage("router_topk_w", B["router_w"]); stage("routed_mid", snap["mid"])
    assert torch.equal(refv["router_topk_ids"].contiguous().view(torch.int32), ids)
    quantisation_point("shared_silu", B["sh_mid"], ops.quantize_q8_0_rows)
    quantisation_point("routed_mid", snap["mid"], ops.quantize_q8_K_rows)
    stage("ffn_shexp", B["shexp_out"]); stage("ffn_moe_out", B["moe_out"])
    refv["resid_out"] = want.view(T, 4 * N)
    stage("resid_out", got.view(T, 4 * N))
    print("worst error per stage over the tokens (max-abs / max of the stage):", "; ".join(report))
    print("int8 values moved at quantisation points:", "; ".join(flips) if flips else "none")
    print(f"tokens that reached the end of the layer without one: {marked.count(False)} of {T}")
    assert marked.count(False) * 2 >= T, flips

    R.ds4ref_session_destroy(session)
    R.ds4ref_model_destroy(model)
