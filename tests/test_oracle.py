"""CPU tests of the oracle: known-answer constants the reference states,
independent numpy restatements, and domain properties."""
import math

import numpy as np
import pytest

import inputs


# ---- E4M3FN (cuda/fp8_kv.cu:11-35) -------------------------------------------

def test_e4m3_table_endpoints_and_spot_values(oracle):
    L = oracle.lib()
    assert L.ds4o_e4m3_value(0) == 0.0
    assert L.ds4o_e4m3_value(1) == 1.0 / 512.0          # cuda/fp8_kv.cu:21
    assert L.ds4o_e4m3_value(126) == 448.0              # cuda/fp8_kv.cu:21
    spot = {7: 7 * 2.0 ** -9, 8: 2.0 ** -6, 21: 0.05078125, 42: 0.3125, 63: 1.875, 84: 12.0,
            105: 72.0}
    for i, v in spot.items():
        assert L.ds4o_e4m3_value(i) == v
    vals = [L.ds4o_e4m3_value(i) for i in range(127)]
    assert all(b > a for a, b in zip(vals, vals[1:]))   # strictly increasing table


def test_e4m3_matches_ml_dtypes_table(oracle):
    ml_dtypes = pytest.importorskip("ml_dtypes")
    codes = np.arange(127, dtype=np.uint8)
    want = codes.view(ml_dtypes.float8_e4m3fn).astype(np.float32)
    got = np.array([oracle.lib().ds4o_e4m3_value(int(i)) for i in codes], dtype=np.float32)
    assert np.array_equal(got, want)


def test_e4m3_nearest_ties_to_even_index_and_saturation(oracle):
    L = oracle.lib()
    for i in range(126):
        lo, hi = L.ds4o_e4m3_value(i), L.ds4o_e4m3_value(i + 1)
        mid = np.float32((np.float64(lo) + np.float64(hi)) / 2)
        assert float(mid) * 2 == lo + hi                 # midpoint is exact in f32
        even = i if i % 2 == 0 else i + 1
        assert L.ds4o_e4m3_nearest_index(float(mid)) == even
        assert L.ds4o_e4m3_nearest_index(float(np.nextafter(mid, np.float32(0)))) == i
        assert L.ds4o_e4m3_nearest_index(float(np.nextafter(mid, np.float32(1e9)))) == i + 1
    assert L.ds4o_e4m3_nearest_index(448.0) == 126
    assert L.ds4o_e4m3_nearest_index(1e9) == 126
    assert L.ds4o_e4m3_encode(-0.0) == 0x80 and L.ds4o_e4m3_encode(0.0) == 0
    assert L.ds4o_e4m3_encode(-1e9) == 0xFE


def test_e4m3_encode_matches_ml_dtypes_rne(oracle):
    ml_dtypes = pytest.importorskip("ml_dtypes")
    g = inputs.rng(11)
    x = np.concatenate([inputs.normal(g, 20000, 50.0), inputs.normal(g, 20000, 0.01),
                        np.float32([0.0, -0.0, 448.0, -448.0, 2.0 ** -10, 3 * 2.0 ** -10])])
    x = np.clip(x, -448, 448).astype(np.float32)
    want = x.astype(ml_dtypes.float8_e4m3fn).view(np.uint8)
    got = oracle.e4m3_encode(x)
    assert np.array_equal(got, want)
    back = oracle.e4m3_decode(got)
    assert np.array_equal(back, want.view(ml_dtypes.float8_e4m3fn).astype(np.float32))


# ---- conversions ------------------------------------------------------------------

def test_f16_conversion_exhaustive(oracle):
    L = oracle.lib()
    bits = np.arange(65536, dtype=np.uint16)
    want = bits.view(np.float16).astype(np.float32)
    got = np.array([L.ds4o_f16_to_f32(int(b)) for b in bits], dtype=np.float32)
    ok = np.isnan(want) | (got.view(np.uint32) == want.view(np.uint32))
    assert ok.all()


def test_f32_to_f16_and_bf16_round_to_nearest_even(oracle):
    import torch
    L = oracle.lib()
    g = inputs.rng(12)
    x = np.concatenate([inputs.normal(g, 5000, 3.0), inputs.normal(g, 2000, 1e-6),
                        np.float32([65504.0, 65520.0, 1e-8, 6e-8, 2.0 ** -24, 0.0, -0.0])])
    want16 = x.astype(np.float16).view(np.uint16)
    got16 = np.array([L.ds4o_f32_to_f16(float(v)) for v in x], dtype=np.uint16)
    assert np.array_equal(got16, want16)
    wantb = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    gotb = np.array([L.ds4o_f32_to_bf16(float(v)) for v in x], dtype=np.uint16)
    assert np.array_equal(gotb, wantb)


def test_q8_0_block_is_34_bytes_and_dequant_is_one_multiply(oracle):
    g = inputs.rng(13)
    vocab, n = 64, 256
    table = inputs.q8_0_table(g, vocab, n)
    assert table.shape[-1] == 34                          # cuda/common.cuh:33
    ids = g.integers(0, vocab, 40).astype(np.int32)
    rows, _, _ = oracle.embed_gather_rows(table, oracle.TABLE_Q8_0, ids, n)
    d = table[ids][:, :, 0:2].copy().view(np.float16).astype(np.float32)       # [T, nb, 1]
    q = table[ids][:, :, 2:].copy().view(np.int8).astype(np.float32)           # [T, nb, 32]
    want = (d * q).reshape(len(ids), n)
    assert np.array_equal(rows[:, 0, :].view(np.uint32), want.view(np.uint32))


def test_f16_gather_is_exact_and_replicates(oracle):
    g = inputs.rng(14)
    table = inputs.f16_table(g, 50, 128)
    ids = np.array([0, 49, 7, 7], dtype=np.int32)
    rows, _, _ = oracle.embed_gather_rows(table, oracle.TABLE_F16, ids, 128, n_replicas=4)
    want = table[ids].astype(np.float32)
    for rep in range(4):
        assert np.array_equal(rows[:, rep, :], want)


# ---- RMSNorm / add --------------------------------------------------------------------

def test_rms_norm_against_float64(oracle):
    g = inputs.rng(15)
    x, w, r = inputs.normal(g, (9, 4096)), inputs.uniform(g, (4096,), 0.5, 1.5), inputs.normal(g, (9, 4096))
    y, yb, ro = oracle.rms_norm_rows(x, w, residual=r, want_bf16=True, want_residual=True)
    s = (x + r).astype(np.float64)
    want = s / np.sqrt((s * s).mean(axis=1, keepdims=True) + 1e-6) * w
    assert np.array_equal(ro, x + r)
    assert np.abs(y - want).max() <= 1e-5 * np.abs(want).max()
    import torch
    assert np.array_equal(yb, torch.from_numpy(y).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16))
    y0, _, _ = oracle.rms_norm_rows(x)                    # unit gain
    assert np.abs((y0.astype(np.float64) ** 2).mean(axis=1) - 1).max() < 1e-4
    assert np.array_equal(oracle.add(x, r), x + r)


# ---- RoPE -----------------------------------------------------------------------------------

def test_rope_parameter_anchors(oracle):
    p0 = oracle.rope_params_for_layer(0)
    assert np.float32(p0.theta_scale).view(np.uint32) == 0x3f3ff911
    assert (p0.freq_scale, p0.ext_factor, p0.attn_factor) == (1.0, 0.0, 1.0)
    p2 = oracle.rope_params_for_layer(2)
    assert np.float32(p2.theta_scale).view(np.uint32) == 0x3f300a3a
    assert (p2.freq_scale, p2.ext_factor) == (0.0625, 1.0)
    assert (p2.corr_low, p2.corr_high) == (15.0, 25.0)
    assert np.float32(p2.attn_factor).view(np.uint32) == 0x3f486de1
    p3 = oracle.rope_params_explicit(10000.0, 16.0, 4096)
    assert (p3.corr_low, p3.corr_high) == (10.0, 23.0)
    for il, same_as in ((1, 0), (3, 2), (42, 2)):
        a, b = oracle.rope_params_for_layer(il), oracle.rope_params_for_layer(same_as)
        assert bytes(a) == bytes(b)


def test_rope_prefix_untouched_inverse_undoes_forward_and_norm_is_kept(oracle):
    g = inputs.rng(16)
    x = inputs.normal(g, (5, 3, 512))
    pos = np.array([0, 1, 9, 1234, 4095], dtype=np.int32)
    for il in (0, 2):
        p = oracle.rope_params_for_layer(il)
        y = oracle.rope_rows(x, pos, p)
        assert np.array_equal(y[..., :448], x[..., :448])
        assert np.array_equal(y[0], x[0])                 # pos 0: identity (cos 1, sin 0, mscale 1)
        back = oracle.rope_rows(y, pos, p, inverse=True)
        assert np.abs(back - x).max() < 5e-6
        n0 = np.hypot(x[..., 448::2], x[..., 449::2])
        n1 = np.hypot(y[..., 448::2], y[..., 449::2])
        assert np.abs(n0 - n1).max() < 5e-6


def test_rope_against_float64_angles(oracle):
    g = inputs.rng(17)
    x = inputs.normal(g, (1, 2, 512))
    pos = np.array([1234], dtype=np.int32)
    p = oracle.rope_params_explicit(10000.0, 1.0, 0)
    y = oracle.rope_rows(x, pos, p)
    ts = np.float32(p.theta_scale)
    te = np.float32(1234.0)
    for k in range(32):
        c, s = math.cos(float(te)), math.sin(float(te))
        x0, x1 = x[0, :, 448 + 2 * k].astype(np.float64), x[0, :, 449 + 2 * k].astype(np.float64)
        assert np.abs(y[0, :, 448 + 2 * k] - (x0 * c - x1 * s)).max() < 2e-6
        assert np.abs(y[0, :, 449 + 2 * k] - (x0 * s + x1 * c)).max() < 2e-6
        te = np.float32(te * ts)


# ---- FP8 KV -----------------------------------------------------------------------------------

def test_fp8_round_trip_properties(oracle):
    g = inputs.rng(18)
    kv = inputs.normal(g, (33, 512), 1.5)
    out = oracle.fp8_kv_round_trip_rows(kv)
    assert np.array_equal(out[:, 448:], kv[:, 448:])      # tail copied
    again = oracle.fp8_kv_round_trip_rows(out)
    assert np.array_equal(again, out)                     # idempotent
    blocks = kv[:, :448].reshape(33, 7, 64)
    amax = np.maximum(np.abs(blocks).max(axis=2), 1e-4)
    scale = np.exp2(np.ceil(np.log2(amax / 448.0))).astype(np.float32)
    err = np.abs(out[:, :448].reshape(33, 7, 64) - blocks)
    assert (err <= 0.0625 * np.abs(blocks) + scale[..., None] * 2.0 ** -10 + 1e-12).all()
    codes, scales, tail = oracle.fp8_encode_rows(kv, 64, oracle.FP8_BLOCK64_POW2)
    assert np.array_equal(scales, scale) and np.array_equal(tail, kv[:, 448:])
    deq = oracle.e4m3_decode(codes[:, :448]).reshape(33, 7, 64) * scales[..., None]
    assert np.array_equal(deq.reshape(33, 448), out[:, :448])
    assert not codes[:, 448:].any()


def test_fp8_row_amax_mode_and_slot_scatter(oracle):
    g = inputs.rng(19)
    kv = inputs.normal(g, (8, 512), 1.5)
    kv[3] = 0.0
    slots = np.array([5, 0, 9, 2, 7, 1, 3, 8], dtype=np.int32)
    codes, scales, _ = oracle.fp8_encode_rows(kv, 64, oracle.FP8_ROW_AMAX, n_slots=10, slots=slots)
    want_scale = np.maximum(np.abs(kv).max(axis=1), 1e-4).astype(np.float32) / np.float32(448.0)
    assert np.array_equal(scales[slots, 0], want_scale)
    assert not codes[2].any()                              # all-zero row -> zero codes
    assert not codes[[4, 6]].any() and not scales[[4, 6]].any()   # untouched slots
    deq = oracle.e4m3_decode(codes[slots]).reshape(8, 512) * scales[slots]
    assert np.abs(deq - kv).max() <= np.abs(kv).max() * 0.0625 + 1e-6
    assert (np.abs(deq).max(axis=1)[[0, 1, 2]] > 0).all()


# ---- SwiGLU -------------------------------------------------------------------------------------

def test_swiglu_modes(oracle):
    g = inputs.rng(20)
    gate, up = inputs.normal(g, (3, 6, 64), 8.0), inputs.normal(g, (3, 6, 64), 8.0)
    w = inputs.router_weights(g, 3, 6)
    g64, u64 = gate.astype(np.float64), up.astype(np.float64)
    plain = oracle.swiglu_rows(gate, up)
    want = g64 / (1 + np.exp(-g64)) * u64
    assert np.abs(plain - want).max() <= 1e-5 * np.abs(want).max()
    ref = oracle.swiglu_rows(gate, up, w, oracle.GLU_CLAMP_REF, 10.0)
    gc, uc = np.minimum(g64, 10), np.clip(u64, -10, 10)
    want = gc / (1 + np.exp(-gc)) * uc * w[..., None]
    assert np.abs(ref - want).max() <= 1e-5 * np.abs(want).max()
    sym = oracle.swiglu_rows(gate, up, w, oracle.GLU_CLAMP_SYM, 10.0)
    gs = np.clip(g64, -10, 10)
    want_sym = gs / (1 + np.exp(-gs)) * uc * w[..., None]
    assert np.abs(sym - want_sym).max() <= 1e-5 * np.abs(want_sym).max()
    assert (gate < -10).any() and not np.array_equal(ref, sym)     # the two rules differ
    comb = oracle.swiglu_rows(gate, up, w, oracle.GLU_CLAMP_REF, 10.0, combine=True)
    acc = ref[:, 0].copy()
    for s in range(1, 6):
        acc = acc + ref[:, s]
    assert np.array_equal(comb, acc)                       # slot order 0..5, f32
    off = oracle.swiglu_rows(gate, up, None, oracle.GLU_CLAMP_REF, 0.0)   # clamp <= 1e-6: off
    want_off = g64 / (1 + np.exp(-g64)) * u64
    assert np.abs(off - want_off).max() <= 1e-5 * np.abs(want_off).max()
    big = oracle.swiglu_rows(np.float32([[[-100.0, 100.0, -88.0]]]), np.float32([[[1.0, 1.0, 1.0]]]))
    assert np.isfinite(big).all() and big[0, 0, 1] == 100.0


# ---- hyper-connections ----------------------------------------------------------------------------

def test_sinkhorn_is_doubly_stochastic_and_positive(oracle):
    g = inputs.rng(21)
    for _ in range(20):
        c = oracle.sinkhorn_4x4(inputs.normal(g, 16, 2.0)).reshape(4, 4)     # c[dst][src]
        assert (c > 0).all()
        assert np.abs(c.sum(axis=0) - 1).max() < 1e-5      # last pass normalises columns
        assert np.abs(c.sum(axis=1) - 1).max() < 5e-2   # rows converge more slowly
    one = oracle.sinkhorn_4x4(inputs.normal(g, 16), iters=1).reshape(4, 4)
    assert np.abs(one.sum(axis=0) - 1).max() < 1e-5


def test_hc_pre_and_post_against_float64(oracle):
    g = inputs.rng(22)
    n = 256
    resid = inputs.normal(g, (3, 4, n))
    wts = inputs.hc_pre_weights(6, n)
    post, comb, out, mix = oracle.hc_pre_rows(resid, wts["fn"], wts["scale"], wts["base"])
    x = resid.reshape(3, 4 * n).astype(np.float64)
    rms = 1 / np.sqrt((x * x).mean(axis=1, keepdims=True) + 1e-6)
    mix64 = (x * rms) @ wts["fn"].astype(np.float64).T
    assert np.abs(mix - mix64).max() <= 1e-5 * np.abs(mix64).max()
    sig = lambda z: 1 / (1 + np.exp(-z))
    pre64 = sig(mix64[:, :4] * wts["scale"][0] + wts["base"][:4]) + 1e-6
    post64 = 2 * sig(mix64[:, 4:8] * wts["scale"][1] + wts["base"][4:8])
    assert np.abs(post - post64).max() < 1e-5
    want_out = np.einsum("th,thd->td", pre64, resid.astype(np.float64))
    assert np.abs(out - want_out).max() <= 1e-5 * np.abs(want_out).max()
    for t in range(3):
        v = (mix[t, 8:] * wts["scale"][2] + wts["base"][8:]).astype(np.float32)
        assert np.array_equal(comb[t], oracle.sinkhorn_4x4(v))
    block = inputs.normal(g, (3, n))
    block2 = inputs.normal(g, (3, n))
    o = oracle.hc_post_rows(block, resid, post, comb)
    c = comb.reshape(3, 4, 4).astype(np.float64)           # [t][src][dst] for index dst + 4*src
    want = block[:, None, :].astype(np.float64) * post[:, :, None] + np.einsum(
        "tsd,tsn->tdn", c, resid.astype(np.float64))
    assert np.abs(o - want).max() <= 1e-5 * np.abs(want).max()
    o2 = oracle.hc_post_rows(block, resid, post, comb, block_out2=block2)
    assert np.array_equal(o2, oracle.hc_post_rows(block + block2, resid, post, comb))
    mixed, comb2 = oracle.hc_sinkhorn_mix_rows(mix[:, 8:], resid)
    for t in range(3):
        assert np.array_equal(comb2[t], oracle.sinkhorn_4x4(mix[t, 8:]))
    want_mix = np.einsum("tsd,tsn->tdn", comb2.reshape(3, 4, 4).astype(np.float64),
                         resid.astype(np.float64))
    assert np.abs(mixed - want_mix).max() <= 1e-5 * np.abs(want_mix).max()


def test_fused_kv_chain_equals_its_parts(oracle):
    g = inputs.rng(23)
    kv, w = inputs.normal(g, (6, 512), 1.5), inputs.uniform(g, (512,), 0.5, 1.5)
    pos = np.array([0, 3, 77, 1234, 4094, 4095], dtype=np.int32)
    p = oracle.rope_params_explicit(10000.0, 16.0, 4096)
    codes, scales, tail, rope_out = oracle.rope_fp8_store_rows(kv, pos, p, 64, oracle.FP8_ROW_AMAX, norm_w=w)
    normed, _, _ = oracle.rms_norm_rows(kv, w)
    roped = oracle.rope_rows(normed[:, None, :], pos, p)[:, 0, :]
    assert np.array_equal(rope_out, roped)
    c2, s2, _ = oracle.fp8_encode_rows(roped, 64, oracle.FP8_ROW_AMAX)
    assert np.array_equal(codes, c2) and np.array_equal(scales, s2)


def test_f16_round_and_window_push(oracle):
    g = inputs.rng(24)
    x = inputs.normal(g, 1000, 3.0)
    assert np.array_equal(oracle.f16_round(x), x.astype(np.float16).astype(np.float32))
    assert np.array_equal(oracle.f16_round(oracle.f16_round(x)), oracle.f16_round(x))      # idempotent
    win = np.zeros((8, 16), dtype=np.float32)
    rows = inputs.normal(g, (13, 16))
    w1, n1 = oracle.swa_window_push(win, 0, rows[:5])
    assert n1 == 5 and np.array_equal(w1[:5], oracle.f16_round(rows[:5])) and not w1[5:].any()
    w2, n2 = oracle.swa_window_push(w1, n1, rows[5:])
    assert n2 == 8 and np.array_equal(w2, oracle.f16_round(rows[5:]))                      # the last 8 of 13


def test_activation_quantisers(oracle):
    g = inputs.rng(25)
    x = inputs.normal(g, 2048, 2.0)
    q, s = oracle.quantize_q8_0_rows(x)
    blocks = x.reshape(-1, 32)
    assert np.array_equal(s, (np.abs(blocks).max(axis=1) / np.float32(127.0)).astype(np.float32))
    assert np.abs(q.reshape(-1, 32) * s[:, None] - blocks).max() <= s.max() * 0.5 + 1e-7
    assert (np.abs(q.reshape(-1, 32)).max(axis=1) == 127).all()
    qk, sk, bk = oracle.quantize_q8_K_rows(x)
    assert np.array_equal(bk, qk.reshape(-1, 16).astype(np.int32).sum(axis=1).astype(np.int16))
    assert np.abs(qk.reshape(-1, 256) * sk[:, None] - x.reshape(-1, 256)).max() <= np.abs(sk).max() * 0.5 + 1e-7
    # the element of largest magnitude maps to -127 * sign(scale) ... i.e. q = -127 and scale = -max/127
    k = np.abs(x[:256]).argmax()
    assert qk[k] == -127 and np.isclose(sk[0], -x[k] / 127.0)


# ------------------------------------------------------------------ streaming compressor step

def _compressor_inputs(g, head_dim, ratio, n_steps):
    coff = 2 if ratio == 4 else 1
    width = coff * head_dim
    return dict(
        width=width, rows=8 if ratio == 4 else ratio,
        kv=inputs.normal(g, (n_steps, width)), sc=inputs.normal(g, (n_steps, width), 2.0),
        ape=inputs.normal(g, (ratio, width), 0.5).astype(np.float16).view(np.uint16),
        norm_w=inputs.uniform(g, (head_dim,), 0.5, 1.5))


@pytest.mark.parametrize("head_dim,ratio,is_attn", [(512, 4, 1), (128, 4, 0), (128, 16, 0)])
def test_compressor_step_against_float64(oracle, head_dim, ratio, is_attn):
    g = inputs.rng(900 + head_dim + ratio)
    n_steps = 2 * ratio
    d = _compressor_inputs(g, head_dim, ratio, n_steps)
    width = d["width"]
    p = oracle.rope_params_for_layer(2)
    state_kv = np.zeros((d["rows"], width), dtype=np.float32)
    state_sc = np.full((d["rows"], width), -1.0e30, dtype=np.float32)
    for pos in range(n_steps):
        kv, sc = d["kv"][pos].copy(), d["sc"][pos].copy()
        before_kv, before_sc = state_kv.copy(), state_sc.copy()
        emit = oracle.compressor_step(is_attn, kv, sc, d["ape"], d["norm_w"], head_dim, ratio, pos, p,
                                      state_kv, state_sc)
        ape = d["ape"][pos % ratio].view(np.float16).astype(np.float32)
        np.testing.assert_array_equal(sc, d["sc"][pos] + ape)          # one f32 add, written back
        row = ratio + pos % ratio if ratio == 4 else pos % ratio
        if (pos + 1) % ratio:
            assert emit is None
            np.testing.assert_array_equal(state_kv[row], kv)
            np.testing.assert_array_equal(state_sc[row], sc)
            continue
        # the window closed: rebuild the emit in float64 from the state as it was before the roll
        skv, ssc = before_kv.astype(np.float64), before_sc.astype(np.float64)
        skv[row], ssc[row] = kv, sc
        if ratio == 4:
            scores = np.concatenate([ssc[0:4, :head_dim], ssc[4:8, head_dim:]], axis=0)
            values = np.concatenate([skv[0:4, :head_dim], skv[4:8, head_dim:]], axis=0)
        else:
            scores, values = ssc[:, :head_dim], skv[:, :head_dim]
        w = np.exp(scores - scores.max(axis=0))
        pooled = (w * values).sum(axis=0) / w.sum(axis=0)
        normed = pooled / np.sqrt((pooled ** 2).mean() + 1e-6) * d["norm_w"]
        want = oracle.rope_rows(normed.astype(np.float32)[None, None, :], np.array([pos + 1 - ratio], np.int32), p)[0, 0]
        if is_attn:
            want = oracle.fp8_kv_round_trip_rows(want[None, :])[0]
            n_nope = head_dim - 64
            assert (emit[:n_nope] != want[:n_nope]).mean() < 0.02        # a value on a rounding boundary may flip
            assert np.abs(emit - want).max() <= 0.07 * np.abs(want).max()
            assert np.abs(emit[n_nope:] - want[n_nope:]).max() <= 2e-5 * np.abs(want).max()
        else:
            assert np.abs(emit - want).max() <= 2e-5 * np.abs(want).max()
        if ratio == 4:
            np.testing.assert_array_equal(state_kv[0:4], state_kv[4:8])
            np.testing.assert_array_equal(state_sc[0:4], state_sc[4:8])
