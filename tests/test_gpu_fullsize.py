"""GPU tests at the benchmark's full sizes (4096 tokens): the CUDA path against
the oracle on sampled tokens, plus size-independent properties over all rows."""
import numpy as np
import pytest
import torch

import inputs
from test_gpu_parity import assert_bits, assert_close, bf16_of, dev, host, to_ops_params

pytestmark = pytest.mark.gpu
T = 4096


def test_config2_embed_residual_norm_full_size(ops, oracle):
    c = inputs.config2(T=T)
    table = dev(c["table"])
    assert table.numel() == 129280 * 128 * 34
    rows, nf, nb = ops.embed_gather_rows(table, ops.TABLE_Q8_0, dev(c["ids"]), 4096, residual=dev(c["residual"]),
                                         norm_w=dev(c["w"]), want_f32=True, want_bf16=True)
    assert ops.device_status() == 0
    pick = np.sort(inputs.rng(20).permutation(T)[:96])
    want_rows, want_nf, _ = oracle.embed_gather_rows(c["table"], oracle.TABLE_Q8_0, c["ids"][pick], 4096,
                                                     residual=c["residual"][pick], norm_w=c["w"])
    assert_bits(host(rows)[pick], want_rows, "residual' rows")
    assert_close(host(nf)[pick], want_nf, what="normed rows")
    assert_bits(host(nb), bf16_of(host(nf)), "bf16 of every row")
    # every row: unit RMS before the gain
    y = host(nf).astype(np.float64) / c["w"]
    assert np.abs((y * y).mean(axis=1) - 1).max() < 1e-4
    # pure gather of the whole batch, bit-exact against numpy's dequantisation
    raw, _, _ = ops.embed_gather_rows(table, ops.TABLE_Q8_0, dev(c["ids"]), 4096)
    blk = c["table"][c["ids"]]
    d = blk[:, :, 0:2].copy().view(np.float16).astype(np.float32)
    q = blk[:, :, 2:].copy().view(np.int8).astype(np.float32)
    assert_bits(host(raw)[:, 0, :], (d * q).reshape(T, 4096), "all 4096 dequantised rows")


def test_config3_rope_fp8_store_full_size(ops, oracle):
    c = inputs.config3(T=T)
    p = oracle.rope_params_explicit(10000.0, 16.0, 4096)
    n_slots = 65536
    codes = torch.zeros((n_slots, 512), dtype=torch.uint8, device="cuda")
    scales = torch.zeros((n_slots, 1), device="cuda")
    rope_out = torch.empty(T, 512, device="cuda")
    ops.rope_fp8_store_rows(dev(c["kv"]), dev(c["pos"]), to_ops_params(ops, p), 64, ops.FP8_ROW_AMAX, codes,
                            scales, slots=dev(c["pos"]), rope_out=rope_out)
    assert not host(codes[T:]).any() and not host(scales[T:]).any()      # slots beyond pos untouched
    r = host(rope_out)
    want_c, want_s, _ = oracle.fp8_encode_rows(r, 64, oracle.FP8_ROW_AMAX)
    assert_bits(host(codes[:T]), want_c, "codes of all 4096 rows from the GPU's rotated rows")
    assert_bits(host(scales[:T]), want_s, "scales of all 4096 rows")
    _, _, _, want_r = oracle.rope_fp8_store_rows(c["kv"], c["pos"], p, 64, oracle.FP8_ROW_AMAX)
    assert_close(r, want_r, what="rotated rows, positions 0..4095")
    # decode -> within half a code step of the rotated row
    deq = host(ops.e4m3_decode(codes[:T])) * host(scales[:T])
    assert (np.abs(deq - r) <= 0.0625 * np.abs(r) + host(scales[:T]) * 2.0 ** -10 + 1e-12).all()
    # the same rows through the reference's scale rule
    codes7 = torch.zeros((n_slots, 512), dtype=torch.uint8, device="cuda")
    scales7 = torch.zeros((n_slots, 7), device="cuda")
    tail = torch.zeros((n_slots, 64), device="cuda")
    ops.rope_fp8_store_rows(dev(c["kv"]), dev(c["pos"]), to_ops_params(ops, p), 64, ops.FP8_BLOCK64_POW2, codes7,
                            scales7, slots=dev(c["pos"]), tail_out=tail)
    c7, s7, t7 = oracle.fp8_encode_rows(r, 64, oracle.FP8_BLOCK64_POW2)
    assert_bits(host(codes7[:T]), c7, "BLOCK64_POW2 codes")
    assert_bits(host(scales7[:T]), s7, "BLOCK64_POW2 scales")
    assert_bits(host(tail[:T]), t7, "f32 tail")


def test_config4_swiglu_combine_full_size(ops, oracle):
    c = inputs.config4(T=T)
    gate, up, w = dev(c["gate"]), dev(c["up"]), dev(c["weights"])
    out = ops.swiglu_rows(gate, up, w, ops.GLU_CLAMP_REF, inputs.CLAMP, combine=True)
    pick = np.sort(inputs.rng(40).permutation(T)[:128])
    want = oracle.swiglu_rows(c["gate"][pick], c["up"][pick], c["weights"][pick], oracle.GLU_CLAMP_REF,
                              inputs.CLAMP, combine=True)
    assert_close(host(out)[pick], want, what="clamped SwiGLU x weights, summed (reference clamp)")
    sym = ops.swiglu_rows(gate, up, w, ops.GLU_CLAMP_SYM, inputs.CLAMP, combine=True)
    want_sym = oracle.swiglu_rows(c["gate"][pick], c["up"][pick], c["weights"][pick], oracle.GLU_CLAMP_SYM,
                                  inputs.CLAMP, combine=True)
    assert_close(host(sym)[pick], want_sym, what="symmetric clamp")
    # linearity in the router weights over the whole batch: doubling them doubles the output exactly
    out2 = ops.swiglu_rows(gate, up, w * 2, ops.GLU_CLAMP_REF, inputs.CLAMP, combine=True)
    assert torch.equal(out2, out * 2)
    # un-combined slots summed in slot order reproduce the combined output exactly
    slots = ops.swiglu_rows(gate, up, w, ops.GLU_CLAMP_REF, inputs.CLAMP, combine=False)
    acc = slots[:, 0].clone()
    for s in range(1, 6):
        acc += slots[:, s]
    assert torch.equal(acc, out)


def test_config5_sinkhorn_mix_full_size(ops, oracle):
    c = inputs.config5(T=T)
    resid, logits = dev(c["resid"]), dev(c["logits"])
    out, comb = ops.hc_sinkhorn_mix_rows(logits, resid, inputs.SINKHORN_ITERS, inputs.EPS, want_comb=True)
    pick = np.sort(inputs.rng(50).permutation(T)[:128])
    want, want_comb = oracle.hc_sinkhorn_mix_rows(c["logits"][pick], c["resid"][pick])
    assert_close(host(comb)[pick], want_comb, what="Sinkhorn matrices")
    assert_close(host(out)[pick], want, what="mixed streams")
    # every token: comb[src + 4*dst] is positive, sums to 1 over dst exactly after the last
    # pass and to 1 over src up to the Sinkhorn residual; the mix reads it as comb[dst + 4*src],
    # so the four outputs add up to the four inputs up to that residual
    cm = host(comb).reshape(T, 4, 4)                       # [t][dst][src]
    assert (cm > 0).all()
    assert np.abs(cm.sum(axis=1) - 1).max() < 1e-5
    assert np.abs(cm.sum(axis=2) - 1).max() < 5e-2
    total_in = resid.double().sum(dim=1)
    total_out = out.double().sum(dim=1)
    assert (total_out - total_in).abs().max().item() < 5e-2 * resid.abs().max().item() * 4


def test_hc_pre_full_token_batch(ops, oracle):
    g = inputs.rng(60)
    Tn = 512
    resid = inputs.normal(g, (Tn, 4, 4096))
    wts = inputs.hc_pre_weights(6, 4096)
    post, comb, out = ops.hc_pre_rows(dev(resid), dev(wts["fn"]), dev(wts["scale"]), dev(wts["base"]))
    pick = np.sort(g.permutation(Tn)[:24])
    wpost, wcomb, wout, _ = oracle.hc_pre_rows(resid[pick], wts["fn"], wts["scale"], wts["base"])
    assert_close(host(post)[pick], wpost, what="post")
    assert_close(host(comb)[pick], wcomb, what="comb")
    assert_close(host(out)[pick], wout, what="out")
