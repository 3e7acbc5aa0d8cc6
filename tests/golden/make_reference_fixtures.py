"""Generate tests/golden/reference_kernels_config1.npz on a GPU box.

Runs the REFERENCE's own kernels (rebuilt for sm_100a into oracle/_ref by
`make -C oracle ref`) on the seeded single-token inputs of benchmark config 1
and stores their outputs, so that the CPU test suite can pin the oracle against
the real reference without a GPU.  Inputs are not stored: they are regenerated
from the seed, and their SHA-256 digests are stored to detect generator drift.

    python tests/golden/make_reference_fixtures.py [out.npz]
"""
import hashlib
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path[:0] = [str(ROOT), str(ROOT / "oracle"), str(ROOT / "tests")]
import inputs  # noqa: E402
import ref_lib  # noqa: E402


def golden_inputs():
    """Everything the fixture's outputs were computed from (seeded)."""
    c1 = inputs.config1(seed=1)
    g = inputs.rng(77)
    d = dict(c1)
    d["kv"] = inputs.normal(g, (3, 512), 1.5)
    d["kv"][0, :8] = [0.0, -0.0, 1e-9, -1e-9, 448.0, -448.0, 1e-4, 3.0]
    d["kv"][1, :64] = 0.0
    d["f16_table"] = inputs.f16_table(g, 16, 4096)
    d["q8_blocks"] = inputs.q8_0_table(g, 1, 64 * 32)
    d["hc_resid"] = inputs.normal(g, (1, 4, 4096))
    d["hc_block"] = inputs.normal(g, (1, 4096))
    w = inputs.hc_pre_weights(6, 4096)
    d["hc_fn"], d["hc_scale"], d["hc_base"] = w["fn"], w["scale"], w["base"]
    d["add_b"] = inputs.normal(g, (4096,))
    # appended after the first fixture was made: draws above keep their values
    d["head_fn"] = (g.standard_normal((4, 16384), dtype=np.float32) / 128).astype(np.float16)
    d["head_scale"] = inputs.uniform(g, (1,), 0.5, 1.5)
    d["head_base"] = inputs.normal(g, (4,), 0.5)
    d["out_norm_w"] = inputs.uniform(g, (4096,), 0.5, 1.5)
    # streaming compressor, ratio 4, 128 output columns, 8 steps (two windows)
    d["comp_x"] = inputs.normal(g, (8, 256))
    d["comp_w_kv"] = (g.standard_normal((256, 256), dtype=np.float32) / 16).astype(np.float16)
    d["comp_w_gate"] = (g.standard_normal((256, 256), dtype=np.float32) / 8).astype(np.float16)
    d["comp_ape"] = (g.standard_normal((4, 256), dtype=np.float32) / 2).astype(np.float16)
    d["comp_norm_w"] = inputs.uniform(g, (128,), 0.5, 1.5)
    return d


def digest(d):
    return {k: hashlib.sha256(np.ascontiguousarray(v).tobytes()).hexdigest() for k, v in d.items()}


def main(out_path):
    assert ref_lib.available(), "build oracle/_ref first: make -C oracle ref"
    d = golden_inputs()
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    out = {}
    x, w = dev(d["x"][0]), dev(d["w"])
    y = torch.empty_like(x)
    ref_lib.call("rms_norm_f32", x, w, y, 4096, 1e-6)
    out["rms_norm"] = y.cpu().numpy()
    q = dev(d["q"][0])
    yq = torch.empty_like(q)
    ref_lib.call("rms_norm_batch_f32", q, None, 0, yq, 64, 512, 1e-6)
    out["rms_norm_batch_unit"] = yq.cpu().numpy()
    for il, pos in ((0, 9), (0, 1234), (2, 1234), (3, 4095)):
        r, ri = torch.empty_like(q), torch.empty_like(q)
        ref_lib.call("tail_rope_yarn_f32", q, r, 64, 512, 64, pos, il)
        ref_lib.call("tail_rope_yarn_inverse_f32", q, ri, 64, 512, 64, pos, il)
        assert torch.equal(r[:, :448], q[:, :448])
        out[f"rope_tail_il{il}_pos{pos}"] = r[:, 448:].cpu().numpy()
        out[f"rope_inv_tail_il{il}_pos{pos}"] = ri[:, 448:].cpu().numpy()
    gt, up = dev(d["gate"][0, 0]), dev(d["up"][0, 0])
    s = torch.empty_like(gt)
    ref_lib.call("silu_mul_f32", gt, up, s, 2048)
    out["silu_mul"] = s.cpu().numpy()
    a = torch.empty_like(x)
    ref_lib.call("add_f32", x, dev(d["add_b"]), a, 4096)
    out["add"] = a.cpu().numpy()
    kv = dev(d["kv"])
    kvo = torch.empty_like(kv)
    ref_lib.call("fp8_kv_quantize_round_trip_f32", kv, kvo, 3, 512, 64)
    out["fp8_round_trip"] = kvo.cpu().numpy()
    e = torch.empty(4096, device="cuda")
    ref_lib.call("embed_token_f16_to_f32", dev(d["f16_table"]), 11, 4096, e)
    out["embed_f16_row11"] = e.cpu().numpy()
    dq = torch.empty(64 * 32, device="cuda")
    ref_lib.call("dequant_q8_0_to_f32", dev(d["q8_blocks"]), dq, 64)
    out["dequant_q8_0"] = dq.cpu().numpy()
    resid, fn, sc, base = dev(d["hc_resid"]), dev(d["hc_fn"]), dev(d["hc_scale"]), dev(d["hc_base"])
    post, comb, hout = torch.empty(4, device="cuda"), torch.empty(16, device="cuda"), torch.empty(4096, device="cuda")
    scratch = torch.zeros(32, device="cuda")
    ref_lib.call("hc_attn_pre_v2_f32", resid, fn, sc, base, post, comb, hout, 4096, 4, 20, 1e-6, scratch, scratch[8:])
    out["hc_pre_post"], out["hc_pre_comb"], out["hc_pre_out"] = post.cpu().numpy(), comb.cpu().numpy(), hout.cpu().numpy()
    out["hc_pre_mix"] = scratch[8:32].cpu().numpy()
    p1, c1_, o1 = torch.empty(4, device="cuda"), torch.empty(16, device="cuda"), torch.empty(4096, device="cuda")
    ref_lib.call("hc_attn_pre_f32", resid, fn, sc, base, p1, c1_, o1, 4096, 4, 20, 1e-6)
    assert torch.equal(p1, post) and torch.equal(c1_, comb) and torch.equal(o1, hout), "v1 != v2"
    hp = torch.empty(4, 4096, device="cuda")
    ref_lib.call("hc_post_f32", dev(d["hc_block"][0]), resid, post, comb, hp, 4, 4096)
    out["hc_post"] = hp.cpu().numpy()
    ho = torch.empty(4096, device="cuda")
    ref_lib.call("output_hc_head_f32", resid, dev(d["head_fn"]), dev(d["head_scale"]), dev(d["head_base"]), ho,
                 4096, 4, 1e-6)
    hn = torch.empty(4096, device="cuda")
    ref_lib.call("rms_norm_f32", ho, dev(d["out_norm_w"]), hn, 4096, 1e-6)
    out["output_hc_head"], out["output_norm"] = ho.cpu().numpy(), hn.cpu().numpy()
    # the reference's compressor step launcher (cuda/compressor.cu:357-420), attention flavour
    # (FP8 round trip on), layer 2; its two projections are stored too: they are the inputs of
    # everything after them
    width, in_dim, hd = 256, 256, 128
    w_kv, w_gate, ape = dev(d["comp_w_kv"].view(np.int16)), dev(d["comp_w_gate"].view(np.int16)), dev(d["comp_ape"].view(np.int16))
    nw = dev(d["comp_norm_w"])
    s_kv, s_sc = torch.zeros(8, width, device="cuda"), torch.full((8, width), -1.0e30, device="cuda")
    emit, sk, ss = torch.zeros(hd, device="cuda"), torch.empty(width, device="cuda"), torch.empty(width, device="cuda")
    kv_cur, sc_pre, emits = [], [], []
    for pos in range(8):
        xx = dev(d["comp_x"][pos])
        a, b = torch.empty(width, device="cuda"), torch.empty(width, device="cuda")
        ref_lib.call("mul_mv_f16_f32", w_kv, xx, a, width, in_dim)
        ref_lib.call("mul_mv_f16_f32", w_gate, xx, b, width, in_dim)
        kv_cur.append(a.cpu().numpy()); sc_pre.append(b.cpu().numpy())
        ref_lib.call("compressor_decode_step_prealloc", 1, xx, w_kv, w_gate, ape, nw, in_dim, hd, 4, pos, 2,
                     s_kv, s_sc, emit, sk, ss)
        if (pos + 1) % 4 == 0:
            emits.append(emit.cpu().numpy().copy())
    out["comp_kv_cur"], out["comp_sc_pre"] = np.stack(kv_cur), np.stack(sc_pre)
    out["comp_state_kv"], out["comp_state_score"] = s_kv.cpu().numpy(), s_sc.cpu().numpy()
    out["comp_emit"] = np.stack(emits)
    torch.cuda.synchronize()
    meta = {"gpu": torch.cuda.get_device_name(0), "cuda": torch.version.cuda}
    np.savez_compressed(out_path, __digests__=np.array(repr(digest(d))), __meta__=np.array(repr(meta)), **out)
    print("wrote", out_path, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else str(ROOT / "tests" / "golden" / "reference_kernels_config1.npz"))
