"""The row stages of one layer in the order ds4_forward_layer runs them (cuda/forward_layer.cu:808-1461),
batched over T tokens through the C ABI, against the same chain on the CPU oracle.  The outputs of the
matvec and attention stages in between are seeded stand-ins, the same on both sides."""
import numpy as np
import pytest
import torch

import inputs

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.cpu().numpy()


def close(got, want, rel, what):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    err = np.abs(got - want).max()
    assert err <= rel * np.abs(want).max(), f"{what}: {err:.3e} > {rel * np.abs(want).max():.3e}"


@pytest.mark.parametrize("T", [5, 80])          # 80 tokens: the HC pre steps run on the tensor cores
def test_layer_row_stages_in_forward_order(ops, oracle, T):
    g = inputs.rng(990 + T)
    n, il = 4096, 2
    resid_hc = inputs.normal(g, (T, 4, n))
    wa, wf = inputs.hc_pre_weights(6, n), inputs.hc_pre_weights(7, n)
    w_attn, w_ffn = inputs.uniform(g, (n,), 0.5, 1.5), inputs.uniform(g, (n,), 0.5, 1.5)
    w_qa, w_kva = inputs.uniform(g, (1024,), 0.5, 1.5), inputs.uniform(g, (512,), 0.5, 1.5)
    pos = (100 + np.arange(T)).astype(np.int32)
    # stand-ins for what the matvecs and the attention hand to the next row stage
    q_lora, kv_raw = inputs.normal(g, (T, 1024)), inputs.normal(g, (T, 512), 1.5)
    q_raw, kqv = inputs.normal(g, (T, 64, 512)), inputs.normal(g, (T, 64, 512))
    attn_out, moe_out, shexp = inputs.normal(g, (T, n)), inputs.normal(g, (T, n)), inputs.normal(g, (T, n))
    sh_gate, sh_up = inputs.normal(g, (T, 1, 2048), 2.0), inputs.normal(g, (T, 1, 2048), 2.0)
    gate, up = inputs.normal(g, (T, 6, 2048), 2.0), inputs.normal(g, (T, 6, 2048), 2.0)
    w_r = inputs.router_weights(g, T, 6)
    p_o = oracle.rope_params_for_layer(il)
    p_d = ops.rope_params_for_layer(il)

    # ---- device chain
    post_a, comb_a, x = ops.hc_pre_rows(dev(resid_hc), dev(wa["fn"]), dev(wa["scale"]), dev(wa["base"]))
    xn, _, xq, xs = ops.rms_norm_q8_0_rows(x, dev(w_attn))
    qn, _, _ = ops.rms_norm_rows(dev(q_lora), dev(w_qa))
    raw = torch.zeros(T, 512, device="cuda")
    ops.kv_rows_to_raw(dev(kv_raw), dev(pos), p_d, raw, norm_w=dev(w_kva))
    q_cur = ops.rope_rows(dev(q_raw), dev(pos), p_d, unit_rms=True)
    kqv_back = ops.rope_rows(dev(kqv), dev(pos), p_d, inverse=True)
    resid_attn = ops.hc_post_rows(dev(attn_out), dev(resid_hc), post_a, comb_a)
    post_f, comb_f, xf = ops.hc_pre_rows(resid_attn, dev(wf["fn"]), dev(wf["scale"]), dev(wf["base"]))
    xfn, _, _, _ = ops.rms_norm_q8_0_rows(xf, dev(w_ffn))
    sh = ops.swiglu_rows(dev(sh_gate), dev(sh_up))
    mq, ms, mb, mid = ops.swiglu_q8_K_rows(dev(gate), dev(up), dev(w_r), ops.GLU_CLAMP_REF, 10.0, want_f32=True)
    out_hc = ops.hc_post_rows(dev(moe_out), resid_attn, post_f, comb_f, block_out2=dev(shexp))
    torch.cuda.synchronize()
    assert ops.device_status() == 0

    # ---- the same chain on the oracle, from the same first inputs
    o_post_a, o_comb_a, o_x, _ = oracle.hc_pre_rows(resid_hc, wa["fn"], wa["scale"], wa["base"])
    o_xn = oracle.rms_norm_rows(o_x, w_attn)[0]
    o_qn = oracle.rms_norm_rows(q_lora, w_qa)[0]
    o_q = oracle.rope_rows(q_raw, pos, p_o, unit_rms=True)
    o_back = oracle.rope_rows(kqv, pos, p_o, inverse=True)
    o_resid_attn = oracle.hc_post_rows(attn_out, resid_hc, o_post_a, o_comb_a)
    o_post_f, o_comb_f, o_xf, _ = oracle.hc_pre_rows(o_resid_attn, wf["fn"], wf["scale"], wf["base"])
    o_xfn = oracle.rms_norm_rows(o_xf, w_ffn)[0]
    o_sh = oracle.swiglu_rows(sh_gate, sh_up)
    o_mid = oracle.swiglu_rows(gate, up, w_r, oracle.GLU_CLAMP_REF, 10.0, False)
    o_out = oracle.hc_post_rows(moe_out, o_resid_attn, o_post_f, o_comb_f, block_out2=shexp)

    close(host(x), o_x, 1e-5, "hc_attn_pre out")
    close(host(xn), o_xn, 1e-5, "attn_norm")
    close(host(qn), o_qn, 1e-5, "q_a_norm")
    close(host(q_cur), o_q, 2e-5, "q_norm + RoPE")
    close(host(kqv_back), o_back, 2e-5, "inverse RoPE")
    close(host(resid_attn), o_resid_attn, 1e-5, "hc_attn_post")
    close(host(xf), o_xf, 2e-5, "hc_ffn_pre out (second hop of the chain)")
    close(host(xfn), o_xfn, 2e-5, "ffn_norm")
    close(host(sh), o_sh, 1e-5, "shared silu*up")
    close(host(mid), o_mid, 1e-5, "routed epilogue rows")
    close(host(out_hc), o_out, 2e-5, "residual streams after the layer")
    # integer outputs are exact on the device's own f32 rows
    wq, ws = oracle.quantize_q8_0_rows(host(xn))
    assert np.array_equal(host(xq).ravel(), wq) and np.array_equal(host(xs).ravel(), ws.ravel())
    kq, ks, kb = oracle.quantize_q8_K_rows(host(mid).ravel())
    assert np.array_equal(host(mq).ravel(), kq) and np.array_equal(host(ms).ravel(), ks)
    assert np.array_equal(host(mb).ravel(), kb.ravel())
    # raw KV rows are f16-representable and agree with the oracle chain up to single grid steps
    o_raw = oracle.kv_rows_to_raw(kv_raw, pos, p_o, norm_w=w_kva)
    got_raw = host(raw)
    assert np.array_equal(oracle.f16_round(got_raw), got_raw)
    assert (got_raw != o_raw).mean() < 5e-3 and np.abs(got_raw - o_raw).max() <= 0.07 * np.abs(o_raw).max()


def test_layer_rows_entry_point_sequences_the_same_chain(ops):
    """ds4b200_layer_rows_f32 with a hook that supplies the stand-ins == the same stages called one by one."""
    import ctypes as C
    from ds4cuda_b200 import _lib
    L = _lib.load()
    T, n, H, hd, ql, ff, k, il = 70, 4096, 64, 512, 1024, 2048, 6, 2
    g = inputs.rng(995)
    resid_hc = dev(inputs.normal(g, (T, 4, n)))
    wa, wf = inputs.hc_pre_weights(6, n), inputs.hc_pre_weights(7, n)
    W = dict(hc_attn_fn=dev(wa["fn"]), hc_attn_scale=dev(wa["scale"]), hc_attn_base=dev(wa["base"]),
             attn_norm=dev(inputs.uniform(g, (n,), 0.5, 1.5)), q_a_norm=dev(inputs.uniform(g, (ql,), 0.5, 1.5)),
             kv_a_norm=dev(inputs.uniform(g, (hd,), 0.5, 1.5)), hc_ffn_fn=dev(wf["fn"]),
             hc_ffn_scale=dev(wf["scale"]), hc_ffn_base=dev(wf["base"]), ffn_norm=dev(inputs.uniform(g, (n,), 0.5, 1.5)))
    pos = dev((100 + np.arange(T)).astype(np.int32))
    S = dict(q_lora=dev(inputs.normal(g, (T, ql))), kv_raw=dev(inputs.normal(g, (T, hd), 1.5)),
             q=dev(inputs.normal(g, (T, H, hd))), kqv=dev(inputs.normal(g, (T, H, hd))),
             attn_out=dev(inputs.normal(g, (T, n))), sh_gate=dev(inputs.normal(g, (T, 1, ff), 2.0)),
             sh_up=dev(inputs.normal(g, (T, 1, ff), 2.0)), gate=dev(inputs.normal(g, (T, k, ff), 2.0)),
             up=dev(inputs.normal(g, (T, k, ff), 2.0)), router_w=dev(inputs.router_weights(g, T, k)),
             moe_out=dev(inputs.normal(g, (T, n))), shexp_out=dev(inputs.normal(g, (T, n))))
    f32 = lambda *shape: torch.zeros(*shape, device="cuda")
    B = dict(x=f32(T, n), x_norm=f32(T, n), xq=torch.zeros(T, n, dtype=torch.int8, device="cuda"), xscale=f32(T, n // 32),
             q_lora=f32(T, ql), q_lora_norm=f32(T, ql), kv_raw=f32(T, hd), raw_rows=f32(T, hd), q=f32(T, H, hd),
             kqv=f32(T, H, hd), attn_out=f32(T, n), post=f32(T, 4), comb=f32(T, 16), resid_mid=f32(T, 4, n),
             sh_gate=f32(T, 1, ff), sh_up=f32(T, 1, ff), sh_mid=f32(T, 1, ff), gate=f32(T, k, ff), up=f32(T, k, ff),
             router_w=f32(T, k), mid_q=torch.zeros(T, k, ff, dtype=torch.int8, device="cuda"),
             mid_scale=f32(T, k, ff // 256), mid_bsums=torch.zeros(T, k, ff // 256, 16, dtype=torch.int16, device="cuda"),
             moe_out=f32(T, n), shexp_out=f32(T, n))
    fills = {_lib.STAGE_QKV_A: ("q_lora", "kv_raw"), _lib.STAGE_Q_B: ("q",), _lib.STAGE_ATTENTION: ("kqv",),
             _lib.STAGE_ATTN_OUT: ("attn_out",), _lib.STAGE_FFN_UP: ("sh_gate", "sh_up", "gate", "up", "router_w"),
             _lib.STAGE_FFN_DOWN: ("moe_out", "shexp_out")}
    seen, snap = [], {}

    def hook(user, stage, n_tokens, stream):
        seen.append(stage)
        if stage == _lib.STAGE_QKV_A:
            snap["x_norm"], snap["xq"] = B["x_norm"].clone(), B["xq"].clone()    # the attention half's, before reuse
        for name in fills[stage]:
            B[name].copy_(S[name])
        return 0

    dims = _lib.LayerDims(n, H, hd, 64, ql, ff, k, 20, il, 1, 1e-6, 10.0)
    weights = _lib.LayerWeights(*[W[nm].data_ptr() for nm in _lib.LayerWeights.NAMES])
    buffers = _lib.LayerBuffers(*[B[nm].data_ptr() for nm in _lib.LayerBuffers.NAMES])
    out = torch.zeros(T, 4, n, device="cuda")
    cb = _lib.StageHook(hook)
    rc = L.ds4b200_layer_rows_f32(C.byref(dims), C.byref(weights), C.byref(buffers), resid_hc.data_ptr(),
                                  pos.data_ptr(), T, out.data_ptr(), cb, None, None)
    assert rc == 0, L.ds4b200_last_error()
    torch.cuda.synchronize()
    assert seen == list(range(6))

    # ---- the same stages one by one
    p = ops.rope_params_for_layer(il)
    post_a, comb_a, x = ops.hc_pre_rows(resid_hc, W["hc_attn_fn"], W["hc_attn_scale"], W["hc_attn_base"])
    xn, _, xq, _ = ops.rms_norm_q8_0_rows(x, W["attn_norm"])
    qn, _, _ = ops.rms_norm_rows(S["q_lora"], W["q_a_norm"])
    raw = torch.zeros(T, hd, device="cuda")
    ops.kv_rows_to_raw(S["kv_raw"], pos, p, raw, norm_w=W["kv_a_norm"])
    q_cur = ops.rope_rows(S["q"], pos, p, unit_rms=True)
    kqv_back = ops.rope_rows(S["kqv"], pos, p, inverse=True)
    resid_attn = ops.hc_post_rows(S["attn_out"], resid_hc, post_a, comb_a)
    post_f, comb_f, xf = ops.hc_pre_rows(resid_attn, W["hc_ffn_fn"], W["hc_ffn_scale"], W["hc_ffn_base"])
    xfn, _, xfq, _ = ops.rms_norm_q8_0_rows(xf, W["ffn_norm"])
    sh = ops.swiglu_rows(S["sh_gate"], S["sh_up"])
    mq, ms, mb, _ = ops.swiglu_q8_K_rows(S["gate"], S["up"], S["router_w"], ops.GLU_CLAMP_REF, 10.0, fast_exp=True)
    want = ops.hc_post_rows(S["moe_out"], resid_attn, post_f, comb_f, block_out2=S["shexp_out"])
    torch.cuda.synchronize()
    def eq(a, b, what):
        if not torch.equal(a, b):
            where = (a != b).nonzero()
            pytest.fail(f"{what} differs at {where.shape[0]} of {a.numel()} places, first {where[:4].tolist()}: "
                        f"{a[tuple(where[0])].item()!r} against {b[tuple(where[0])].item()!r}")
    eq(snap["x_norm"], xn, "attn norm"); eq(snap["xq"], xq, "attn norm Q8_0")
    eq(B["q_lora_norm"], qn, "q_a norm"); eq(B["raw_rows"], raw, "raw KV rows")
    eq(B["q"], q_cur, "q norm + RoPE"); eq(B["kqv"], kqv_back, "inverse RoPE")
    eq(B["resid_mid"], resid_attn, "hc attn post"); eq(B["x_norm"], xfn, "ffn norm"); eq(B["xq"], xfq, "ffn norm Q8_0")
    eq(B["sh_mid"], sh, "shared silu*up"); eq(B["mid_q"], mq, "routed epilogue Q8_K values")
    eq(B["mid_scale"], ms, "routed epilogue Q8_K scales"); eq(B["mid_bsums"], mb, "routed epilogue Q8_K sums")
    eq(out, want, "residual streams after the layer")

    # ---- with the optional Q8_0 buffers the inverse RoPE leaves the out-projection's activation blocks and
    # does not rewrite kqv; everything else is unchanged
    kq = torch.zeros(T, H, hd, dtype=torch.int8, device="cuda")
    ks = torch.zeros(T, H, hd // 32, device="cuda")
    cs = torch.zeros(T, 32, 2, device="cuda")       # and the angle table: same bits in every RoPE stage
    qlq = torch.zeros(T, ql, dtype=torch.int8, device="cuda")     # the q_a norm's row as Q8_0 blocks
    qls = torch.zeros(T, ql // 32, device="cuda")
    shq = torch.zeros(T, ff, dtype=torch.int8, device="cuda")     # the shared expert's rows as Q8_0 blocks, no f32
    shs = torch.zeros(T, ff // 32, device="cuda")
    fkq = torch.zeros(T, n, dtype=torch.int8, device="cuda")      # and the ffn norm's row as Q8_K blocks
    fks, fkb = torch.zeros(T, n // 256, device="cuda"), torch.zeros(T, n // 16, dtype=torch.int16, device="cuda")
    buffers_q = _lib.LayerBuffers(*[B[nm].data_ptr() for nm in _lib.LayerBuffers.NAMES], kq.data_ptr(), ks.data_ptr(),
                                  cs.data_ptr(), fkq.data_ptr(), fks.data_ptr(), fkb.data_ptr(), shq.data_ptr(),
                                  shs.data_ptr(), qlq.data_ptr(), qls.data_ptr())
    out_q = torch.zeros(T, 4, n, device="cuda")
    B["sh_mid"].fill_(-7.0)                          # must stay untouched when the Q8_0 form is asked for
    rc = L.ds4b200_layer_rows_f32(C.byref(dims), C.byref(weights), C.byref(buffers_q), resid_hc.data_ptr(),
                                  pos.data_ptr(), T, out_q.data_ptr(), cb, None, None)
    assert rc == 0, L.ds4b200_last_error()
    torch.cuda.synchronize()
    wq, ws = ops.quantize_q8_0_rows(kqv_back)
    eq(kq.view(-1), wq.view(-1), "inverse RoPE Q8_0 values"); eq(ks.view(-1), ws.view(-1), "inverse RoPE Q8_0 scales")
    eq(B["kqv"], S["kqv"], "kqv left as the attention stage wrote it"); eq(out_q, want, "residual streams (Q8_0 form)")
    eq(B["q"], q_cur, "q norm + RoPE from the table"); eq(B["raw_rows"], raw, "raw KV rows from the table")
    eq(cs, ops.rope_table_rows(pos, p), "angle table")
    wlq, wls = ops.quantize_q8_0_rows(qn)
    eq(qlq.view(-1), wlq.view(-1), "q_a norm Q8_0 values"); eq(qls.view(-1), wls.view(-1), "q_a norm Q8_0 scales")
    eq(B["q_lora_norm"], qn, "q_a norm beside its Q8_0 form")
    wsq, wss = ops.quantize_q8_0_rows(sh)
    eq(shq.view(-1), wsq.view(-1), "shared silu*up Q8_0 values"); eq(shs.view(-1), wss.view(-1), "shared silu*up Q8_0 scales")
    assert bool((B["sh_mid"] == -7.0).all()), "sh_mid rewritten beside its Q8_0 form"
    wkq, wks, wkb = ops.quantize_q8_K_rows(xfn)
    eq(fkq, wkq, "ffn norm Q8_K values"); eq(fks.view(-1), wks, "ffn norm Q8_K scales")
    eq(fkb.view(-1), wkb, "ffn norm Q8_K sums"); eq(B["x_norm"], xfn, "ffn norm beside its Q8_K form")
    eq(B["xq"], xfq, "ffn norm Q8_0 beside its Q8_K form")

    # a hook that fails stops the layer with its code
    bad = _lib.StageHook(lambda user, stage, n_tokens, stream: -7 if stage == _lib.STAGE_Q_B else 0)
    assert L.ds4b200_layer_rows_f32(C.byref(dims), C.byref(weights), C.byref(buffers), resid_hc.data_ptr(),
                                    pos.data_ptr(), T, out.data_ptr(), bad, None, None) == -7
    assert b"stage 1" in L.ds4b200_last_error()
    torch.cuda.synchronize()


def test_chunk_rows_runs_the_layers_in_turn(ops):
    """ds4b200_chunk_rows_f32 over three layers (indices 1..3: both RoPE parameter sets) == three calls of
    ds4b200_layer_rows_f32 with the streams handed from one to the next; the hook sees (layer, stage)."""
    import ctypes as C
    from ds4cuda_b200 import _lib
    L = _lib.load()
    T, n, H, hd, ql, ff, k = 70, 4096, 64, 512, 1024, 2048, 6
    n_layers, first = 3, 1
    g = inputs.rng(996)
    resid0 = dev(inputs.normal(g, (T, 4, n)))
    pos = dev((200 + np.arange(T)).astype(np.int32))
    per_layer = []
    for i in range(n_layers):
        wa, wf = inputs.hc_pre_weights(20 + 2 * i, n), inputs.hc_pre_weights(21 + 2 * i, n)
        per_layer.append(dict(hc_attn_fn=dev(wa["fn"]), hc_attn_scale=dev(wa["scale"]), hc_attn_base=dev(wa["base"]),
                              attn_norm=dev(inputs.uniform(g, (n,), 0.5, 1.5)), q_a_norm=dev(inputs.uniform(g, (ql,), 0.5, 1.5)),
                              kv_a_norm=dev(inputs.uniform(g, (hd,), 0.5, 1.5)), hc_ffn_fn=dev(wf["fn"]),
                              hc_ffn_scale=dev(wf["scale"]), hc_ffn_base=dev(wf["base"]),
                              ffn_norm=dev(inputs.uniform(g, (n,), 0.5, 1.5))))
    # stand-ins for what the caller's matvecs / attention would write, one set per layer
    shapes = dict(q_lora=(T, ql), kv_raw=(T, hd), q=(T, H, hd), kqv=(T, H, hd), attn_out=(T, n), sh_gate=(T, 1, ff),
                  sh_up=(T, 1, ff), gate=(T, k, ff), up=(T, k, ff), moe_out=(T, n), shexp_out=(T, n))
    S = [{nm: dev(inputs.normal(g, shp)) for nm, shp in shapes.items()} for _ in range(n_layers)]
    for s in S:
        s["router_w"] = dev(inputs.router_weights(g, T, k))
    f32 = lambda *shape: torch.zeros(*shape, device="cuda")
    B = dict(x=f32(T, n), x_norm=f32(T, n), xq=torch.zeros(T, n, dtype=torch.int8, device="cuda"), xscale=f32(T, n // 32),
             q_lora=f32(T, ql), q_lora_norm=f32(T, ql), kv_raw=f32(T, hd), raw_rows=f32(T, hd), q=f32(T, H, hd),
             kqv=f32(T, H, hd), attn_out=f32(T, n), post=f32(T, 4), comb=f32(T, 16), resid_mid=f32(T, 4, n),
             sh_gate=f32(T, 1, ff), sh_up=f32(T, 1, ff), sh_mid=f32(T, 1, ff), gate=f32(T, k, ff), up=f32(T, k, ff),
             router_w=f32(T, k), mid_q=torch.zeros(T, k, ff, dtype=torch.int8, device="cuda"),
             mid_scale=f32(T, k, ff // 256), mid_bsums=torch.zeros(T, k, ff // 256, 16, dtype=torch.int16, device="cuda"),
             moe_out=f32(T, n), shexp_out=f32(T, n))
    fills = {_lib.STAGE_QKV_A: ("q_lora", "kv_raw"), _lib.STAGE_Q_B: ("q",), _lib.STAGE_ATTENTION: ("kqv",),
             _lib.STAGE_ATTN_OUT: ("attn_out",), _lib.STAGE_FFN_UP: ("sh_gate", "sh_up", "gate", "up", "router_w"),
             _lib.STAGE_FFN_DOWN: ("moe_out", "shexp_out")}

    def fill(layer, stage):
        for name in fills[stage]:
            B[name].copy_(S[layer][name])

    buffers = _lib.LayerBuffers(*[B[nm].data_ptr() for nm in _lib.LayerBuffers.NAMES])
    W = (_lib.LayerWeights * n_layers)(*[_lib.LayerWeights(*[w[nm].data_ptr() for nm in _lib.LayerWeights.NAMES])
                                        for w in per_layer])
    # layer by layer
    cur, nxt = resid0.clone(), torch.zeros_like(resid0)
    raws = []
    for i in range(n_layers):
        dims = _lib.LayerDims(n, H, hd, 64, ql, ff, k, 20, first + i, 1, 1e-6, 10.0)
        cb = _lib.StageHook(lambda user, stage, n_tokens, stream, i=i: fill(i, stage) or 0)
        rc = L.ds4b200_layer_rows_f32(C.byref(dims), C.byref(W[i]), C.byref(buffers), cur.data_ptr(), pos.data_ptr(), T,
                                      nxt.data_ptr(), cb, None, None)
        assert rc == 0, L.ds4b200_last_error()
        raws.append(B["raw_rows"].clone())
        cur, nxt = nxt, cur
    want = cur.clone()
    # the same through one call
    a, b = resid0.clone(), torch.zeros_like(resid0)
    seen, raws2 = [], []

    def chook(user, il, stage, n_tokens, stream):
        seen.append((il, stage))
        if stage == _lib.STAGE_Q_B:
            raws2.append(B["raw_rows"].clone())
        fill(il - first, stage)
        return 0

    dims = _lib.LayerDims(n, H, hd, 64, ql, ff, k, 20, 99, 1, 1e-6, 10.0)       # il is taken from the loop, not from here
    final = C.c_void_p()
    cb2 = _lib.ChunkHook(chook)
    rc = L.ds4b200_chunk_rows_f32(C.byref(dims), W, n_layers, first, C.byref(buffers), a.data_ptr(), b.data_ptr(),
                                  pos.data_ptr(), T, cb2, None, None, C.byref(final))
    assert rc == 0, L.ds4b200_last_error()
    torch.cuda.synchronize()
    assert seen == [(first + i, st) for i in range(n_layers) for st in range(6)]
    got = a if final.value == a.data_ptr() else b
    assert final.value == (b if n_layers % 2 else a).data_ptr()
    assert torch.equal(got, want)
    for r1, r2 in zip(raws, raws2):
        assert torch.equal(r1, r2)                                               # the KV rows, RoPE of each layer's index
    # a failing hook stops the chunk with its code
    stop = _lib.ChunkHook(lambda user, il, stage, n_tokens, stream: -9 if (il, stage) == (first + 1, 2) else 0)
    assert L.ds4b200_chunk_rows_f32(C.byref(dims), W, n_layers, first, C.byref(buffers), a.data_ptr(), b.data_ptr(),
                                    pos.data_ptr(), T, stop, None, None, None) == -9
    torch.cuda.synchronize()
    assert ops.device_status() == 0
