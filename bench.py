#!/usr/bin/env python
"""Benchmark of the fused elementwise / row-reduction prefill path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one pass of the path over a batch of 4096 synthetic tokens per GPU:
for each of 43 layers the four fused launches (Q8_0 embedding gather + residual
+ RMSNorm -> f32 + bf16; YaRN RoPE + E4M3 KV-cache store; clamped SwiGLU x
router weights summed over 6 experts; 4x4 Sinkhorn + mix of the 4
hyper-connection streams).  Rank 0 prints ONE JSON line.

`--impl reference` times the CPU restatement of the same path (the oracle) on
the host cores; it is the only mode, with the `cpu_baseline` leg of the default
mode, that touches anything under oracle/.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

T_TOKENS, N_EMBD, VOCAB, KV_DIM, N_ROT, N_SLOTS, FF_DIM, TOP_K, N_LAYERS = (
    4096, 4096, 129280, 512, 64, 65536, 2048, 6, 43)
OP_NAMES = ("gather", "kvstore", "swiglu", "hcmix", "sinkhorn")
METRIC, UNIT = "fused_path_tokens_per_s", "tokens/s"
FALLBACK_HBM_GBS = 6650.0      # earlier measurement on this pool, used only without MEASURED_PEAKS.json

TRAFFIC_FILE = ROOT / "profiles" / "dram_traffic_prefill_path.txt"


def ncu_traffic_bytes(kernel, tokens):
    """dram__bytes_read.sum + dram__bytes_write.sum per launch of `kernel`, from the committed ncu figures
    (captured at a smaller token count), scaled in proportion to `tokens`; None when there is no figure."""
    try:
        for line in TRAFFIC_FILE.read_text().splitlines():
            f = line.split()
            if len(f) == 4 and f[0] == kernel:
                return int((int(f[2]) + int(f[3])) * tokens / int(f[1]))
    except (OSError, ValueError):
        pass
    return None


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--tokens", type=int, default=T_TOKENS, help="token rows per GPU (weak) or per job (strong)")
    ap.add_argument("--layers", type=int, default=N_LAYERS)
    ap.add_argument("--scaling", choices=["weak", "strong"], default="weak")
    ap.add_argument("--graph", type=int, default=1, help="replay the layer chain from a CUDA graph")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--e2e-chunks", type=int, default=8, help="row slices pipelined over H2D / compute / D2H")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="CPU work budget of the baseline sample")
    ap.add_argument("--only", default=None, help="run ONE batched op in a loop (for a one-kernel ncu capture) "
                                                 "and print its median time; see ONLY_OPS")
    ap.add_argument("--only-tokens", type=int, default=2048)
    ap.add_argument("--only-reps", type=int, default=6)
    return ap.parse_args()


def workload_config(args, tokens_per_gpu):
    return {
        "workload": "43-layer fused-op chain over 4096-token prefill rows (BASELINE configs[4]: "
                    "per layer the ops of configs[1..4] at their full shapes)",
        "tokens_per_gpu": tokens_per_gpu, "n_layers": args.layers, "n_embd": N_EMBD, "vocab": VOCAB,
        "embedding": "Q8_0", "kv_dim": KV_DIM, "n_rot": N_ROT, "kv_slots": N_SLOTS,
        "rope": "base 10000, YaRN factor 16, orig ctx 4096", "fp8_scale": "per-row amax/448",
        "ff_dim": FF_DIM, "top_k": TOP_K, "glu": "gate<=10, |up|<=10 (reference clamp), hardware exp as in the reference epilogue",
        "sinkhorn_iters": 20, "sharding": "token rows per rank, no collective",
        "l2": "inputs larger than L2: 1.17 GB touched per layer between reuses of any buffer",
    }


# ----------------------------------------------------------------------------- inputs

def make_inputs(tokens, seed):
    """Seeded synthetic host inputs with the benchmark configs' shapes and distributions."""
    import numpy as np
    sys.path.insert(0, str(ROOT / "tests"))
    import inputs as gen
    g = gen.rng(seed)
    return dict(
        ids=g.integers(0, VOCAB, tokens).astype(np.int32), pos=np.arange(tokens, dtype=np.int32),
        residual=gen.normal(g, (tokens, N_EMBD)), norm_w=gen.uniform(g, (N_EMBD,), 0.5, 1.5),
        kv=gen.normal(g, (tokens, KV_DIM), 1.5), gate=gen.normal(g, (tokens, TOP_K, FF_DIM), 2.0),
        up=gen.normal(g, (tokens, TOP_K, FF_DIM), 2.0), router_w=gen.router_weights(g, tokens, TOP_K),
        hc_logits=gen.normal(g, (tokens, 16)), hc_resid=gen.normal(g, (tokens, 4, N_EMBD)))


def make_table(seed=1234):
    sys.path.insert(0, str(ROOT / "tests"))
    import inputs as gen
    return gen.q8_0_table(gen.rng(seed), VOCAB, N_EMBD)


# ----------------------------------------------------------------------------- clocks

class ClockSampler(threading.Thread):
    """Polls SM clock and throttle reasons through NVML (read-only) while running."""

    REASONS = {0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
               0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.under_load, self.stop_flag = index, [], False, False
        self.max_mhz, self.reasons, self.ok = None, set(), False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        while not self.stop_flag:
            try:
                mhz = self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM)
                try:
                    mask = self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                self.samples.append((self.under_load, mhz))
                if self.under_load:
                    self.reasons |= {n for b, n in self.REASONS.items() if mask & b}
            except Exception:
                pass
            time.sleep(0.005)

    def summary(self):
        loaded = [m for u, m in self.samples if u] or [m for _, m in self.samples]
        return {"sm_mhz": statistics.median(loaded) if loaded else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(loaded)}


def physical_gpu_index(local_rank):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except (ValueError, IndexError):
            return local_rank
    return local_rank


# ----------------------------------------------------------------------------- CPU legs

def oracle_layer_pass(oracle, table, x, rope, lo, hi):
    """One layer of the path for rows [lo, hi) through the CPU oracle."""
    import numpy as np
    s = slice(lo, hi)
    oracle.embed_gather_rows(table, oracle.TABLE_Q8_0, x["ids"][s], N_EMBD, residual=x["residual"][s],
                             norm_w=x["norm_w"], want_bf16=True)
    oracle.rope_fp8_store_rows(x["kv"][s], x["pos"][s], rope, N_ROT, oracle.FP8_ROW_AMAX)
    oracle.swiglu_rows(x["gate"][s], x["up"][s], x["router_w"][s], oracle.GLU_CLAMP_REF, 10.0, combine=True)
    oracle.hc_sinkhorn_mix_rows(x["hc_logits"][s], x["hc_resid"][s])
    return hi - lo


def cpu_path_seconds(x, table, n_tokens, n_layers, threads):
    """Time n_layers of the path over the first n_tokens rows with `threads` host threads."""
    sys.path.insert(0, str(ROOT / "oracle"))
    import oracle_lib as oracle
    oracle.lib()
    rope = oracle.rope_params_explicit(10000.0, 16.0, 4096)
    bounds = [(n_tokens * i // threads, n_tokens * (i + 1) // threads) for i in range(threads)]

    def work(lo, hi):
        for _ in range(n_layers):
            oracle_layer_pass(oracle, table, x, rope, lo, hi)

    t0 = time.perf_counter()
    if threads == 1:
        work(0, n_tokens)
    else:
        ts = [threading.Thread(target=work, args=b) for b in bounds if b[1] > b[0]]
        [t.start() for t in ts]
        [t.join() for t in ts]
    dt = time.perf_counter() - t0
    return dt


def cpu_baseline_leg(x, table, budget_s, full_layers):
    """Scalar oracle, one thread, on a bounded sample; throughput scaled to the full layer count."""
    sample_tokens = min(128, len(x["ids"]))
    probe = cpu_path_seconds(x, table, sample_tokens, 1, 1)
    layers = max(1, min(full_layers, int(budget_s / max(probe, 1e-6))))
    dt = cpu_path_seconds(x, table, sample_tokens, layers, 1)
    per_layer = dt / layers
    value = sample_tokens / (per_layer * full_layers)
    return {"value": value, "unit": UNIT, "cores": 1, "kind": "port",
            "sample": f"{sample_tokens} tokens x {layers} layers in {dt:.2f} s on one thread; "
                      f"scaled to {full_layers} layers"}


def reference_kernels_leg(tokens, n_layers):
    """Baseline leg: the reference's OWN CUDA kernels for these stages, rebuilt unchanged for
    sm_100a (oracle/_ref), driven the way the reference drives them — one token per launch
    where it has no batched form — on a bounded sample of tokens, scaled to the full batch.
    Returns None when oracle/_ref has not been built."""
    import torch
    sys.path.insert(0, str(ROOT / "oracle"))
    import ref_lib
    if not ref_lib.available():
        return None
    sample = min(256, tokens)
    dev = "cuda"
    blocks = torch.randint(0, 255, (sample, 128 * 34), dtype=torch.uint8, device=dev)
    row, row2, row3 = (torch.empty(sample, N_EMBD, device=dev) for _ in range(3))
    resid, w = torch.randn(sample, N_EMBD, device=dev), torch.rand(N_EMBD, device=dev) + 0.5
    kv = torch.randn(sample, KV_DIM, device=dev)
    gate, up = torch.randn(sample * TOP_K * FF_DIM, device=dev), torch.randn(sample * TOP_K * FF_DIM, device=dev)
    mid = torch.empty_like(gate)
    hc, hc_out = torch.randn(sample, 4, N_EMBD, device=dev), torch.empty(sample, 4, N_EMBD, device=dev)
    post, comb, block = torch.rand(4, device=dev), torch.rand(16, device=dev), torch.randn(N_EMBD, device=dev)

    def gather():        # Q8_0 dequant + add + RMSNorm, per token (cuda/dense_q8.cu:75, elementwise.cu:46, norm.cu:109)
        ref_lib.call("loop_q8_gather_add_norm", blocks, resid, w, row, row2, row3, sample, N_EMBD, 1e-6)

    def kvstore():       # KV RoPE per token (one pos per launch), FP8 round trip batched over rows
        ref_lib.call("loop_kv_rope_fp8", kv, sample, KV_DIM, N_ROT, 0)

    def swiglu():        # its elementwise SwiGLU takes any n: one launch over all slots (no clamp, no combine)
        ref_lib.call("silu_mul_f32", gate, up, mid, sample * TOP_K * FF_DIM)

    def hcmix():         # HC post per token (cuda/hc_sinkhorn.cu:687)
        ref_lib.call("loop_hc_post", block, hc, post, comb, hc_out, sample, N_EMBD)

    out = {}
    for name, fn in (("gather", gather), ("kvstore", kvstore), ("swiglu", swiglu), ("hcmix", hcmix)):
        fn()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        fn()
        torch.cuda.synchronize()
        out[name + "_us_per_4096_tokens"] = round((time.perf_counter() - t0) * 1e6 * tokens / sample, 1)
    layer_us = sum(out.values())
    out["tokens_per_s"] = tokens / (layer_us * 1e-6 * n_layers)
    out["sample"] = (f"{sample} tokens, wall clock incl. launch overhead, scaled to {tokens} tokens x {n_layers} layers; "
                     "single-token launchers looped from C++ as the reference's forward pass does")
    return out


# ----------------------------------------------------------------------------- parity of the timed run

def parity_leg(x, table, out, n_layers, rows=64):
    """Per-op error figures of THIS run: the outputs the end-to-end call just copied back, first `rows`
    token rows, against the CPU oracle on the same inputs.  Runs after the timed regions."""
    import numpy as np
    sys.path.insert(0, str(ROOT / "oracle"))
    import oracle_lib as oracle
    r = min(rows, len(x["ids"]))
    sl = {k: (v if k == "norm_w" else v[:r]) for k, v in x.items()}
    rope = oracle.rope_params_explicit(10000.0, 16.0, 4096)
    res = {"rows": r}
    want_rows, want_norm, want_bf16 = oracle.embed_gather_rows(table, oracle.TABLE_Q8_0, sl["ids"], N_EMBD, residual=sl["residual"],
                                                               norm_w=sl["norm_w"], want_bf16=True)
    got = np.asarray(out["residual_out"])[:r]
    res["gather_residual_mismatching_values"] = int((got.view(np.uint32) != want_rows[:, 0, :].view(np.uint32)).sum())
    got_b = np.asarray(out["normed_bf16"])[:r].view(np.uint16)
    res["gather_normed_bf16_mismatching_values"] = int((got_b != np.asarray(want_bf16).view(np.uint16).reshape(got_b.shape)).sum())
    codes, scales, _, _ = oracle.rope_fp8_store_rows(sl["kv"], sl["pos"], rope, N_ROT, oracle.FP8_ROW_AMAX)
    res["kvstore_mismatching_code_bytes"] = int((np.asarray(out["kv_codes"])[:r] != codes).sum())
    res["kvstore_code_bytes"] = int(codes.size)
    res["kvstore_mismatching_scales"] = int((np.asarray(out["kv_scales"])[:r].view(np.uint32) != scales.view(np.uint32)).sum())
    want_ffn = oracle.swiglu_rows(sl["gate"], sl["up"], sl["router_w"], oracle.GLU_CLAMP_REF, 10.0, True)
    err = np.abs(np.asarray(out["ffn_out"])[:r].astype(np.float64) - want_ffn).max()
    res["swiglu_max_abs_err_over_max"] = float(err / np.abs(want_ffn).max())
    hc = sl["hc_resid"]
    for _ in range(n_layers):
        hc, _ = oracle.hc_sinkhorn_mix_rows(sl["hc_logits"], hc)
    err = np.abs(np.asarray(out["hc_out"])[:r].astype(np.float64) - hc).max()
    res["hcmix_max_abs_err_over_max_after_all_layers"] = float(err / np.abs(hc).max())
    res["bar"] = "gather residual bit-exact; bf16 and FP8 codes differ only at rounding boundaries; f32 ops <= 1e-5 x max per op"
    return res


# ----------------------------------------------------------------------------- strong split and copy floor

def strong_split_leg(args, rank, world, table, weak_value):
    """The same `--tokens` batch split T/N rows per rank (no collective): ms per step, whole-job tokens/s."""
    import torch
    from ds4cuda_b200 import shard
    from ds4cuda_b200.path import PrefillPath
    a, b = shard.token_range(rank, world, args.tokens)
    n = b - a
    path = PrefillPath(n_tokens=max(n, 1), max_layers=args.layers, use_graph=args.graph, glu_fast_exp=1)
    path.upload_table(table)
    x = make_inputs(max(n, 1), seed=500 + rank)
    path.upload({k: torch.from_numpy(v).pin_memory() for k, v in x.items()})
    for _ in range(args.warmup):
        path.run_device(args.layers)
    torch.cuda.synchronize()
    shard.barrier()
    ms = path.time_device(args.layers, 0, args.steps)
    torch.cuda.synchronize()
    shard.barrier()
    ms_step = shard.max_over_ranks(ms) / args.steps
    path.close()
    value = args.tokens / (ms_step * 1e-3)
    return {"tokens_per_rank": n, "ms_per_step": ms_step, "value": value, "unit": UNIT,
            "efficiency_vs_weak": round(value / weak_value, 4),     # weak_value = world x the per-GPU rate at full batches
            "what": f"one {args.tokens}-token batch split into contiguous row ranges, one per rank",
            "bound": "at 512 rows per GPU the three dependent kernels of a layer move 22 us of traffic "
                     "but each launch has a latency floor of a few us: the step is launch/latency bound"
                     if n <= 1024 else "HBM"}


def copy_floor_leg(h2d_tensors, d2h_tensors, reps=3):
    """The end-to-end step's copies alone: the same pinned host buffers in and out with plain
    cudaMemcpyAsync on two streams and no kernel, every rank at once.  ms per step, max over ranks."""
    import torch
    from ds4cuda_b200 import shard
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    dev_in = [torch.empty(t.shape, dtype=t.dtype, device="cuda") for t in h2d_tensors]
    dev_out = [torch.empty(t.shape, dtype=t.dtype, device="cuda") for t in d2h_tensors]
    torch.cuda.synchronize()
    shard.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        with torch.cuda.stream(s_in):
            for d, h in zip(dev_in, h2d_tensors):
                d.copy_(h, non_blocking=True)
        with torch.cuda.stream(s_out):
            for h, d in zip(d2h_tensors, dev_out):
                h.copy_(d, non_blocking=True)
    torch.cuda.current_stream().wait_stream(s_in)
    torch.cuda.current_stream().wait_stream(s_out)
    b.record()
    torch.cuda.synchronize()
    shard.barrier()
    return shard.max_over_ranks(a.elapsed_time(b) / reps)


# ----------------------------------------------------------------------------- one op in a loop

def only_ops(tokens):
    """name -> (callable, algorithmic bytes, description) for `--only`: every batched op outside the
    five-kernel chain, at `tokens` token rows, on resident synthetic inputs."""
    import torch
    from ds4cuda_b200 import ops
    dev, T, n = "cuda", tokens, N_EMBD
    g = torch.Generator(device=dev).manual_seed(13)
    rnd = lambda *shape, s=1.0: torch.randn(*shape, device=dev, generator=g) * s
    reg = {}

    def add(name, make):
        reg[name] = make

    def hc_pre():
        resid, fn = rnd(T, 4, n), (rnd(24, 4 * n) / 128).half()
        sc, base = torch.ones(3, device=dev), torch.zeros(24, device=dev)
        return (lambda: ops.hc_pre_rows(resid, fn, sc, base)), T * (4 * n * 4 + n * 4 + 80) + fn.numel() * 2, \
            "full HC pre: 24 dots per token on the tensor cores + gates + stream sum + Sinkhorn sweeps"

    def hc_post_block():
        resid, block = rnd(T, 4, n), rnd(T, n)
        post, comb = torch.rand(T, 4, device=dev, generator=g), torch.rand(T, 16, device=dev, generator=g)
        return (lambda: ops.hc_post_rows(block, resid, post, comb)), T * (2 * 4 * n * 4 + n * 4 + 80), "HC post with the block term"

    def hc_head():
        resid, fn = rnd(T, 4, n), (rnd(4, 4 * n) / 128).half()
        sc, base, w = torch.ones(1, device=dev), torch.zeros(4, device=dev), torch.rand(n, device=dev, generator=g) + 0.5
        return (lambda: ops.output_hc_head_rows(resid, fn, sc, base, norm_w=w)), T * (4 * n * 4 + 2 * n * 4), "output HC head + output norm"

    def rms_norm_cta():
        x, w = rnd(T, n), torch.rand(n, device=dev, generator=g) + 0.5
        return (lambda: ops.rms_norm_rows(x, w)), T * n * 8, "RMSNorm, 4096-wide rows (one CTA per row)"

    def rms_norm_q8_0():
        x, w = rnd(T, n), torch.rand(n, device=dev, generator=g) + 0.5
        return (lambda: ops.rms_norm_q8_0_rows(x, w, want_f32=False)), T * (n * 4 + n + n // 8), "RMSNorm with the Q8_0 blocks as only output"

    def rms_norm_q8_K():
        x, w = rnd(T, n), torch.rand(n, device=dev, generator=g) + 0.5
        return (lambda: ops.rms_norm_q8_K_rows(x, w, want_f32=False, want_q8_0=True)), \
            T * (n * 4 + n + n // 8 + n + n // 256 * 36), "RMSNorm leaving the row as Q8_0 and Q8_K blocks (ffn norm)"

    def rms_norm_warp():
        x = rnd(T * 64, 512)
        return (lambda: ops.rms_norm_rows(x, None)), T * 64 * 512 * 8, "unit-gain RMSNorm, 512-wide head rows (one warp per row)"

    def rope_rows():
        q, pos = rnd(T, 64, KV_DIM), torch.arange(T, device=dev, dtype=torch.int32)
        rp = ops.rope_params_for_layer(2)
        return (lambda: ops.rope_rows(q, pos, rp, unit_rms=True, out=q)), T * 64 * KV_DIM * 8, "q_norm + tail RoPE over 64 heads per token"

    def rope_inverse():
        q, pos = rnd(T, 64, KV_DIM), torch.arange(T, device=dev, dtype=torch.int32)
        rp = ops.rope_params_for_layer(2)
        return (lambda: ops.rope_rows(q, pos, rp, inverse=True, out=q)), T * 64 * KV_DIM * 8, "inverse tail RoPE over 64 heads per token"

    def rope_inverse_q8_0():
        q, pos = rnd(T, 64, KV_DIM), torch.arange(T, device=dev, dtype=torch.int32)
        rp = ops.rope_params_for_layer(2)
        return (lambda: ops.rope_q8_0_rows(q, pos, rp, inverse=True)), T * 64 * (KV_DIM * 4 + KV_DIM + KV_DIM // 8), \
            "inverse tail RoPE leaving as the out-projection's Q8_0 blocks (no f32 copy)"

    def rope_inverse_q8_0_table():
        q, pos = rnd(T, 64, KV_DIM), torch.arange(T, device=dev, dtype=torch.int32)
        table = ops.rope_table_rows(pos, ops.rope_params_for_layer(2))
        return (lambda: ops.rope_q8_0_rows(q, None, None, inverse=True, table=table)), \
            T * (64 * (KV_DIM * 4 + KV_DIM + KV_DIM // 8) + 256), "the same, angles from the chunk's table"

    def rope_rows_table():
        q, pos = rnd(T, 64, KV_DIM), torch.arange(T, device=dev, dtype=torch.int32)
        table = ops.rope_table_rows(pos, ops.rope_params_for_layer(2))
        return (lambda: ops.rope_rows(q, None, None, unit_rms=True, out=q, table=table)), T * (64 * KV_DIM * 8 + 256), \
            "q_norm + tail RoPE over 64 heads per token, angles from the chunk's table"

    def rope_table():
        pos = torch.arange(T, device=dev, dtype=torch.int32)
        rp = ops.rope_params_for_layer(2)
        return (lambda: ops.rope_table_rows(pos, rp)), T * (4 + 256), "the chunk's angle table (once per chunk and parameter set)"

    def fp8_round_trip():
        rows = T * 16
        kv = rnd(rows, KV_DIM, s=1.5)
        return (lambda: ops.fp8_kv_round_trip_rows(kv)), rows * KV_DIM * 8, "FP8 E4M3 round trip (reference scale mode), 16 rows per token"

    def rope_fp8_store():
        rows = T * 16
        kv = rnd(rows, KV_DIM, s=1.5)
        pos = (torch.arange(rows, device=dev, dtype=torch.int32) % 4096).contiguous()
        slots = torch.arange(rows, device=dev, dtype=torch.int32)
        codes, scales = torch.zeros(rows, KV_DIM, dtype=torch.uint8, device=dev), torch.zeros(rows, 1, device=dev)
        rp = ops.rope_params_explicit(10000.0, 16.0, 4096, N_ROT)
        return (lambda: ops.rope_fp8_store_rows(kv, pos, rp, N_ROT, ops.FP8_ROW_AMAX, codes, scales, slots=slots)), \
            rows * (KV_DIM * 4 + KV_DIM + 8), "RoPE + E4M3 cache store, 16 rows per token"

    def rope_fp8_store_table():
        rows = T * 16
        kv = rnd(rows, KV_DIM, s=1.5)
        pos = (torch.arange(rows, device=dev, dtype=torch.int32) % 4096).contiguous()
        slots = torch.arange(rows, device=dev, dtype=torch.int32)
        codes, scales = torch.zeros(rows, KV_DIM, dtype=torch.uint8, device=dev), torch.zeros(rows, 1, device=dev)
        table = ops.rope_table_rows(pos, ops.rope_params_explicit(10000.0, 16.0, 4096, N_ROT))
        return (lambda: ops.rope_fp8_store_rows(kv, None, None, N_ROT, ops.FP8_ROW_AMAX, codes, scales, slots=slots,
                                                table=table)), \
            rows * (KV_DIM * 4 + KV_DIM + 8 + N_ROT * 4), "the same, angles from a table (one row of 32 pairs per KV row)"

    def swiglu_q8k():
        gate, up = rnd(T, TOP_K, FF_DIM, s=2.0), rnd(T, TOP_K, FF_DIM, s=2.0)
        w = torch.softmax(rnd(T, TOP_K), -1)
        return (lambda: ops.swiglu_q8_K_rows(gate, up, w, ops.GLU_CLAMP_REF, 10.0, fast_exp=True)), \
            T * TOP_K * (FF_DIM * 8 + FF_DIM + FF_DIM // 256 * 36), "expert epilogue leaving as Q8_K blocks"

    def swiglu_q8_0():
        gate, up = rnd(T, 1, FF_DIM), rnd(T, 1, FF_DIM)
        return (lambda: ops.swiglu_q8_0_rows(gate, up)), T * (FF_DIM * 8 + FF_DIM + FF_DIM // 8), "shared expert's silu*up leaving as Q8_0 blocks"

    def quantize_q8_K():
        x = rnd(T * TOP_K, FF_DIM)
        return (lambda: ops.quantize_q8_K_rows(x)), T * TOP_K * (FF_DIM * 4 + FF_DIM + FF_DIM // 256 * 36), "Q8_K activation quantiser"

    for f in (hc_pre, hc_post_block, hc_head, rms_norm_cta, rms_norm_q8_0, rms_norm_q8_K, rms_norm_warp, rope_rows, rope_inverse,
              rope_inverse_q8_0, rope_inverse_q8_0_table, rope_rows_table, rope_table, fp8_round_trip, rope_fp8_store, rope_fp8_store_table, swiglu_q8k, swiglu_q8_0, quantize_q8_K):
        add(f.__name__, f)
    return reg


def run_only(args):
    """`--only OP`: a few launches of one op between L2 flushes; one JSON line with its median time."""
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product path has no CPU fallback")
    reg = only_ops(args.only_tokens)
    if args.only not in reg:
        raise SystemExit(f"--only: unknown op {args.only!r}; one of {sorted(reg)}")
    fn, nbytes, what = reg[args.only]()
    flush = torch.empty(192 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    ts = []
    for i in range(args.only_reps):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); fn(); b.record(); torch.cuda.synchronize()
        if i >= 2:
            ts.append(a.elapsed_time(b) * 1e3)
    us = sorted(ts)[len(ts) // 2]
    peak = measured_peak()[0]
    print(json.dumps({"only": args.only, "tokens": args.only_tokens, "us_per_launch": round(us, 1),
                      "algorithmic_bytes": int(nbytes), "gbs": round(nbytes / us / 1e3, 1),
                      "frac_of_peak": round(nbytes / us / 1e3 / peak, 4), "what": what}), flush=True)


def measured_peak():
    peaks_file = ROOT / "MEASURED_PEAKS.json"
    if peaks_file.exists():
        return float(json.loads(peaks_file.read_text())["hbm_gbs"]), "measured"
    return FALLBACK_HBM_GBS, "fallback"


def standalone_ops_leg(tokens, peak):
    """The batched forms the layer chain does not contain.  Two figures per op, CUDA events on torch's current
    stream (the stream these wrappers launch on):
    `us_per_launch`: one launch on its own between L2 flushes, median of 9; it carries the launch latency and
    the ramp of a cold, empty GPU (about 8 us whatever the op);
    `us_back_to_back`: several instances of the op on their own buffers (together more than twice the L2)
    replayed back to back from one CUDA graph, the way a stage runs inside a layer; time per instance."""
    import torch
    flush = torch.empty(192 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    out = {}
    for name, make in only_ops(tokens).items():
        fn, nbytes, what = make()
        ts = []
        for i in range(12):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(); b.record(); torch.cuda.synchronize()
            if i >= 3:
                ts.append(a.elapsed_time(b) * 1e3)
        us = sorted(ts)[len(ts) // 2]
        gbs = nbytes / us / 1e3
        out[name] = {"us_per_launch": round(us, 1), "algorithmic_bytes": int(nbytes), "gbs": round(gbs, 1),
                     "frac_of_peak": round(gbs / peak, 4), "what": what}
        # back to back: enough instances that no buffer is still in L2 when its turn comes again
        n_sets = max(2, min(8, int(300e6 // max(nbytes, 1)) + 2))
        try:
            fns = [fn] + [make()[0] for _ in range(n_sets - 1)]
            for f in fns:
                f()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for f in fns:
                    f()
            graph.replay()
            torch.cuda.synchronize()
            rounds = 5
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(rounds):
                graph.replay()
            b.record(); torch.cuda.synchronize()
            us_b2b = a.elapsed_time(b) * 1e3 / (rounds * n_sets)
            out[name].update({"us_back_to_back": round(us_b2b, 1), "instances": n_sets,
                              "frac_back_to_back": round(nbytes / us_b2b / 1e3 / peak, 4)})
            del graph, fns
        except Exception as e:                                    # noqa: BLE001 — report, keep the single-launch figure
            out[name]["us_back_to_back"] = None
            out[name]["back_to_back_error"] = str(e)[:120]
        del fn
        torch.cuda.empty_cache()
    return out


def layer_row_stages_leg(tokens, peak):
    """Every row stage of one layer in the order ds4_forward_layer runs them (cuda/forward_layer.cu:808-1461),
    batched over `tokens` rows, with resident synthetic buffers standing in for the outputs of the matvec and
    attention stages between them (those stages are outside this library).  One launch per stage between L2
    flushes, CUDA events on torch's current stream; reports µs per stage and their sum."""
    import torch
    from ds4cuda_b200 import ops
    dev, T, n = "cuda", tokens, N_EMBD
    g = torch.Generator(device=dev).manual_seed(11)
    rnd = lambda *shape, s=1.0: torch.randn(*shape, device=dev, generator=g) * s
    flush = torch.empty(192 * 1024 * 1024, dtype=torch.uint8, device=dev)
    resid_hc = rnd(T, 4, n)
    fn_a, fn_f = (rnd(24, 4 * n) / 128).half(), (rnd(24, 4 * n) / 128).half()
    scale3, base24 = torch.ones(3, device=dev), torch.zeros(24, device=dev)
    w_n = torch.rand(n, device=dev, generator=g) + 0.5
    w_q = torch.rand(1024, device=dev, generator=g) + 0.5
    w_kv = torch.rand(KV_DIM, device=dev, generator=g) + 0.5
    pos = torch.arange(T, device=dev, dtype=torch.int32)
    rope = ops.rope_params_for_layer(2)
    q_lora, kv_raw = rnd(T, 1024), rnd(T, KV_DIM, s=1.5)
    q_raw, kqv = rnd(T, 64, KV_DIM), rnd(T, 64, KV_DIM)
    attn_out, moe_out, shexp = rnd(T, n), rnd(T, n), rnd(T, n)
    sh_gate, sh_up = rnd(T, 1, FF_DIM, s=2.0), rnd(T, 1, FF_DIM, s=2.0)
    gate, up = rnd(T, TOP_K, FF_DIM, s=2.0), rnd(T, TOP_K, FF_DIM, s=2.0)
    w_r = torch.softmax(rnd(T, TOP_K), -1)
    raw_rows = torch.empty(T, KV_DIM, device=dev)
    st = {}

    def stage(name, fn):
        ts = []
        for i in range(8):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); r = fn(); b.record(); torch.cuda.synchronize()
            if i >= 2:
                ts.append(a.elapsed_time(b) * 1e3)
        st[name] = round(sorted(ts)[len(ts) // 2], 1)
        return r

    post_a, comb_a, x = stage("hc_attn_pre", lambda: ops.hc_pre_rows(resid_hc, fn_a, scale3, base24))
    stage("attn_norm+q8_0", lambda: ops.rms_norm_q8_0_rows(x, w_n))
    stage("q_a_norm+q8_0", lambda: ops.rms_norm_q8_0_rows(q_lora, w_q))
    # the KV row chain evaluates the 32 angles of its token anyway: it leaves them as the chunk's angle table
    table = torch.zeros(T, N_ROT // 2, 2, device=dev)
    stage("kv_norm+rope+fp8+f16+angle_table", lambda: ops.kv_rows_to_raw(kv_raw, pos, rope, raw_rows, norm_w=w_kv,
                                                                        table_out=table))
    stage("q_norm+rope", lambda: ops.rope_rows(q_raw, None, None, unit_rms=True, out=q_raw, table=table))
    stage("attn_out_inverse_rope+q8_0", lambda: ops.rope_q8_0_rows(kqv, None, None, inverse=True, table=table))
    resid_attn = stage("hc_attn_post", lambda: ops.hc_post_rows(attn_out, resid_hc, post_a, comb_a))
    post_f, comb_f, xf = stage("hc_ffn_pre", lambda: ops.hc_pre_rows(resid_attn, fn_f, scale3, base24))
    stage("ffn_norm+q8_0+q8_K", lambda: ops.rms_norm_q8_K_rows(xf, w_n, want_q8_0=True))
    stage("shared_silu_mul+q8_0", lambda: ops.swiglu_q8_0_rows(sh_gate, sh_up))
    stage("expert_swiglu+q8_K", lambda: ops.swiglu_q8_K_rows(gate, up, w_r, ops.GLU_CLAMP_REF, 10.0, fast_exp=True))
    stage("add+hc_ffn_post", lambda: ops.hc_post_rows(moe_out, resid_attn, post_f, comb_f, block_out2=shexp))
    # the same twelve stages through the one-call entry point (no-op hook: the stand-ins above are
    # already in place), back to back without flushes: what the row stages of a layer cost in a chunk
    import ctypes as C
    from ds4cuda_b200 import _lib
    L = _lib.load()
    z = lambda *shape, dt=torch.float32: torch.zeros(*shape, dtype=dt, device=dev)
    bufs = dict(x=z(T, n), x_norm=z(T, n), xq=z(T, n, dt=torch.int8), xscale=z(T, n // 32), q_lora=q_lora,
                q_lora_norm=z(T, 1024), kv_raw=kv_raw, raw_rows=raw_rows, q=q_raw, kqv=kqv, attn_out=attn_out,
                post=z(T, 4), comb=z(T, 16), resid_mid=z(T, 4, n), sh_gate=sh_gate, sh_up=sh_up, sh_mid=z(T, FF_DIM),
                gate=gate, up=up, router_w=w_r, mid_q=z(T, TOP_K, FF_DIM, dt=torch.int8),
                mid_scale=z(T, TOP_K, FF_DIM // 256), mid_bsums=z(T, TOP_K, FF_DIM // 256, 16, dt=torch.int16),
                moe_out=moe_out, shexp_out=shexp, kqv_q=z(T, 64, KV_DIM, dt=torch.int8), kqv_scale=z(T, 64, KV_DIM // 32),
                rope_cs=z(T, N_ROT // 2, 2), ffn_kq=z(T, n, dt=torch.int8), ffn_kscale=z(T, n // 256),
                ffn_kbsums=z(T, n // 16, dt=torch.int16), sh_q=z(T, FF_DIM, dt=torch.int8), sh_scale=z(T, FF_DIM // 32),
                ql_q=z(T, 1024, dt=torch.int8), ql_scale=z(T, 32))
    wts = dict(hc_attn_fn=fn_a, hc_attn_scale=scale3, hc_attn_base=base24, attn_norm=w_n, q_a_norm=w_q, kv_a_norm=w_kv,
               hc_ffn_fn=fn_f, hc_ffn_scale=scale3, hc_ffn_base=base24, ffn_norm=w_n)
    dims = _lib.LayerDims(n, 64, KV_DIM, N_ROT, 1024, FF_DIM, TOP_K, 20, 2, 1, 1e-6, 10.0)
    lw = _lib.LayerWeights(*[wts[k].data_ptr() for k in _lib.LayerWeights.NAMES])
    lb = _lib.LayerBuffers(*[bufs[k].data_ptr() for k in _lib.LayerBuffers.NAMES + _lib.LayerBuffers.OPTIONAL])
    hook = _lib.StageHook(lambda user, stage, n_tok, stream: 0)
    out_hc = torch.empty_like(resid_hc)

    def whole():
        rc = L.ds4b200_layer_rows_f32(C.byref(dims), C.byref(lw), C.byref(lb), resid_hc.data_ptr(), pos.data_ptr(), T,
                                      out_hc.data_ptr(), hook, None, None)
        if rc:
            raise RuntimeError(L.ds4b200_last_error().decode())

    whole(); torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(5):
        whole()
    b.record(); torch.cuda.synchronize()
    chain_us = round(a.elapsed_time(b) * 1e3 / 5, 1)
    return {"tokens": T, "us_per_stage": st, "us_per_layer": round(sum(st.values()), 1),
            "us_per_layer_one_call": chain_us,
            "what": "batched row stages of one layer in forward_layer order; matvec / attention outputs are resident stand-ins"}


def run_reference_arm(args):
    """The reference's CPU path: the scalar C restatement, all host threads, bounded sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = len(os.sched_getaffinity(0))
    tokens = min(args.tokens, 8 * threads)
    x = make_inputs(tokens, seed=100)
    table = make_table()
    probe = cpu_path_seconds(x, table, tokens, 1, threads)
    total_steps = args.steps + args.warmup
    layers = max(1, min(args.layers, int(120.0 / max(probe * total_steps, 1e-6))))
    for _ in range(args.warmup):
        cpu_path_seconds(x, table, tokens, layers, threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_path_seconds(x, table, tokens, layers, threads)
    dt = (time.perf_counter() - t0) / args.steps
    ms_per_step = dt / layers * args.layers * 1e3 * (args.tokens / tokens)
    value = args.tokens / (ms_per_step * 1e-3)
    sample = (f"each step: {tokens} tokens x {layers} layers on {threads} threads "
              f"({dt:.2f} s), scaled to {args.tokens} tokens x {args.layers} layers")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, args.tokens),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "extrapolated": True,
        "measured_sample": {"tokens": tokens, "layers": layers, "seconds_per_step": dt,
                            "tokens_x_layers_per_s": tokens * layers / dt},
        "what_this_is": "own CPU oracle (scalar C restatement of the reference kernels' arithmetic) on all host "
                        "threads; NOT the upstream GPU code.  The reference's own kernels rebuilt for sm_100a are "
                        "timed in the main arm's reference_kernels_sm100a leg (vs_reference_kernels_sm100a)",
        "note": "the reference ships no CPU implementation of this path (its CPU model, antirez/ds4, is not "
                "in its tree); the value scales the measured sample linearly in rows and layers",
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- GPU arm

def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    from ds4cuda_b200 import shard
    from ds4cuda_b200.path import PrefillPath

    tokens = shard.tokens_per_rank(world, args.tokens, args.scaling)[rank]
    # glu_fast_exp=1: the reference's expert epilogue uses the hardware exp (cuda/moe_iq2_pair.cu:364,367)
    path = PrefillPath(n_tokens=tokens, max_layers=args.layers, use_graph=args.graph, glu_fast_exp=1)
    table = make_table()
    path.upload_table(table)
    x = make_inputs(tokens, seed=100 + rank)
    pinned_in = {k: torch.from_numpy(v).pin_memory() for k, v in x.items()}
    path.upload(pinned_in)

    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()

    # ---- device-resident timing: W warm-up steps, then exactly K timed steps
    for _ in range(args.warmup):
        path.run_device(args.layers)
    torch.cuda.synchronize()
    shard.barrier()
    torch.cuda.synchronize()
    sampler.under_load = True
    ms_total = path.time_device(args.layers, 0, args.steps)
    torch.cuda.synchronize()
    sampler.under_load = False
    shard.barrier()
    ms_step = shard.max_over_ranks(ms_total) / args.steps
    job_tokens = shard.sum_over_ranks(tokens)
    value = job_tokens / (ms_step * 1e-3)

    # ---- per-kernel durations inside the chain (events around every launch)
    per_op_ms = path.profile_ops(50)
    # one launch of each kernel on its own (events around a single launch; includes the launch gap)
    single_ms = path.profile_ops(1)
    ops_table = {}
    peak, peak_src = measured_peak()
    for i, name in enumerate(OP_NAMES):
        us = per_op_ms[name] * 1e3
        gbs = path.op_bytes(i) / (us * 1e-6) / 1e9
        ops_table[name] = {"us_per_launch": round(us, 2), "us_single_launch": round(single_ms[name] * 1e3, 2),
                           "algorithmic_bytes": path.op_bytes(i),
                           "gbs": round(gbs, 1), "frac_of_peak": round(gbs / peak, 4),
                           "frac_of_8000": round(gbs / 8000.0, 4)}
    dominant = max(OP_NAMES, key=lambda n: ops_table[n]["us_per_launch"])
    roofline = {"bound": "hbm", "kernel": dominant, "achieved": ops_table[dominant]["gbs"], "peak": peak,
                "peak_source": peak_src, "unit": "GB/s", "frac": ops_table[dominant]["frac_of_peak"],
                "traffic": ncu_traffic_bytes(dominant, tokens)}
    step_bytes = sum(path.op_bytes(i) for i in range(len(OP_NAMES))) * args.layers
    hbm_gbs_step = step_bytes / (ms_step * 1e-3) / 1e9

    # ---- end to end through the host-buffer entry point: H2D of every input,
    #      the layer chain, D2H of every output, per step
    out_shapes = path.output_shapes()
    tdt = {"float32": torch.float32, "uint16": torch.int16, "uint8": torch.uint8}
    pinned_out = {k: torch.empty(s, dtype=tdt[np.dtype(d).name]).pin_memory()
                  for k, (s, d) in out_shapes.items() if k != "kv_tail"}
    h2d = sum(t.numel() * t.element_size() for t in pinned_in.values())
    d2h = sum(t.numel() * t.element_size() for t in pinned_out.values())
    path.run_host(pinned_in, args.layers, pinned_out, n_chunks=args.e2e_chunks)            # warm-up
    torch.cuda.synchronize()
    shard.barrier()
    sampler.under_load = True
    e2e_ms = 0.0
    for _ in range(max(1, args.e2e_steps)):
        e2e_ms += path.run_host(pinned_in, args.layers, pinned_out, n_chunks=args.e2e_chunks)["ms"]
    sampler.under_load = False
    torch.cuda.synchronize()
    shard.barrier()
    e2e_ms_step = shard.max_over_ranks(e2e_ms) / max(1, args.e2e_steps)
    e2e_value = job_tokens / (e2e_ms_step * 1e-3)
    parity_rows = {k: v[:64].clone().numpy() for k, v in pinned_out.items()}       # before the buffers are reused
    # the same bytes with no kernels: what the host's memory / PCIe complex allows when every rank copies at once
    copy_floor_ms = copy_floor_leg(list(pinned_in.values()), list(pinned_out.values()))

    sampler.stop_flag = True
    sampler.join(timeout=2)
    clocks = sampler.summary()

    cpu, ref_kernels, parity = None, None, None
    if rank == 0:
        try:      # error figures of the outputs this run produced (checker only, after the timed regions)
            parity = parity_leg(x, table, parity_rows, args.layers)
        except Exception as e:                      # noqa: BLE001
            parity = {"error": f"{type(e).__name__}: {e}"}
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline_leg(x, table, args.cpu_seconds, args.layers)
        ref_kernels = reference_kernels_leg(tokens, args.layers)

    launches = path.launches_per_run(args.layers) * args.steps
    path.close()
    strong = None
    if world > 1 and args.scaling == "weak":
        try:
            strong = strong_split_leg(args, rank, world, table, value)
        except Exception as e:                      # noqa: BLE001
            strong = {"error": f"{type(e).__name__}: {e}"}
    # extra single-GPU legs; a failure there must not cost the main line
    standalone = layer_stages = None
    if rank == 0 and world == 1:
        try:
            standalone = standalone_ops_leg(tokens, peak)
        except Exception as e:                      # noqa: BLE001
            standalone = {"error": f"{type(e).__name__}: {e}"}
        try:
            layer_stages = layer_row_stages_leg(tokens, peak)
        except Exception as e:                      # noqa: BLE001
            layer_stages = {"error": f"{type(e).__name__}: {e}"}
    if world > 1:
        dist.destroy_process_group()
    if rank != 0:
        return
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": args.scaling,
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, tokens),
        "hbm_gbs_per_gpu": round(hbm_gbs_step, 1),
        "hbm_frac_of_peak": round(hbm_gbs_step / peak, 4), "hbm_frac_of_8000": round(hbm_gbs_step / 8000.0, 4),
        "ops": ops_table, "roofline": roofline, "cpu_baseline": cpu,
        "reference_kernels_sm100a": ref_kernels, "standalone_ops": standalone, "layer_row_stages": layer_stages,
        "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": e2e_ms_step,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "copy_floor_ms": copy_floor_ms, "ms_per_step_over_copy_floor": round(e2e_ms_step / copy_floor_ms, 3),
                "pipeline": f"{args.e2e_chunks} row slices over copy-in / compute / copy-out streams; copy_floor_ms "
                            "is the same host buffers copied in and out with no kernel, all ranks at once"},
        "parity": parity, "strong_split": strong,
        "vs_reference_kernels_sm100a": (round(value / ref_kernels["tokens_per_s"], 1)
                                        if ref_kernels and ref_kernels.get("tokens_per_s") else None),
        "gpu_launches": launches, "cuda_graph": bool(args.graph), "clocks": clocks,
    }
    print(json.dumps(line), flush=True)


def main():
    args = parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.gpus > 1 and world == 1 and "RANK" not in os.environ:
        # launched without torchrun: start one rank per GPU ourselves
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", str(29400 + os.getpid() % 500),
               str(Path(__file__).resolve())] + sys.argv[1:]
        raise SystemExit(subprocess.call(cmd))
    if args.only:
        run_only(args)
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
