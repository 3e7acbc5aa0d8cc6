"""CPU tests of the multi-rank host logic: row partition and the timing
reduction, on two gloo ranks; the compute stand-in is the oracle, so a sharded
batch must reproduce the unsharded one bit for bit."""
import os
import sys

import numpy as np
import pytest
import torch.multiprocessing as mp

import inputs


def test_token_range_partitions_exactly():
    from ds4cuda_b200.shard import token_range, tokens_per_rank
    for world in (1, 2, 3, 4, 8):
        for n in (0, 1, 7, 8, 4096, 4099):
            spans = [token_range(r, world, n) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
            assert tokens_per_rank(world, n, "strong") == sizes
            assert tokens_per_rank(world, n, "weak") == [n] * world
    with pytest.raises(ValueError):
        token_range(2, 2, 10)
    with pytest.raises(ValueError):
        tokens_per_rank(2, 10, "sideways")


def _rank_main(rank, world, port, tmp):
    import torch.distributed as dist
    sys.path.insert(0, os.path.join(os.path.dirname(__file__), "..", "oracle"))
    sys.path.insert(0, os.path.dirname(__file__))
    import oracle_lib
    from ds4cuda_b200 import shard
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    T = 37
    c = inputs.config4(seed=9, T=T, k=6, n=64)
    a, b = shard.token_range(rank, world, T)
    out = oracle_lib.swiglu_rows(c["gate"][a:b], c["up"][a:b], c["weights"][a:b], oracle_lib.GLU_CLAMP_REF,
                                 10.0, combine=True)
    np.save(os.path.join(tmp, f"out{rank}.npy"), out)
    ms = 10.0 * (rank + 1)                                  # rank 1 is the slow one
    worst = shard.max_over_ranks(ms)
    total = shard.sum_over_ranks(b - a)
    tput = shard.job_throughput(b - a, ms)
    shard.barrier()
    np.save(os.path.join(tmp, f"red{rank}.npy"), np.array([worst, total, tput]))
    dist.destroy_process_group()


def test_two_gloo_ranks_shard_rows_and_reduce_timing(tmp_path, oracle):
    world, port = 2, 29500 + os.getpid() % 2000
    mp.spawn(_rank_main, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    T = 37
    c = inputs.config4(seed=9, T=T, k=6, n=64)
    want = oracle.swiglu_rows(c["gate"], c["up"], c["weights"], oracle.GLU_CLAMP_REF, 10.0, combine=True)
    got = np.concatenate([np.load(tmp_path / f"out{r}.npy") for r in range(world)])
    assert np.array_equal(got, want)
    for r in range(world):
        worst, total, tput = np.load(tmp_path / f"red{r}.npy")
        assert worst == 20.0 and total == T and tput == pytest.approx(T / 0.020)
