"""GPU test of the allocation-free Sinkhorn mixing entry point.

Collected last on purpose (file name): a run that stops at the first failure has
then already run every other test.  The entry point keeps its intermediate in a
fixed device array inside the library, for callers that may not allocate device
memory and have no spare buffer to lend; this test drives it through the C ABI,
twice in a row with different batch sizes, and compares each result with the
ordinary entry point (caller-provided intermediate) on the same inputs and with
the CPU oracle.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import inputs

pytestmark = pytest.mark.gpu

REL_TOL = 1e-5      # the f32 bar of the parity tests: max-abs error <= REL_TOL * max|want|


def _run_both(L, T, n_embd, seed):
    g = inputs.rng(seed)
    logits = torch.from_numpy(inputs.normal(g, (T, 16))).cuda()
    resid = torch.from_numpy(inputs.normal(g, (T, 4, n_embd))).cuda()
    want, comb = torch.empty_like(resid), torch.empty(T, 16, device="cuda")
    got = torch.full_like(resid, float("nan"))
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = L.ds4b200_hc_sinkhorn_mix_rows_f32(logits.data_ptr(), resid.data_ptr(), want.data_ptr(), comb.data_ptr(),
                                            T, n_embd, 20, 1e-6, stream)
    assert rc == 0, L.ds4b200_last_error()
    rc = L.ds4b200_hc_sinkhorn_mix_rows_static_f32(logits.data_ptr(), resid.data_ptr(), got.data_ptr(), T, n_embd,
                                                   20, 1e-6, stream)
    assert rc == 0, L.ds4b200_last_error()
    torch.cuda.synchronize()
    got, want = got.cpu().numpy().astype(np.float64), want.cpu().numpy().astype(np.float64)
    assert np.isfinite(got).all()
    err = np.abs(got - want).max()
    assert err <= REL_TOL * np.abs(want).max(), f"T={T}: max-abs error {err:.3e}"
    # and against the CPU oracle, not only against the sibling entry point
    import oracle_lib as oracle
    oracle.lib()
    mixed, _ = oracle.hc_sinkhorn_mix_rows(logits.cpu().numpy(), resid.cpu().numpy())
    err = np.abs(got - mixed).max()
    assert err <= REL_TOL * np.abs(mixed).max(), f"T={T}: max-abs error vs the oracle {err:.3e}"


def test_static_scratch_entry_point_matches_the_ordinary_one_twice_in_a_row():
    assert torch.cuda.is_available()
    from ds4cuda_b200 import _lib
    L = _lib.load()
    # first call: a large batch fills many rows of the built-in array ...
    _run_both(L, 700, 4096, seed=901)
    # ... second call: a smaller batch with other values must not see them
    _run_both(L, 33, 1024, seed=902)
    # beyond the built-in capacity: refused with a message, nothing launched
    p = C.c_void_p(0x1000)
    rc = L.ds4b200_hc_sinkhorn_mix_rows_static_f32(p, p, p, 16385, 4096, 20, 1e-6, None)
    assert rc == -22 and b"exceed the built-in scratch" in L.ds4b200_last_error()
    assert L.ds4b200_hc_sinkhorn_mix_rows_static_f32(None, None, None, 0, 4096, 20, 1e-6, None) == 0
