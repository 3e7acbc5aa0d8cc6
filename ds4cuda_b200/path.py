"""Python handle on the C++ prefill path object (include/ds4b200_path.h)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import FP8_ROW_AMAX, GLU_CLAMP_REF, TABLE_Q8_0, PathConfig, PathIO, RopeParams, check

KERNELS = ("gather", "kvstore", "swiglu", "hcmix", "sinkhorn")


class PrefillPath:
    """Owns the device buffers, stream and launch chain of one T-token pass."""

    def __init__(self, n_tokens=4096, n_embd=4096, vocab=129280, table_dtype=TABLE_Q8_0, kv_dim=512,
                 n_rot=64, n_slots=65536, ff_dim=2048, top_k=6, max_layers=43, sinkhorn_iters=20,
                 fp8_scale_mode=FP8_ROW_AMAX, glu_mode=GLU_CLAMP_REF, glu_fast_exp=0, use_graph=0,
                 eps=1e-6, clamp=10.0, rope: RopeParams | None = None):
        self.lib = _lib.load()
        if rope is None:
            rope = RopeParams()
            self.lib.ds4b200_rope_params_explicit(10000.0, 16.0, 4096, n_rot, C.byref(rope))
        self.cfg = PathConfig(n_tokens, n_embd, vocab, table_dtype, kv_dim, n_rot, n_slots, ff_dim, top_k,
                              max_layers, sinkhorn_iters, fp8_scale_mode, glu_mode, glu_fast_exp, use_graph,
                              eps, clamp, rope)
        self.handle = self.lib.ds4b200_path_create(C.byref(self.cfg))
        if not self.handle:
            raise _lib.Ds4Error("path_create: " + self.lib.ds4b200_last_error().decode())
        self.n_scales = (kv_dim - n_rot) // 64 if fp8_scale_mode == _lib.FP8_BLOCK64_POW2 else 1

    def close(self):
        if self.handle:
            self.lib.ds4b200_path_destroy(self.handle)
            self.handle = None

    def __del__(self):
        self.close()

    # -- setup ---------------------------------------------------------------
    def upload_table(self, table: np.ndarray):
        table = np.ascontiguousarray(table)
        check(self.lib.ds4b200_path_upload_table(self.handle, table.ctypes.data_as(C.c_void_p), table.nbytes))

    @staticmethod
    def _io(arrays: dict) -> PathIO:
        io = PathIO()
        for k, a in arrays.items():
            ptr = a.data_ptr() if hasattr(a, "data_ptr") else np.ascontiguousarray(a).ctypes.data
            setattr(io, k, ptr)
        return io

    def upload(self, inputs: dict):
        keep = {k: (v if hasattr(v, "data_ptr") else np.ascontiguousarray(v)) for k, v in inputs.items()}
        check(self.lib.ds4b200_path_upload(self.handle, C.byref(self._io(keep))))

    def buffer(self, name: str):
        n = C.c_int64()
        ptr = self.lib.ds4b200_path_buffer(self.handle, name.encode(), C.byref(n))
        return ptr, n.value

    @property
    def stream(self):
        return self.lib.ds4b200_path_stream(self.handle)

    # -- running -----------------------------------------------------------------
    def run_device(self, n_layers: int):
        check(self.lib.ds4b200_path_run_device(self.handle, n_layers))

    def output_shapes(self):
        c = self.cfg
        T = c.n_tokens
        return {"residual_out": ((T, c.n_embd), np.float32), "normed_bf16": ((T, c.n_embd), np.uint16),
                "kv_codes": ((T, c.kv_dim), np.uint8), "kv_scales": ((T, self.n_scales), np.float32),
                "kv_tail": ((T, c.n_rot), np.float32), "ffn_out": ((T, c.ff_dim), np.float32),
                "hc_out": ((T, 4, c.n_embd), np.float32)}

    def run_host(self, inputs: dict, n_layers: int, outputs: dict | None = None, n_chunks: int = 1) -> dict:
        """One end-to-end call on host arrays (numpy, or pinned torch tensors).
        n_chunks > 1 pipelines copy-in, compute and copy-out over row slices."""
        keep = {k: (v if hasattr(v, "data_ptr") else np.ascontiguousarray(v)) for k, v in inputs.items()}
        if outputs is None:
            outputs = {k: np.empty(s, dtype=d) for k, (s, d) in self.output_shapes().items()
                       if k != "kv_tail" or self.cfg.fp8_scale_mode == _lib.FP8_BLOCK64_POW2}
        io = self._io({**keep, **outputs})
        ms = C.c_float()
        if n_chunks > 1:
            check(self.lib.ds4b200_path_run_host_chunked(self.handle, C.byref(io), n_layers, n_chunks, C.byref(ms)))
        else:
            check(self.lib.ds4b200_path_run_host(self.handle, C.byref(io), n_layers, C.byref(ms)))
        res = dict(outputs)
        res["ms"] = ms.value
        return res

    def time_device(self, n_layers: int, warmup: int, steps: int) -> float:
        ms = C.c_float()
        check(self.lib.ds4b200_path_time_device(self.handle, n_layers, warmup, steps, C.byref(ms)))
        return ms.value

    def profile_ops(self, reps: int) -> dict:
        """Average ms per launch of each kernel (back-to-back launches of it alone)."""
        ms = (C.c_float * len(KERNELS))()
        check(self.lib.ds4b200_path_profile_ops(self.handle, reps, ms))
        return dict(zip(KERNELS, ms))

    def launches_per_run(self, n_layers: int) -> int:
        return self.lib.ds4b200_path_launches_per_run(self.handle, n_layers)

    def op_bytes(self, op: int) -> int:
        return self.lib.ds4b200_path_op_bytes(self.handle, op)
