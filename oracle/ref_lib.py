"""ctypes binding of oracle/_ref/libds4ref.so: the reference's own CUDA
launchers for this path, rebuilt for sm_100a by `make -C oracle ref`.

Test infrastructure: used on a GPU box to check the product kernels and the CPU
oracle against the real reference, and to time the reference kernels beside
ours.  Arguments are torch CUDA tensors; the default stream is used.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "_ref" / "libds4ref.so"
_lib = None


def reference_tree() -> Path | None:
    """Where the reference's sources are, if they are reachable from here: $DS4_REFERENCE, else a
    directory named `reference` beside this repository.  None on a box that only has the built library."""
    import os
    cand = os.environ.get("DS4_REFERENCE")
    path = Path(cand) if cand else Path(__file__).resolve().parent.parent.parent / "reference"
    return path if (path / "cuda" / "norm.cu").exists() else None


def available() -> bool:
    return LIB_PATH.exists()


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(str(LIB_PATH))
    return _lib


def _p(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream():
    import torch
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def call(name: str, *args) -> None:
    """Call ds4ref_<name>; tensors become pointers, floats c_float, ints c_int."""
    fn = getattr(lib(), "ds4ref_" + name)
    fn.restype = None
    conv = []
    for a in args:
        if hasattr(a, "data_ptr") or a is None:
            conv.append(_p(a))
        elif isinstance(a, float):
            conv.append(C.c_float(a))
        else:
            conv.append(C.c_int(int(a)))
    fn(*conv, _stream())
