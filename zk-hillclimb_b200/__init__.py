"""B200 (sm_100a) prover kernels for the Goldilocks / Basefold proving path.

The directory name carries a hyphen, so import it through ``zkh_import.load()``
at the repository root (registers the package as ``zk_hillclimb_b200``).

Layout:
  csrc/       CUDA kernels and the C ABI (include/zkh.h) -> libzkh.so
  build.py    nvcc recipe (sm_100a, in-tree)
  _lib.py     ctypes binding of the C ABI; raises if the library is missing
  p3.py       host-side mirror of the reference's in-process prover interface
  ig.py       integer-layer gadgets (residual add, SwiGLU, ...) as host logic over the engine
  ig_dev.py   the layer's witness chain on the GPU (imported on demand; needs torch)
  hwl.py      the fp8 (Hawkeye) matmul gadget: tables, witness replay as tensor arithmetic, prover (on demand; needs torch)
  tfart.py    pinned table artefact of the fp8 transformer layer's bf16 gadgets (exact integer rounding; numpy)
  tfg.py      bf16 gadgets of the fp8 transformer layer (SwiGLU, ...) as host logic over the engine (on demand; needs torch)
  zkm.py      hiding mode: masks, salted commitments, blinded sumcheck, blinded batched openings, the zk matmul proof
  fr.py       host-side mirror of the BLS12-381 Fr pieces (eq tensors, folds, product sumchecks)
"""
from . import _lib  # noqa: F401
from ._lib import ZkhError, lib_path, load_library  # noqa: F401
from . import p3  # noqa: F401
from . import fr  # noqa: F401
from . import ig  # noqa: F401
from .p3 import (F_GKR, F_LOGUP, F_PROD2, F_PROD3, GL_P, Prover, Transcript)  # noqa: F401


def __getattr__(name):
    """The torch-based modules load on first use."""
    if name in ("hwl", "ig_dev", "tfg", "tfart", "zkm"):
        import importlib
        return importlib.import_module("." + name, __name__)
    raise AttributeError(name)
