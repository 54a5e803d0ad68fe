"""CPU stand-in engine for zk_hillclimb_b200.p3.imm_prove built on the oracle (test infrastructure)."""
import ctypes as C

import numpy as np

from lu_helpers import _Arr

GL_P = 0xFFFFFFFF00000001


class OracleImmEngine:
    def __init__(self, orc):
        self.orc = orc

    def build_eq_gpu(self, z):
        return _Arr(self.orc.build_eq(np.ascontiguousarray(z, dtype=np.uint64)))

    def eval_h_gpu(self, col, z):
        return self.orc.mle_eval(col.a, np.ascontiguousarray(z, dtype=np.uint64))

    def element(self, col, i):
        return int(col.a[i])

    def matvec(self, M, rows, cols, w, along_rows):
        A = M.a.astype(object).reshape(rows, cols)
        ww = w.a.astype(object)
        out = (A * ww[None, :]).sum(axis=1) if along_rows else (A * ww[:, None]).sum(axis=0)
        return _Arr(np.array([int(x) % GL_P for x in out], dtype=np.uint64))

    def scale(self, col, s):
        return _Arr(np.array([int(x) * s % GL_P for x in col.a], dtype=np.uint64))

    def sc_prove_gpu(self, tr, tag, cols, functor, nt, par=()):
        st, m, r, fin = self.orc.sumcheck(tr.state, tag, functor, nt, [c.a for c in cols], par)
        tr.state = st
        return r, m, fin

    def prove_class(self, tr, pts, ents, R, Q, label):
        pf, st = self.orc.bo_prove_class(tr.state, pts, [e[0].a for e in ents], [e[1] for e in ents],
                                         [e[2] for e in ents], R, Q, label)
        tr.state = st
        return pf


def matmul_instance(orc, lj, lk, li, seed):
    """int8-style operands lifted into the field (BASELINE configs[0] shape, scaled down by the caller)."""
    rng = np.random.default_rng(seed)
    J, K, I = 1 << lj, 1 << lk, 1 << li
    Xi = rng.integers(-127, 128, (I, J))
    Wi = rng.integers(-127, 128, (J, K))
    Yi = Xi @ Wi
    lift = lambda a: np.array([int(v) % GL_P for v in a.reshape(-1)], dtype=np.uint64)
    return lift(Xi), lift(Wi), lift(Yi)      # X[j | i<<lj], W[k | j<<lk], Y[k | i<<lk]


def ref_imm_verify(ref, st, roots, lj, lk, li, R, Q, proof):
    s = (C.c_uint8 * 32)(*st)
    ok = ref.lib.ref_imm_verify(s, roots[0], roots[1], roots[2], C.c_uint32(lj), C.c_uint32(lk), C.c_uint32(li),
                                C.c_uint32(R), C.c_uint32(Q), bytes(proof), C.c_size_t(len(proof)))
    return bool(ok), bytes(s)
