"""CPU stand-in engine, seeded inputs and reference windows for the fp8 (Hawkeye) matmul gadget (test infrastructure)."""
import ctypes as C

import numpy as np

from ig_helpers import OracleGadgetEngine
from lu_helpers import _Arr


class OracleHwlEngine(OracleGadgetEngine):
    """The gadget engine plus the fp8 gadget's quartic summands, evaluated by the reference's host loop sc5_prove."""

    def __init__(self, orc, ref):
        super().__init__(orc)
        self.ref = ref

    def sc5_run(self, tr, tag, cols, functor, lam):
        st, m, r = self.ref.sc5_prove_lam(tr.state, tag, functor, [c.a for c in cols], lam)
        tr.state = st
        return r, m, None


def host_col(t):
    """witness tensor (CPU) -> numpy-backed engine column"""
    a = t.numpy()
    return _Arr(a.view(np.uint64) if a.dtype == np.int64 else a.view(np.uint32))


def layer_inputs(B, K, N, seed):
    """Seeded fp8-e4m3 codes (NaN codes 0x7f / 0xff excluded) and positive normal fp32 scales."""
    rng = np.random.default_rng(seed)
    codes = lambda n: rng.choice(np.array([c for c in range(256) if c & 0x7F != 0x7F], dtype=np.uint8), size=n)
    x, w = codes(B * K), codes(N * K)
    xs = np.abs(rng.normal(1.0, 0.3, size=B)).astype(np.float32) + np.float32(0.01)
    ws = np.abs(rng.normal(0.02, 0.005, size=N)).astype(np.float32) + np.float32(0.001)
    return x, w, xs.view(np.uint32), ws.view(np.uint32)


_vp = lambda a: a.ctypes.data_as(C.c_void_p)


def ref_witness_column(ref, dims, inp, dom, c, n, idx=False):
    f = ref.lib.ref_hwl_witness
    f.restype = C.c_size_t
    x, w, xs, ws = inp
    out = np.zeros(n, dtype=np.uint32 if idx else np.uint64)
    got = f(*[C.c_uint32(v) for v in dims], _vp(x), _vp(w), _vp(xs), _vp(ws), dom, c, None if idx else _vp(out), _vp(out) if idx else None)
    assert got == n, (dom, c, got, n)
    return out


def ref_hwl_verify(ref, st, dims, roots4, Y, R, Q, proof):
    s = (C.c_uint8 * 32)(*st)
    Yc = np.ascontiguousarray(Y, dtype=np.uint16)
    ok = ref.lib.ref_hwl_verify(s, *[C.c_uint32(v) for v in dims], b"".join(roots4), _vp(Yc), C.c_uint32(R), C.c_uint32(Q),
                                bytes(proof), C.c_size_t(len(proof)))
    return bool(ok), bytes(s)


def ref_hwl_prove(ref, st, dims, inp, R, Q, gpu=True):
    """The reference's own gen_witness + commit_operands + prove: (proof bytes, state, operand roots, Y, [ms])."""
    s = (C.c_uint8 * 32)(*st)
    x, w, xs, ws = inp
    cap = 512 << 20
    out = (C.c_uint8 * cap)()
    roots = (C.c_uint8 * 128)()
    Y = np.zeros(dims[0] * dims[2], dtype=np.uint16)
    ms = (C.c_double * 3)()
    f = ref.lib.ref_hwl_prove
    f.restype = C.c_size_t
    n = f(s, *[C.c_uint32(v) for v in dims], _vp(x), _vp(w), _vp(xs), _vp(ws), C.c_uint32(R), C.c_uint32(Q), int(gpu), roots, _vp(Y),
          out, C.c_size_t(cap), ms)
    rb = bytes(roots)
    return bytes(out[:n]), bytes(s), [rb[i * 32:(i + 1) * 32] for i in range(4)], Y, list(ms)
