"""CPU stand-in engine and helpers for zk_hillclimb_b200.p3.irs_prove (test infrastructure)."""
import ctypes as C

import numpy as np

from imm_helpers import OracleImmEngine
from lu_helpers import OracleLookupEngine, _Arr

GL_P = 0xFFFFFFFF00000001


def lift(a):
    a = np.asarray(a, dtype=np.int64)
    return np.where(a < 0, a.astype(np.uint64) + np.uint64(GL_P), a.astype(np.uint64))


def rescale_witness(acc_signed, sf, rng):
    """p3irs::gen_witness (zkllm-src/p3_int_gadgets.cuh:234-281) in numpy, signed inputs."""
    a = np.asarray(acc_signed, dtype=np.int64)
    H = 1 << (sf - 1)
    y = (a + H) >> sf
    rem = (a + H) - (y << sf)
    win = (1 << 19) if rng == 1 else (1 << 15)
    if rng and ((y < -win) | (y >= win)).any():
        raise ValueError("irs: y out of range (data too large)")
    nl = 1 if sf <= 16 else 2
    L = [lift(rem & 0xFFFF)] + ([lift(rem >> 16)] if nl == 2 else [])
    iL = [l.astype(np.uint32) for l in L]
    iY = (y + win).astype(np.uint32) if rng else None
    return lift(y), L, iL, iY


class OracleIrsEngine(OracleLookupEngine, OracleImmEngine):
    """CPU engine: the lookup and sumcheck stand-ins plus the rescale witness and table upload."""

    def __init__(self, orc):
        self.orc = orc

    def upload(self, arr):
        return _Arr(arr)

    def irs_witness(self, acc, sf, rng):
        a = acc.a.astype(np.int64)          # canonical field elements above p/2 are negative ints
        a = np.where(acc.a > np.uint64(GL_P >> 1), (acc.a - np.uint64(GL_P)).astype(np.int64), a)
        y, L, iL, iY = rescale_witness(a, sf, rng)
        return _Arr(y), [_Arr(l) for l in L], [_Arr(i) for i in iL], (_Arr(iY) if iY is not None else None)


def irs_tables(zk, sf):
    rt = zk.p3.range_table
    return {"R16": rt(16, 0), "R14": rt(14, 0), "RTOP": rt(sf - 16 if 16 < sf < 32 else 1, 0),
            "RS16": rt(16, -(1 << 15)), "RS20": rt(20, -(1 << 19))}


def ref_irs_verify(ref, st, rootX, rootY, le, sf, rng, R, Q, proof):
    s = (C.c_uint8 * 32)(*st)
    ok = ref.lib.ref_irs_verify(s, rootX, rootY, C.c_uint32(le), C.c_uint32(sf), C.c_int(rng), C.c_uint32(R),
                                C.c_uint32(Q), bytes(proof), C.c_size_t(len(proof)))
    return bool(ok), bytes(s)


def ref_irs_witness(ref, acc, le, sf, rng):
    N = 1 << le
    y, L0, L1 = (np.zeros(N, dtype=np.uint64) for _ in range(3))
    i0, i1, iY = (np.zeros(N, dtype=np.uint32) for _ in range(3))
    vp = lambda a: a.ctypes.data_as(C.c_void_p)
    nl = ref.lib.ref_irs_witness(vp(np.ascontiguousarray(acc)), C.c_uint32(le), C.c_uint32(sf), C.c_int(rng),
                                 vp(y), vp(L0), vp(L1), vp(i0), vp(i1), vp(iY))
    return nl, y, [L0, L1][:nl], [i0, i1][:nl], iY


class OracleStandaloneLuEngine(OracleIrsEngine):
    """Adds what the standalone lookup (p3.lu_prove) needs on top of the gadget engine."""

    def combine(self, cols, g):
        return _Arr(self.orc.combine([c.a for c in cols], g))

    def inv_all_add(self, A, beta):
        return _Arr(self.orc.inv_all_add(A.a, beta))

    def mul(self, a, b):
        return _Arr(np.array([int(x) * int(y) % GL_P for x, y in zip(a.a, b.a)], dtype=np.uint64))

    def prove_eval_dev(self, col, z, y, R, Q, cw0, seed):
        return self.orc.bf_prove_eval(col.a, np.ascontiguousarray(z, dtype=np.uint64), y, R, Q,
                                      self.orc.rs_encode(col.a, R), seed)


def ref_lu_prove_v(ref, st, tcols, wcols, committed, idx, R, Q, label, gpu):
    u64p, u32p = C.POINTER(C.c_uint64), C.POINTER(C.c_uint32)
    c = len(tcols)
    m = len(tcols[0]).bit_length() - 1
    n = len(idx).bit_length() - 1
    ta = [np.ascontiguousarray(t, dtype=np.uint64) for t in tcols]
    wa = [np.ascontiguousarray(w, dtype=np.uint64) for w in wcols]
    tp = (u64p * c)(*[a.ctypes.data_as(u64p) for a in ta])
    wp = (u64p * c)(*[a.ctypes.data_as(u64p) for a in wa])
    ix = np.ascontiguousarray(idx, dtype=np.uint32)
    s = (C.c_uint8 * 32)(*st)
    roots = (C.c_uint8 * (32 * c))()
    rA = np.zeros(n, dtype=np.uint64)
    cap = 64 << 20
    out = (C.c_uint8 * cap)()
    f = ref.lib.ref_lu_prove_v
    f.restype = C.c_size_t
    k = f(s, tp, C.c_uint32(m), C.c_uint32(c), wp, bytes(committed), ix.ctypes.data_as(u32p), C.c_uint32(n), C.c_uint32(R),
          C.c_uint32(Q), label.encode(), C.c_int(gpu), roots, rA.ctypes.data_as(u64p), out, C.c_size_t(cap))
    return bytes(out)[:k], bytes(s), [bytes(roots)[32 * i:32 * i + 32] for i in range(c)], rA


def ref_lu_verify_v(ref, st, tcols, wroots, committed, R, Q, label, proof):
    u64p = C.POINTER(C.c_uint64)
    c = len(tcols)
    m = len(tcols[0]).bit_length() - 1
    ta = [np.ascontiguousarray(t, dtype=np.uint64) for t in tcols]
    tp = (u64p * c)(*[a.ctypes.data_as(u64p) for a in ta])
    s = (C.c_uint8 * 32)(*st)
    rA = np.zeros(64, dtype=np.uint64)
    yv = np.zeros(64, dtype=np.uint64)
    ok = ref.lib.ref_lu_verify_v(s, tp, C.c_uint32(m), C.c_uint32(c), b"".join(wroots), bytes(committed), C.c_uint32(R),
                                 C.c_uint32(Q), label.encode(), bytes(proof), C.c_size_t(len(proof)),
                                 rA.ctypes.data_as(u64p), yv.ctypes.data_as(u64p))
    return bool(ok), bytes(s), rA, yv
