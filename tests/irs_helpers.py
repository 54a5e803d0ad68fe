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
