"""The integer matmul gadget (p3imm::prove, non-zk) on CUDA: same bytes as the oracle-backed run of the
same host logic, accepted by the reference verifier, equal to the reference's own CUDA prover."""
import ctypes as C

import numpy as np
import pytest

from imm_helpers import OracleImmEngine, matmul_instance, ref_imm_verify
from lu_helpers import _Arr

pytestmark = pytest.mark.gpu


def gpu_operands(zk, prover, X, W, Y, R):
    d = [zk.p3.to_device(c) for c in (X, W, Y)]
    roots = [prover.commit_gpu_rootonly(x, R) for x in d]
    return d, roots


@pytest.mark.parametrize("lj,lk,li", [(3, 2, 2), (1, 1, 1), (5, 5, 4), (8, 7, 5), (10, 10, 7)])
def test_imm_prove_matches_oracle_engine(orc, ref_or_none, zk, prover, lj, lk, li):
    R, Q = 1, 24
    X, W, Y = matmul_instance(orc, lj, lk, li, 7 + lj)
    d, roots = gpu_operands(zk, prover, X, W, Y, R)
    tr = zk.Transcript("imm")
    pf = zk.p3.imm_prove(prover, tr, (d[0], roots[0]), (d[1], roots[1]), (d[2], roots[2]), lj, lk, li, R, Q)
    if lj + lk + li <= 16:
        tr2 = zk.Transcript("imm")
        pf2 = zk.p3.imm_prove(OracleImmEngine(orc), tr2, (_Arr(X), roots[0]), (_Arr(W), roots[1]), (_Arr(Y), roots[2]),
                              lj, lk, li, R, Q)
        assert pf == pf2 and tr.state == tr2.state
    if ref_or_none:
        ok, st = ref_imm_verify(ref_or_none, zk.Transcript("imm").state, roots, lj, lk, li, R, Q, pf)
        assert ok and st == tr.state


def test_reference_cuda_imm_same_bytes(orc, ref, zk, prover):
    if not ref.gpu_available():
        pytest.skip("reference shim sees no GPU")
    lj, lk, li, R, Q = 6, 6, 5, 1, 24
    X, W, Y = matmul_instance(orc, lj, lk, li, 321)
    d, roots = gpu_operands(zk, prover, X, W, Y, R)
    tr = zk.Transcript("imm-ref")
    pf = zk.p3.imm_prove(prover, tr, (d[0], roots[0]), (d[1], roots[1]), (d[2], roots[2]), lj, lk, li, R, Q)
    u64p = C.POINTER(C.c_uint64)
    st = (C.c_uint8 * 32)(*zk.Transcript("imm-ref").state)
    out = (C.c_uint8 * (8 << 20))()
    ms = C.c_double(0)
    f = ref.lib.ref_imm_prove
    f.restype = C.c_size_t
    n = f(st, X.ctypes.data_as(u64p), W.ctypes.data_as(u64p), Y.ctypes.data_as(u64p), roots[0], roots[1], roots[2],
          C.c_uint32(lj), C.c_uint32(lk), C.c_uint32(li), C.c_uint32(R), C.c_uint32(Q), out, C.c_size_t(8 << 20),
          C.byref(ms))
    assert n > 0 and bytes(out)[:n] == pf and bytes(st) == tr.state
