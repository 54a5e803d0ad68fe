"""The rescale gadget (p3irs::prove, non-zk) on CUDA: witness kernel equal to the reference's replay,
proof bytes equal to the oracle-backed run of the same host logic and to the reference's own prover,
accepted by the reference's verifier."""
import ctypes as C

import numpy as np
import pytest

from irs_helpers import OracleIrsEngine, irs_tables, lift, ref_irs_verify, rescale_witness
from lu_helpers import _Arr
from test_irs_host_logic import instance

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("le,sf,rng", [(10, 16, 1), (13, 14, 2), (12, 23, 1), (9, 32, 0), (17, 16, 1)])
def test_witness_kernel(zk, prover, le, sf, rng):
    acc = instance(le, sf, rng, le + sf)
    y, L, iL, iY = prover.irs_witness(zk.p3.to_device(lift(acc)), sf, rng)
    ey, eL, eiL, eiY = rescale_witness(acc, sf, rng)
    assert (zk.p3.to_host(y) == ey).all()
    for a, b in zip(L, eL):
        assert (zk.p3.to_host(a) == b).all()
    for a, b in zip(iL, eiL):
        assert (a.cpu().numpy().view(np.uint32) == b).all()
    if rng:
        assert (iY.cpu().numpy().view(np.uint32) == eiY).all()


@pytest.mark.parametrize("le,sf,rng", [(6, 16, 1), (10, 14, 2), (12, 23, 1), (9, 32, 0), (14, 16, 1)])
def test_irs_prove_matches_oracle_and_reference_verifier(orc, ref_or_none, zk, prover, le, sf, rng):
    R, Q = 1, 24
    acc_h = lift(instance(le, sf, rng, 7 * le + sf))
    acc = zk.p3.to_device(acc_h)
    y, L, iL, iY = prover.irs_witness(acc, sf, rng)
    X = (acc, prover.commit_gpu_rootonly(acc, R))
    Y = (y, prover.commit_gpu_rootonly(y, R))
    tr = zk.Transcript("irs-main")
    pf = zk.p3.irs_prove(prover, tr, irs_tables(zk, sf), X, Y, (L, iL, iY), le, sf, rng, R, Q)
    eng = OracleIrsEngine(orc)
    oacc = _Arr(acc_h)
    oy, oL, oiL, oiY = eng.irs_witness(oacc, sf, rng)
    tr2 = zk.Transcript("irs-main")
    pf2 = zk.p3.irs_prove(eng, tr2, irs_tables(zk, sf), (oacc, eng.commit_gpu_rootonly(oacc, R)),
                          (oy, eng.commit_gpu_rootonly(oy, R)), (oL, oiL, oiY), le, sf, rng, R, Q)
    assert pf == pf2 and tr.state == tr2.state
    if ref_or_none:
        ok, st = ref_irs_verify(ref_or_none, zk.Transcript("irs-main").state, X[1], Y[1], le, sf, rng, R, Q, pf)
        assert ok and st == tr.state


@pytest.mark.parametrize("le,sf,rng", [(10, 16, 1), (12, 23, 2)])
def test_reference_prover_same_bytes(ref, zk, prover, le, sf, rng):
    if not ref.gpu_available():
        pytest.skip("reference shim sees no GPU")
    R, Q = 1, 24
    acc_h = lift(instance(le, sf, rng, 3))
    acc = zk.p3.to_device(acc_h)
    y, L, iL, iY = prover.irs_witness(acc, sf, rng)
    X = (acc, prover.commit_gpu_rootonly(acc, R))
    Y = (y, prover.commit_gpu_rootonly(y, R))
    tr = zk.Transcript("irs-ref")
    pf = zk.p3.irs_prove(prover, tr, irs_tables(zk, sf), X, Y, (L, iL, iY), le, sf, rng, R, Q)
    st = (C.c_uint8 * 32)(*zk.Transcript("irs-ref").state)
    out = (C.c_uint8 * (8 << 20))()
    ms = C.c_double(0)
    f = ref.lib.ref_irs_prove
    f.restype = C.c_size_t
    n = f(st, acc_h.ctypes.data_as(C.c_void_p), X[1], Y[1], C.c_uint32(le), C.c_uint32(sf), C.c_int(rng),
          C.c_uint32(R), C.c_uint32(Q), out, C.c_size_t(8 << 20), C.byref(ms))
    assert n > 0 and bytes(out)[:n] == pf and bytes(st) == tr.state
