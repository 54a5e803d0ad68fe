"""The standalone lookup (p3lu::prove_v, non-zk) on CUDA: same bytes as the oracle-backed run of the same
host logic, as the reference's host prover, and as the reference's CUDA path at a size where it takes it."""
import numpy as np
import pytest

from irs_helpers import OracleStandaloneLuEngine, ref_lu_prove_v, ref_lu_verify_v
from lu_helpers import _Arr, make_lookup

pytestmark = pytest.mark.gpu


def run_gpu(zk, prover, tcols, cols, idx, committed, R, Q, seed):
    import torch
    d = [zk.p3.to_device(c) for c in cols]
    W = [(x, prover.commit_gpu_rootonly(x, R) if k else None) for x, k in zip(d, committed)]
    tr = zk.Transcript(seed)
    pf, rA = zk.p3.lu_prove(prover, tr, W, torch.from_numpy(idx.view(np.int32)).cuda(), zk.p3.make_table(tcols), R, Q, "lut")
    return pf, rA, tr.state, W


@pytest.mark.parametrize("m,n,committed", [(4, 5, [1, 1]), (8, 12, [1, 0]), (10, 9, [1, 1])])
def test_matches_oracle_engine_and_reference_host(orc, ref_or_none, zk, prover, m, n, committed):
    R, Q = 1, 24
    tcols, subs = make_lookup(orc, m, [(n, 1)], 7 + m + n)
    cols, idx = subs[0][1][0]
    pf, rA, st, W = run_gpu(zk, prover, tcols, cols, idx, committed, R, Q, "lu-standalone")
    eng = OracleStandaloneLuEngine(orc)
    oW = [(_Arr(c), eng.commit_gpu_rootonly(_Arr(c), R) if k else None) for c, k in zip(cols, committed)]
    tr2 = zk.Transcript("lu-standalone")
    pf2, rA2 = zk.p3.lu_prove(eng, tr2, oW, _Arr(idx), zk.p3.make_table(tcols), R, Q, "lut")
    assert pf == pf2 and st == tr2.state
    if ref_or_none is not None and n <= 10:
        rpf, rst, _, _ = ref_lu_prove_v(ref_or_none, zk.Transcript("lu-standalone").state, tcols, cols, committed, idx, R, Q, "lut", 0)
        assert rpf == pf and rst == st
    if ref_or_none is not None:
        roots = [w[1] if w[1] is not None else b"\0" * 32 for w in W]
        ok, vst, _, _ = ref_lu_verify_v(ref_or_none, zk.Transcript("lu-standalone").state, tcols, roots, committed, R, Q, "lut", pf)
        assert ok and vst == st


def test_matches_reference_cuda_path(orc, ref, zk, prover):
    if not ref.gpu_available():
        pytest.skip("reference shim sees no GPU")
    R, Q = 1, 24
    m, n = 12, 17                     # n >= 16: the reference runs its device-resident sumcheck
    tcols, subs = make_lookup(orc, m, [(n, 1)], 123)
    cols, idx = subs[0][1][0]
    pf, rA, st, W = run_gpu(zk, prover, tcols, cols, idx, [1, 1], R, Q, "lu-cuda")
    rpf, rst, rroots, rrA = ref_lu_prove_v(ref, zk.Transcript("lu-cuda").state, tcols, cols, [1, 1], idx, R, Q, "lut", 1)
    assert rroots == [w[1] for w in W]
    assert rpf == pf and rst == st
