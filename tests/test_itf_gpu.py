"""One decoder layer on CUDA: same proof bytes as the oracle-backed run of the same host logic and as the
reference's own layer prover (witness on the host, commitments / lookups / openings on the GPU); accepted by the
reference's layer verifier."""
import numpy as np
import pytest

from ig_helpers import OracleGadgetEngine, arr, layer_inputs, ref_itf_prove, ref_itf_verify

pytestmark = pytest.mark.gpu


def device_col(zk):
    import torch

    def col(a):
        a = np.ascontiguousarray(a)
        return torch.from_numpy(a.view(np.int32)).cuda() if a.dtype == np.uint32 else zk.p3.to_device(a)
    return col


@pytest.mark.parametrize("dims", [(4, 8, 2, 4, 16, 1), (16, 32, 2, 16, 64, 1)])
def test_layer_same_bytes(orc, ref_or_none, zk, prover, dims):
    R, Q = 1, 24
    ig = zk.ig
    c = ig.Config(*dims)
    T = ig.build_tables(zk.load_library(), c.d, c.btop)
    x0, Wt = layer_inputs(ig, c, 5)
    w = ig.itf_build_witness(c, x0, Wt, T)
    col = device_col(zk)
    o = ig.itf_commit_all(prover, w, Wt, R, col)
    tr = zk.Transcript("itf-layer")
    pf = ig.itf_prove(prover, tr, c, w, o, Wt, T, R, Q, col)
    if dims[0] <= 4:                                    # the Python-integer engine is slow: smallest shape only
        eng = OracleGadgetEngine(orc)
        ocol = lambda a: arr(eng, a)
        oo = ig.itf_commit_all(eng, w, Wt, R, ocol)
        tr2 = zk.Transcript("itf-layer")
        assert ig.itf_prove(eng, tr2, c, w, oo, Wt, T, R, Q, ocol) == pf and tr2.state == tr.state
    if ref_or_none is not None:
        wroots = [x[1] for x in o["w"]] + [o["g1"][1], o["g2"][1]]
        ok, st = ref_itf_verify(ref_or_none, zk.Transcript("itf-layer").state, c, x0, o["x0"][1], wroots, Wt, w["out"], R, Q, pf)
        assert ok and st == tr.state
        if ref_or_none.gpu_available():
            rpf, rst, grid, ms = ref_itf_prove(ref_or_none, zk.Transcript("itf-layer").state, c, x0, Wt, R, Q)
            assert (grid == w["out"]).all()             # the witness chains agree
            assert rpf == pf and rst == tr.state
