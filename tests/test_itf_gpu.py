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


def _same(a, b):
    import torch
    if isinstance(a, (list, tuple)):
        return len(a) == len(b) and all(_same(x, y) for x, y in zip(a, b))
    if isinstance(a, dict):
        return all(_same(a[k], b[k]) for k in a)
    if a is None:
        return b is None
    if isinstance(b, torch.Tensor):
        b = b.cpu().numpy()
        if b.dtype == np.int32:
            b = b.view(np.uint32)
        elif b.dtype == np.int64:
            b = b.view(np.uint64)
    a = np.asarray(a)
    if a.dtype == np.int64:                      # signed host columns (RoPE's public C, S2) against signed device columns
        return bool((a == b.view(np.int64)).all())
    return bool((a.astype(np.uint64) == b.astype(np.uint64)).all())


@pytest.mark.parametrize("dims", [(4, 8, 2, 4, 16, 2), (32, 64, 4, 16, 128, 1)])
def test_device_witness_chain_equals_host_chain(zk, prover, dims):
    """The GPU witness chain (ig_dev) reproduces every column and index array of the host chain, and the proof
    built from it is the same."""
    from zk_hillclimb_b200 import ig_dev
    R, Q = 1, 24
    ig = zk.ig
    c = ig.Config(*dims)
    T = ig.build_tables(zk.load_library(), c.d, c.btop)
    x0, Wt = layer_inputs(ig, c, 9)
    w = ig.itf_build_witness(c, x0, Wt, T)
    wd = ig_dev.itf_build_witness(c, x0, Wt, T, engine=prover)
    px0, pW = ig_dev.pin_inputs(x0, Wt)          # the same chain from signed int32 inputs in pinned memory
    wp = ig_dev.itf_build_witness(c, px0, pW, T, engine=prover)
    for k, v in w.items():
        assert _same(v, wp[k]), k
    for k, v in w.items():
        assert _same(v, wd[k]), k
    ident = lambda a: a
    od = ig.itf_commit_all(prover, wd, wd["dev_W"], R, ident)
    trd = zk.Transcript("itf-layer")
    pfd = ig.itf_prove(prover, trd, c, wd, od, Wt, T, R, Q, ident)
    col = device_col(zk)
    o = ig.itf_commit_all(prover, w, Wt, R, col)
    tr = zk.Transcript("itf-layer")
    assert ig.itf_prove(prover, tr, c, w, o, Wt, T, R, Q, col) == pfd and tr.state == trd.state
