"""Operand views as maps on index bits: the detection of such a map from an index function (host) and the gather /
scatter kernels behind Prover.gather_fn / scatter_fn (p3imm::op_off / y_off, zkllm-src/p3_int_gadgets.cuh:448-470)."""
import numpy as np
import pytest


def head_view(zk):
    """The X view of a per-head product: lane bits, head constant, position bits."""
    from zk_hillclimb_b200.p3 import S_A, S_C, S_J
    return [(S_J, 0), (S_J, 1), (S_J, 2), (S_C, 1), (S_C, 0), (S_A, 0), (S_A, 1), (S_A, 2), (S_A, 3)]


def test_bit_map_detection(zk):
    from zk_hillclimb_b200 import zkm
    from zk_hillclimb_b200.p3 import S_A, S_J
    P = zk.p3.Prover
    xv = head_view(zk)
    fn = lambda t: zkm._view_index(xv, {S_J: t & 7, S_A: t >> 3}) | (1 << 9)
    konst, masks, nb = P._bit_map(fn, 128)
    u = np.arange(128, dtype=np.int64)
    got = np.full(128, konst, dtype=np.int64)
    for b in range(nb):
        got |= np.where((u >> b) & 1, masks.view(np.int64)[b], 0)
    assert (got == fn(u)).all()
    assert P._bit_map(lambda q: (q * 3) & 127, 128) is None            # not a map on bits
    assert P._bit_map(lambda q: (q + 1) & 127, 128) is None
    assert P._bit_map(lambda q: ((q >> 5) << 2) | ((q & 31) >> 3), 1 << 10) is not None   # broadcast pattern


@pytest.mark.gpu
def test_gather_and_scatter_kernels(zk, prover):
    import torch
    from zk_hillclimb_b200 import zkm
    from zk_hillclimb_b200.p3 import S_A, S_J
    xv = head_view(zk)
    fn = lambda t: zkm._view_index(xv, {S_J: t & 7, S_A: t >> 3})
    rng = np.random.default_rng(5)
    col = rng.integers(0, 1 << 62, 1 << 9, dtype=np.int64)
    d = torch.from_numpy(col).cuda()
    u = np.arange(128, dtype=np.int64)
    out = prover.gather_fn(d, 128, fn)
    assert (out.cpu().numpy() == col[fn(u)]).all()
    # a map that is not on bits takes the tensor path and gives the same kind of result
    out2 = prover.gather_fn(d, 128, lambda q: (q * 3) & 127)
    assert (out2.cpu().numpy() == col[(u * 3) & 127]).all()
    vals = torch.from_numpy(rng.integers(0, 1 << 62, 128, dtype=np.int64)).cuda()
    tgt = prover.scatter_fn(torch.zeros(1 << 9, dtype=torch.int64, device="cuda"), 128, fn, vals)
    want = np.zeros(1 << 9, dtype=np.int64)
    want[fn(u)] = vals.cpu().numpy()
    assert (tgt.cpu().numpy() == want).all()
    with pytest.raises(Exception):
        prover.gather_fn(d[:256], 128, fn)           # the view reaches beyond the column
