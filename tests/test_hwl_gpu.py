"""The fp8 (Hawkeye) matmul gadget on CUDA: witness replay on the GPU equals the reference's host replay, the proof
bytes equal the reference's own CUDA prover's, and the reference's host-only verifier accepts."""
import numpy as np
import pytest

from hwl_helpers import layer_inputs, ref_hwl_prove, ref_hwl_verify, ref_witness_column

pytestmark = pytest.mark.gpu


def device_witness(zk, prover, dims, inp, kernel=True):
    """kernel: the CUDA replay kernel (zkh_hwl_witness); otherwise the tensor-arithmetic replay on the same GPU"""
    if kernel:
        return zk.hwl.gen_witness_dev(prover, *dims, *inp)
    return zk.hwl.gen_witness(*dims, *inp, device="cuda:%d" % prover.device, inverse=lambda t: prover.inv_all_add(t.contiguous(), 0))


@pytest.mark.parametrize("kernel", [True, False])
@pytest.mark.parametrize("dims", [(2, 32, 2), (3, 70, 5), (16, 96, 24), (1, 1, 1)])
def test_device_witness_equals_reference_replay(ref, zk, prover, dims, kernel):
    hwl = zk.hwl
    inp = layer_inputs(*dims, seed=sum(dims))
    wt = device_witness(zk, prover, dims, inp, kernel)
    assert (wt["Y"] == hwl.gen_witness(*dims, *inp)["Y"]).all()
    for dom, name, ncol in ((0, "dp", hwl.NDP), (1, "dg", hwl.NDG), (2, "dob", hwl.NDO), (3, "db", hwl.NDS), (4, "dn", hwl.NDS)):
        for c in range(ncol):
            mine = zk.p3.to_host(wt[name][c])
            assert (ref_witness_column(ref, dims, inp, dom, c, len(mine)) == mine).all(), (name, c)
    for i in range(hwl.NLU):
        mine = wt["lidx"][i].cpu().numpy().view(np.uint32)
        assert (ref_witness_column(ref, dims, inp, 5, i, len(mine), idx=True) == mine).all(), i


@pytest.mark.parametrize("dims,R,Q", [((2, 32, 2), 1, 24), ((5, 100, 12), 1, 24), ((16, 128, 32), 2, 24)])
def test_proof_equals_reference_prover_and_verifies(ref, zk, prover, dims, R, Q):
    hwl = zk.hwl
    T = hwl.build_tables()
    inp = layer_inputs(*dims, seed=11 + dims[1])
    wt = device_witness(zk, prover, dims, inp)
    col = lambda t: t
    ops = hwl.commit_operands(prover, wt, R, col)
    tr = zk.Transcript("hwl-layer")
    pf = hwl.prove(prover, tr, wt, T, ops, R, Q, col)
    roots4 = [ops[k][1] for k in ("X", "W", "XS", "WS")]
    st0 = zk.Transcript("hwl-layer").state
    ok, st = ref_hwl_verify(ref, st0, dims, roots4, wt["Y"], R, Q, pf)
    assert ok and st == tr.state
    badY = wt["Y"].copy()
    badY[0] ^= 0x80
    assert not ref_hwl_verify(ref, st0, dims, roots4, badY, R, Q, pf)[0]
    if ref.gpu_available():
        rpf, rst, rroots, rY, _ms = ref_hwl_prove(ref, st0, dims, inp, R, Q)
        assert rroots == roots4 and (rY == wt["Y"]).all()
        assert rpf == pf and rst == tr.state


def test_kept_trees_give_the_same_proof(zk, prover):
    hwl = zk.hwl
    dims, R, Q = (8, 64, 16), 1, 24
    T = hwl.build_tables()
    inp = layer_inputs(*dims, seed=5)
    wt = device_witness(zk, prover, dims, inp)
    col = lambda t: t
    outs = []
    for keep in (False, True):
        prover.keep_trees = keep
        try:
            ops = hwl.commit_operands(prover, wt, R, col)
            tr = zk.Transcript("hwl-layer")
            outs.append((hwl.prove(prover, tr, wt, T, ops, R, Q, col), tr.state))
        finally:
            prover.release_kept()
            prover.keep_trees = False
    assert outs[0] == outs[1]


def test_replay_kernel_equals_tensor_replay_at_scale(zk, prover):
    """64 x 512 . 512 x 128 (2^22 padded products): every column of the kernel equals the tensor-arithmetic replay."""
    dims = (64, 512, 128)
    inp = layer_inputs(*dims, seed=99)
    a, b = device_witness(zk, prover, dims, inp, True), device_witness(zk, prover, dims, inp, False)
    for name in ("dp", "dg", "dob", "db", "dn", "lidx"):
        for c, (u, v) in enumerate(zip(a[name], b[name])):
            assert bool((u == v).all()), (name, c)
    assert bool((a["va"] == b["va"]).all()) and bool((a["vb"] == b["vb"]).all()) and (a["Y"] == b["Y"]).all()


def test_replay_kernel_rejects_unsupported_scale(zk, prover):
    x, w, xs, ws = layer_inputs(2, 32, 2, seed=3)
    ws = ws.copy()
    ws[1] = 0x00000001                                  # subnormal scale
    with pytest.raises(zk.hwl.WitnessError, match="subnormal w-scale"):
        zk.hwl.gen_witness_dev(prover, 2, 32, 2, x, w, xs, ws)
