"""Quartic zero-check sumchecks of the fp8 gadget's constraint summands (p3hwl::sc5_run, non-zk) on CUDA:
messages, challenges, final column values and transcript equal to the reference's host loop over its own
constraint functions (golden vectors; live through oracle/_ref when present) and to the reference's CUDA
engine for the four summands it runs on the GPU."""
import numpy as np
import pytest

from conftest import dig

pytestmark = pytest.mark.gpu

HW_SHAPE = {6: (12, 6), 7: (30, 18), 8: (11, 6), 9: (3, 2), 10: (8, 6), 11: (57, 49)}


def instance(orc, f, logn, seed):
    nc, nlam = HW_SHAPE[f]
    s, cols = seed, []
    for _ in range(nc):
        a, s = orc.lcg(1 << logn, s)
        cols.append(a)
    lam, s = orc.lcg(nlam, s)
    return cols, lam


def test_golden_vectors(golden, orc, zk, prover):
    for gv in golden["hawkeye_sumcheck"]:
        cols, lam = instance(orc, gv["functor"], gv["logn"], gv["seed"])
        tr = zk.Transcript("hw-golden")
        r, m, fin = prover.sc5_run(tr, gv["tag"], [zk.p3.to_device(c) for c in cols], gv["functor"], lam)
        assert tr.state.hex() == gv["state"], gv
        assert dig(m) == gv["msgs_digest"] and [int(x) for x in r] == gv["chals"]
        for c, y in zip(cols, fin):
            assert orc.mle_eval(c, r) == int(y)


@pytest.mark.parametrize("f", sorted(HW_SHAPE))
@pytest.mark.parametrize("logn", [2, 10, 15])
def test_matches_reference_host_loop(orc, ref_or_none, zk, prover, f, logn):
    if ref_or_none is None:
        pytest.skip("reference shim not built")
    cols, lam = instance(orc, f, logn, 1000 + 31 * f + logn)
    tr = zk.Transcript("hw-live")
    r, m, fin = prover.sc5_run(tr, "hwl-dp", [zk.p3.to_device(c) for c in cols], f, lam)
    st, rm, rr = ref_or_none.sc5_prove_lam(zk.Transcript("hw-live").state, "hwl-dp", f, cols, lam)
    assert st == tr.state and (rm == m).all() and (rr == r).all()
    assert orc.mle_eval(cols[-1], r) == int(fin[-1]) and orc.mle_eval(cols[0], r) == int(fin[0])


@pytest.mark.parametrize("f", [6, 7, 8, 9])
def test_matches_reference_cuda_engine(orc, ref, zk, prover, f):
    if not ref.gpu_available():
        pytest.skip("reference shim sees no GPU")
    logn = 17
    cols, lam = instance(orc, f, logn, 77 + f)
    tr = zk.Transcript("hw-cuda")
    r, m, fin = prover.sc5_run(tr, "hwl-dg", [zk.p3.to_device(c) for c in cols], f, lam)
    st, rm, rr, _ms = ref.sc_prove_gpu(zk.Transcript("hw-cuda").state, "hwl-dg", f, 5, cols, [int(x) for x in lam])
    assert st == tr.state and (rm == m).all() and (rr == r).all()


def test_argument_checks(zk, prover):
    cols = [zk.p3.to_device(np.zeros(4, dtype=np.uint64)) for _ in range(3)]
    with pytest.raises(Exception):
        prover.sc5_run(zk.Transcript("x"), "t", cols, 9, [1])                       # wrong coefficient count
    with pytest.raises(Exception):
        prover.sc5_run(zk.Transcript("x"), "t", cols[:2], 9, [1, 2])                # wrong column count
    with pytest.raises(Exception):
        prover.sc5_run(zk.Transcript("x"), "t", cols, 9, [1, 0xFFFFFFFF00000001])   # non-canonical coefficient
    with pytest.raises(Exception):
        prover.sc5_run(zk.Transcript("x"), "t", cols, 2, [1, 2])                    # not a wide summand
