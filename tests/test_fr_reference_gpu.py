"""The Fr path against the UNMODIFIED reference's own CUDA code (oracle/_ref/libfrref.so, built from the
reference's bls12-381.cu, fr-tensor.cu, zkfc.cu, zkob_lookup.cuh ...): this is the pin of both the
Python-integer oracle and the CUDA kernels here for the BLS12-381 stack."""
import random

import pytest

import fr_oracle as fo

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def refA():
    if not fo.ReferenceFr.available():
        pytest.skip("oracle/_ref/libfrref.so not built")
    r = fo.ReferenceFr()
    if not r.gpu_available():
        pytest.skip("reference shim sees no GPU")
    return r


def rnd(rng, n, small=False):
    if small:
        return [rng.randrange(-(1 << 20), 1 << 20) % fo.P for _ in range(n)]
    return [rng.randrange(fo.P) for _ in range(n)]


def test_fold_eq_and_me(refA, zk, prover):
    rng = random.Random(11)
    fr = zk.fr
    t = [0, 1, fo.P - 1, fo.P - 2] + rnd(rng, 252)
    w = rng.randrange(fo.P)
    ref_fold = refA.fold(t, w)
    assert ref_fold == fo.fold(t, w) == fr.to_host(fr.fr_fold(prover, fr.to_device(t), w))
    u = rnd(rng, 8)
    assert refA.eq_build(u) == fo.eq_build(u) == fr.to_host(fr.build_eq_tensor(prover, u))
    assert refA.mle_eval(t, u) == fo.mle_eval(t, u) == fr.mle_eval(prover, fr.to_device(t), u)


@pytest.mark.parametrize("other,logd,window", [(1, 2, 64), (64, 3, 1), (4, 4, 8)])
def test_partial_me(refA, zk, prover, other, logd, window):
    rng = random.Random(other + logd + window)
    fr = zk.fr
    t = rnd(rng, other * (1 << logd) * window, small=True)
    u = rnd(rng, logd)
    # the reference folds dimension `cur_dim` of [other][cur_dim][window] only when other == 1 or window == 1
    # through its two code paths; both are covered by the shapes above
    ref_out = refA.partial_me(t, u, 1 << logd, window) if other == 1 or window == 1 else None
    mine = fr.to_host(fr.partial_me(prover, fr.to_device(t), u, 1 << logd, window))
    assert mine == fo.partial_me(t, other, logd, window, u)
    if ref_out is not None:
        assert ref_out == mine


@pytest.mark.parametrize("logn", [1, 5, 10])
def test_inner_product_rounds(refA, zk, prover, logn):
    rng = random.Random(logn)
    fr = zk.fr
    a, b = rnd(rng, 1 << logn), rnd(rng, 1 << logn, small=True)
    tr = zk.Transcript("fc")
    ev, xs, fin = fr.product_sumcheck(prover, tr, [fr.to_device(a), fr.to_device(b)], ["p0", "p1", "p2"])
    st, rev, rxs, rfin = refA.ip_rounds(zk.Transcript("fc").state, a, b)
    assert st == tr.state and rev == ev and rxs == xs and rfin == fin
    otr = fo.Transcript("fc")
    assert fo.product_sumcheck(otr, [a, b], ["p0", "p1", "p2"]) == (ev, xs, fin) and otr.state == st


@pytest.mark.parametrize("logn", [1, 6, 11])
def test_hadamard_and_quartic(refA, zk, prover, logn):
    rng = random.Random(50 + logn)
    fr = zk.fr
    cols = [rnd(rng, 1 << logn, small=(k > 0)) for k in range(4)]
    d = [fr.to_device(c) for c in cols]
    tr = zk.Transcript("hp")
    ev, ws, fin = fr.product_sumcheck(prover, tr, d[:3], ["hp0", "hp1", "hp2", "hp3"])
    st, rev, rws, rfin = refA.hadamard(zk.Transcript("hp").state, *cols[:3])
    assert st == tr.state and rev == ev and rws == ws and rfin == fin[1:]
    tr = zk.Transcript("qp")
    ev, ws, fin = fr.product_sumcheck(prover, tr, d, ["smx" + "p%d" % i for i in range(5)])
    st, rev, rws, rfin = refA.quartic(zk.Transcript("qp").state, "smx", *cols)
    assert st == tr.state and rev == ev and rws == ws and rfin == fin[1:]


@pytest.mark.parametrize("logD,logN", [(4, 4), (7, 5), (11, 8)])
def test_lookup_sumcheck(refA, zk, prover, logD, logN):
    from test_fr_gpu import lookup_instance
    rng = random.Random(logD * 31 + logN)
    fr = zk.fr
    S, T, m = lookup_instance(rng, logD, logN)
    alpha, beta = rng.randrange(fo.P), rng.randrange(fo.P)
    u = rnd(rng, logD)
    st, rA, rev, rws, rterm = refA.lookup(zk.Transcript("tlookup").state, S, T, m, alpha, beta, u)
    dS, dT, dm = fr.to_device(S), fr.to_device(T), fr.to_device(m)
    dA, dB = fr.inv_add(prover, dS, beta), fr.inv_add(prover, dT, beta)
    assert fr.to_host(dA) == rA == fo.inv_add(S, beta)
    B = fo.inv_add(T, beta)
    Cc = (alpha * alpha - sum(b * mm for b, mm in zip(B, m))) % fo.P
    tr = zk.Transcript("tlookup")
    ev, ws, term = fr.lookup_sumcheck(prover, tr, dA, dS, dB, dT, dm, alpha, beta, Cc, u)
    assert tr.state == st and ev == rev and ws == rws and term == rterm
