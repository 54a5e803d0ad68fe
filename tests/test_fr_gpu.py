"""BLS12-381 Fr back-end on CUDA against the Python-integer restatement (oracle/fr_oracle.py): field
arithmetic through the folds, eq tensors, partial evaluations and the product sumchecks of the
reference's first stack (inner product, Hadamard, bracket), transcript included."""
import random

import pytest

import fr_oracle as fo

pytestmark = pytest.mark.gpu

EDGE = [0, 1, 2, fo.P - 1, fo.P - 2, (1 << 32) - 1, 1 << 32, (1 << 255) % fo.P, fo.P >> 1, (fo.P >> 1) + 1]


def rnd(rng, n, small=False):
    if small:                                  # the reference's tensors hold small signed integers lifted mod p
        return [rng.randrange(-(1 << 20), 1 << 20) % fo.P for _ in range(n)]
    return [rng.randrange(fo.P) for _ in range(n)]


def test_fold_exercises_field_edges(zk, prover):
    rng = random.Random(1)
    fr = zk.fr
    lo = EDGE + rnd(rng, 54)
    hi = list(reversed(EDGE)) + rnd(rng, 54)
    for w in [0, 1, fo.P - 1, 2, rng.randrange(fo.P), (1 << 255) % fo.P]:
        got = fr.to_host(fr.fr_fold(prover, fr.to_device(lo + hi), w))
        assert got == fo.fold(lo + hi, w)


@pytest.mark.parametrize("v", [0, 1, 5, 10, 11, 14])
def test_eq_tensor_and_mle_eval(zk, prover, v):
    rng = random.Random(100 + v)
    fr = zk.fr
    u = rnd(rng, v)
    E = fr.to_host(fr.build_eq_tensor(prover, u))
    assert E == fo.eq_build(u)
    t = rnd(rng, 1 << v, small=(v > 10))
    assert fr.mle_eval(prover, fr.to_device(t), u) == fo.mle_eval(t, u)


@pytest.mark.parametrize("other,logd,window", [(1, 3, 16), (8, 4, 1), (3, 5, 7), (64, 7, 1), (1, 7, 64), (5, 0, 3)])
def test_partial_me(zk, prover, other, logd, window):
    rng = random.Random(other * 100 + logd * 10 + window)
    fr = zk.fr
    t = rnd(rng, other * (1 << logd) * window)
    u = rnd(rng, logd)
    got = fr.to_host(fr.partial_me(prover, fr.to_device(t), u, 1 << logd, window))
    assert got == fo.partial_me(t, other, logd, window, u)


def test_multi_dim_me_matches_fc_claims(zk, prover):
    """claim_X = X.multi_dim_me({u_batch, u_input}, {B, IN}) as zkob_fc computes it (zkob_fc.cu:337-338)."""
    rng = random.Random(5)
    fr = zk.fr
    B, IN = 8, 32
    X = rnd(rng, B * IN, small=True)
    ub, ui = rnd(rng, 3), rnd(rng, 5)
    got = fr.multi_dim_me(prover, fr.to_device(X), [ub, ui], [B, IN])
    red = fo.partial_me(X, B, 5, 1, ui)           # fold IN (last dimension) first
    assert got == fo.mle_eval(red, ub)


LABELS = {2: ["p0", "p1", "p2"], 3: ["hp0", "hp1", "hp2", "hp3"], 4: ["zp0", "zp1", "zp2", "zp3", "zp4"]}


@pytest.mark.parametrize("nc", [2, 3, 4])
@pytest.mark.parametrize("logn", [1, 2, 6, 11])
def test_product_sumcheck(zk, prover, nc, logn):
    rng = random.Random(nc * 50 + logn)
    fr = zk.fr
    cols = [rnd(rng, 1 << logn, small=(k > 0)) for k in range(nc)]
    tr = zk.Transcript("fr-sc")
    ev, ch, fin = fr.product_sumcheck(prover, tr, [fr.to_device(c) for c in cols], LABELS[nc])
    otr = fo.Transcript("fr-sc")
    oev, och, ofin = fo.product_sumcheck(otr, cols, LABELS[nc])
    assert ev == oev and ch == och and fin == ofin and tr.state == otr.state
    # round consistency the reference asserts: claim == p(0) + p(1), next claim by Lagrange
    claim = sum(eval_prod(cols, i) for i in range(1 << logn)) % fo.P
    for e, x in zip(ev, ch):
        assert (e[0] + e[1]) % fo.P == claim
        claim = fo.lagrange(e, x)
    prod = 1
    for f in fin:
        prod = prod * f % fo.P
    assert prod == claim


def eval_prod(cols, i):
    p = 1
    for c in cols:
        p = p * c[i] % fo.P
    return p


def test_inner_product_rounds_as_in_fc(zk, prover):
    """The zkob_fc flow on a small layer: reduce X by u_batch and W by u_output, run the rounds, check
    the terminal values against multi_dim_me claims at u_input = reversed challenges (zkob_fc.cu:279-345)."""
    rng = random.Random(77)
    fr = zk.fr
    B, IN, OUT = 4, 64, 8
    X = rnd(rng, B * IN, small=True)
    W = rnd(rng, IN * OUT, small=True)
    ub, uo = rnd(rng, 2), rnd(rng, 3)
    dX, dW = fr.to_device(X), fr.to_device(W)
    X_red = fr.partial_me(prover, dX, ub, B, IN)
    W_red = fr.partial_me(prover, dW, uo, OUT, 1)
    assert fr.to_host(X_red) == fo.partial_me(X, 1, 2, IN, ub)
    assert fr.to_host(W_red) == fo.partial_me(W, IN, 3, 1, uo)
    tr = zk.Transcript("fc")
    ev, xs, fin = fr.product_sumcheck(prover, tr, [X_red, W_red], ["p0", "p1", "p2"])
    u_input = list(reversed(xs))
    assert fin[0] == fr.multi_dim_me(prover, dX, [ub, u_input], [B, IN])
    assert fin[1] == fr.multi_dim_me(prover, dW, [u_input, uo], [IN, OUT])


def test_argument_checks(zk, prover):
    fr = zk.fr
    t = fr.to_device([1, 2, 3, 4])
    with pytest.raises(Exception):
        fr.fr_fold(prover, t, fo.P)                       # challenge not below p
    with pytest.raises(Exception):
        fr.product_sumcheck(prover, zk.Transcript("x"), [t], ["a", "b"])   # one column
    with pytest.raises(ValueError):
        fr.partial_me(prover, t, [1], 4, 1)


def lookup_instance(rng, logD, logN):
    D, N = 1 << logD, 1 << logN
    T = [rng.randrange(-(1 << 15), 1 << 15) % fo.P for _ in range(N)]
    idx = [min(N - 1, max(0, int(rng.gauss(N / 2, N / 8)))) for _ in range(D)]
    S = [T[i] for i in idx]
    m = [0] * N
    for i in idx:
        m[i] += 1
    return S, T, m


@pytest.mark.parametrize("n", [1, 7, 8, 9, 1000, 4097])
def test_inv_add(zk, prover, n):
    rng = random.Random(n)
    fr = zk.fr
    beta = rng.randrange(fo.P)
    vals = rnd(rng, n)
    vals[0] = (fo.P - beta) % fo.P                      # zero denominator: Fermat's inverse is 0
    if n > 8:
        vals[n // 2] = (fo.P - beta) % fo.P
    got = fr.to_host(fr.inv_add(prover, fr.to_device(vals), beta))
    assert got == fo.inv_add(vals, beta)


@pytest.mark.parametrize("n", [1, 5, 1000, 40000])
def test_elementwise_product(zk, prover, n):
    rng = random.Random(n)
    fr = zk.fr
    a, b = rnd(rng, n), rnd(rng, n)
    a[0], b[n - 1] = fo.P - 1, 0
    da, db = fr.to_device(a), fr.to_device(b)
    want = [x * y % fo.P for x, y in zip(a, b)]
    assert fr.to_host(fr.mul(prover, da, db)) == want
    prover._ck(prover._L.zkh_fr_mul(prover._h, da.data_ptr(), da.data_ptr(), db.data_ptr(), n))     # in place
    assert fr.to_host(da) == want


@pytest.mark.parametrize("logD,logN", [(1, 1), (3, 3), (5, 2), (9, 6), (12, 12), (13, 8)])
def test_lookup_sumcheck(zk, prover, logD, logN):
    rng = random.Random(logD * 31 + logN)
    fr = zk.fr
    S, T, m = lookup_instance(rng, logD, logN)
    alpha, beta = rng.randrange(fo.P), rng.randrange(fo.P)
    u = rnd(rng, logD)
    dS, dT, dm = fr.to_device(S), fr.to_device(T), fr.to_device(m)
    dA, dB = fr.inv_add(prover, dS, beta), fr.inv_add(prover, dT, beta)
    A, B = fo.inv_add(S, beta), fo.inv_add(T, beta)
    assert fr.to_host(dA) == A and fr.to_host(dB) == B
    Cc = (alpha * alpha - sum(b * mm for b, mm in zip(B, m))) % fo.P
    assert fr.dot(prover, dB, dm) == sum(b * mm for b, mm in zip(B, m)) % fo.P
    tr = zk.Transcript("tlookup")
    ev, ws, term = fr.lookup_sumcheck(prover, tr, dA, dS, dB, dT, dm, alpha, beta, Cc, u)
    otr = fo.Transcript("tlookup")
    oev, ows, oterm = fo.lookup_sumcheck(otr, A, S, B, T, m, alpha, beta, Cc, u)
    assert ev == oev and ws == ows and term == oterm and tr.state == otr.state
    claim = (alpha + alpha * alpha) % fo.P               # the honest instance satisfies every round check
    for e, v in zip(ev, ws):
        assert (e[0] + e[1]) % fo.P == claim
        claim = fo.lagrange(e, v)
    # terminals are the columns' multilinear extensions at the reversed challenges
    pt = list(reversed(ws))
    assert term[0] == fo.mle_eval(A, pt) and term[1] == fo.mle_eval(S, pt)
    assert term[4] == fo.mle_eval(m, pt[:logN]) and term[3] == fo.mle_eval(T, pt[:logN])
