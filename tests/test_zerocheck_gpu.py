"""The programmable zero-check engine on CUDA against the Python-integer evaluation and, for the two summands
the library also has as compiled functors (rescale), against those."""
import numpy as np
import pytest

from conftest import lcg_cols
from zc_helpers import zc_sumcheck

pytestmark = pytest.mark.gpu
GL_P = 0xFFFFFFFF00000001

PROGRAMS = {
    "add": (4, [(1, (1,)), (1, (2,)), (GL_P - 1, (3,))], 0),                                   # E*(A+B-O)
    "swiglu": (5, [(1, (1, 2)), (GL_P - 65536, (3,)), (GL_P - 1, (4,))], 32768),              # E*(SIL*U+2^15-MO*2^16-REM)
    "rope": (7, [(1, (1, 5)), (1, (2, 6)), (GL_P - 16384, (3,)), (GL_P - 1, (4,))], 8192),
    "cubic": (9, [(3, (1, 2, 3)), (5, (4, 4)), (7, (8,)), (11, (5, 6, 7))], 99),
    "wide": (20, [(k + 1, (k, 19 - k)) for k in range(1, 10)] + [(2, (10, 11, 12))], 1),
    # a blinded chain: E*X*W + rho*(B1 + E*B2 + E^2*B3 + E^3*B4), the B1 term outside the E factor
    "blinded": (7, [(1, (1, 2)), (77, (4,)), (77, (0, 5)), (77, (0, 0, 6)), (77, (3,), True)], 0),
    "free-mix": (6, [(3, (1, 2, 3)), (5, (4, 5), True), (9, (0, 0, 0), True), (2, (1,), True)], 4),
}


@pytest.mark.parametrize("name", sorted(PROGRAMS))
@pytest.mark.parametrize("logn", [1, 2, 7, 12])
def test_matches_python_evaluation(orc, zk, prover, name, logn):
    nc, terms, konst = PROGRAMS[name]
    if logn == 12 and nc > 9:
        pytest.skip("python evaluation too slow")
    cols = lcg_cols(orc, 1 << logn, nc, 31 * logn + nc)
    tr = zk.Transcript("zc")
    r, m, fin = prover.sc_prove_zc(tr, "isw-sc", [zk.p3.to_device(c) for c in cols], terms, konst)
    st, m0, r0, f0 = zc_sumcheck(orc, orc.tr_init("zc"), "isw-sc", cols, terms, konst)
    assert st == tr.state and (m == m0).all() and (r == r0).all() and (fin == f0).all()


def _large_program(nc, nterms, seed, free_every=0):
    rng = np.random.default_rng(seed)
    terms = []
    for j in range(nterms):
        deg = int(rng.integers(1, 4))
        t = (int(rng.integers(1, GL_P, dtype=np.uint64)), tuple(int(x) for x in rng.integers(0, nc, size=deg)))
        terms.append(t + (True,) if free_every and j % free_every == 0 else t)
    return terms


@pytest.mark.parametrize("nc,nterms,logn", [(40, 100, 1), (59, 400, 6), (33, 10, 9), (130, 900, 5), (224, 2048, 3), (20, 300, 7)])
def test_large_programs_match_python_evaluation(orc, zk, prover, nc, nterms, logn):
    """More than 32 columns or 120 terms: the shared-memory variant (the bf16 gadgets' constraint systems)."""
    terms = _large_program(nc, nterms, nc + nterms)
    cols = lcg_cols(orc, 1 << logn, nc, 7 * nc + logn)
    tr = zk.Transcript("zc")
    r, m, fin = prover.sc_prove_zc(tr, "bfa-scE", [zk.p3.to_device(c) for c in cols], terms, 12345)
    st, m0, r0, f0 = zc_sumcheck(orc, orc.tr_init("zc"), "bfa-scE", cols, terms, 12345)
    assert st == tr.state and (m == m0).all() and (r == r0).all() and (fin == f0).all()


def test_large_program_with_terms_outside_the_factor(orc, zk, prover):
    terms = _large_program(45, 200, 3, free_every=7)
    cols = lcg_cols(orc, 1 << 5, 45, 11)
    tr = zk.Transcript("zc")
    r, m, fin = prover.sc_prove_zc(tr, "z", [zk.p3.to_device(c) for c in cols], terms, 5)
    st, m0, r0, f0 = zc_sumcheck(orc, orc.tr_init("zc"), "z", cols, terms, 5)
    assert st == tr.state and (m == m0).all() and (r == r0).all() and (fin == f0).all()


def test_large_program_equals_small_engine(orc, zk, prover):
    """The same 30-column program through both variants (the second padded with a zero-coefficient term count > 120)."""
    nc, logn = 30, 13
    terms = _large_program(nc, 100, 5)
    cols = [zk.p3.to_device(c) for c in lcg_cols(orc, 1 << logn, nc, 77)]
    tr1, tr2 = zk.Transcript("zc"), zk.Transcript("zc")
    a = prover.sc_prove_zc(tr1, "t", cols, terms, 9)
    b = prover.sc_prove_zc(tr2, "t", cols, terms + [(0, (1,))] * 30, 9)
    assert tr1.state == tr2.state and all((x == y).all() for x, y in zip(a, b))


@pytest.mark.parametrize("nl", [1, 2])
def test_matches_compiled_rescale_summand(orc, zk, prover, nl):
    logn = 15
    cols = lcg_cols(orc, 1 << logn, 3 + nl, 5 + nl)
    H, P2 = 1 << 15, 1 << 16
    d = [zk.p3.to_device(c) for c in cols]
    tr1 = zk.Transcript("zc")
    r1, m1, f1 = prover.sc_prove_gpu(tr1, "irs-sc", d, zk.p3.F_IRS1 if nl == 1 else zk.p3.F_IRS2, 5, [H, P2])
    terms = [(1, (1,)), (GL_P - P2, (2,)), (GL_P - 1, (3,))] + ([(GL_P - 65536, (4,))] if nl == 2 else [])
    tr2 = zk.Transcript("zc")
    r2, m2, f2 = prover.sc_prove_zc(tr2, "irs-sc", d, terms, H)
    assert tr1.state == tr2.state and (m1 == m2).all() and (r1 == r2).all() and (f1 == f2).all()


def test_argument_checks(zk, prover):
    d = [zk.p3.to_device(np.zeros(4, dtype=np.uint64)) for _ in range(3)]
    with pytest.raises(Exception):
        prover.sc_prove_zc(zk.Transcript("x"), "t", d, [(1, (3,))])            # column index out of range
    with pytest.raises(Exception):
        prover.sc_prove_zc(zk.Transcript("x"), "t", d, [(1, (1, 1, 1, 1))])    # degree 4 term
