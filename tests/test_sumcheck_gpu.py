"""Parity of the CUDA sumcheck engine (through the C ABI) with the oracle, the golden
vectors minted from the reference's host loops, and the reference's own CUDA prover."""
import numpy as np
import pytest

from conftest import dig, lcg_cols

pytestmark = pytest.mark.gpu
GL_P = 0xFFFFFFFF00000001
KIND = {"logup": (3, 4), "prod2": (0, 2), "prod3": (1, 3)}


def dev(zk, cols):
    return [zk.p3.to_device(c) for c in cols]


def test_golden_sumchecks(golden, orc, zk, prover):
    for s in golden["sumcheck"]:
        f, nc = KIND[s["kind"]]
        cols = lcg_cols(orc, 1 << s["logn"], nc, s["seed"])
        tr = zk.Transcript("sc-golden")
        r, m, fin = prover.sc_prove_gpu(tr, s["tag"], dev(zk, cols), f, s["nt"], s["par"])
        assert [int(x) for x in r] == s["chals"]
        assert dig(m) == s["msgs_digest"] and tr.state.hex() == s["state"]


@pytest.mark.parametrize("functor,nt,npar", [(0, 3, 0), (0, 5, 0), (1, 4, 0), (1, 5, 0), (2, 4, 1), (3, 4, 2)])
@pytest.mark.parametrize("logn", [1, 2, 3, 7, 11, 12, 13, 14, 17])
def test_matches_oracle(orc, zk, prover, functor, nt, npar, logn):
    nc = zk.p3.FUNCTOR_NC[functor]
    cols = lcg_cols(orc, 1 << logn, nc, 1000 + 31 * logn + functor)
    par = [int(x) for x in orc.lcg(npar, 77 + logn)[0]] if npar else []
    st0 = orc.tr_init("parity")
    st1, m0, r0, fin0 = orc.sumcheck(st0, "tag-%d" % functor, functor, nt, cols, par, nthreads=4)
    d = dev(zk, cols)
    tr = zk.Transcript("parity")
    r, m, fin = prover.sc_prove_gpu(tr, "tag-%d" % functor, d, functor, nt, par)
    assert (m == m0).all() and (r == r0).all() and (fin == fin0).all()
    assert tr.state == st1
    # the caller's columns are left intact
    for a, b in zip(cols, d):
        assert (zk.p3.to_host(b) == a).all()
    # host-buffer entry point: same bytes
    tr2 = zk.Transcript("parity")
    r2, m2, fin2 = prover.sc_prove_host(tr2, "tag-%d" % functor, cols, functor, nt, par)
    assert (m2 == m0).all() and (r2 == r0).all() and (fin2 == fin0).all() and tr2.state == st1


def test_edge_values(orc, zk, prover):
    """All-zero, all-(p-1) and mixed extreme columns exercise every carry path of the lazy sums."""
    n = 1 << 14
    ext = np.array([0, 1, GL_P - 1, GL_P - 2, 0xFFFFFFFF, 0xFFFFFFFF00000000, 1 << 32, (1 << 63) + 5], dtype=np.uint64)
    patterns = [np.zeros(n, np.uint64), np.full(n, GL_P - 1, np.uint64), np.tile(ext, n // 8),
                np.tile(ext[::-1].copy(), n // 8)]
    for functor, nt, par in [(0, 3, []), (1, 5, []), (2, 4, [GL_P - 1]), (3, 4, [GL_P - 1, GL_P - 2])]:
        nc = zk.p3.FUNCTOR_NC[functor]
        for shift in range(3):
            cols = [patterns[(k + shift) % 4] for k in range(nc)]
            st0 = orc.tr_init("edge")
            st1, m0, r0, fin0 = orc.sumcheck(st0, "e", functor, nt, cols, par)
            tr = zk.Transcript("edge")
            r, m, fin = prover.sc_prove_gpu(tr, "e", dev(zk, cols), functor, nt, par)
            assert (m == m0).all() and (r == r0).all() and (fin == fin0).all() and tr.state == st1


@pytest.mark.parametrize("functor,nt,logn", [(0, 3, 24), (1, 4, 22)])
def test_large_verifier_chain(orc, zk, prover, functor, nt, logn):
    """Size-independent property at bench scale: the message chain verifies
    (s0+s1 = claim, next claim = Lagrange evaluation at the challenge, terminal = F(finals))
    and the first claim equals the true sum."""
    nc = zk.p3.FUNCTOR_NC[functor]
    cols = lcg_cols(orc, 1 << logn, nc, 0xBEEF1234)
    tr = zk.Transcript("bench-sc%d" % (nt - 1))
    r, m, fin = prover.sc_prove_gpu(tr, "sc", dev(zk, cols), functor, nt)
    if functor == 0:
        true_sum = orc.eval_h(cols[0], cols[1])
    else:
        acc = 0  # exact big-integer arithmetic, in chunks
        step = 1 << 18
        for o in range(0, 1 << logn, step):
            a = cols[0][o:o + step].astype(object) * cols[1][o:o + step].astype(object) % GL_P
            acc = (acc + int(np.sum(a * cols[2][o:o + step].astype(object) % GL_P))) % GL_P
        true_sum = acc
    claim = (int(m[0][0]) + int(m[0][1])) % GL_P
    assert claim == true_sum
    tr_v = zk.Transcript("bench-sc%d" % (nt - 1))
    for rd in range(logn):
        assert (int(m[rd][0]) + int(m[rd][1])) % GL_P == claim
        tr_v.absorb("sc", m[rd])
        a = tr_v.chal()
        assert a == int(r[rd])
        mm = [int(x) for x in m[rd]]
        claim = orc.quad_eval(*mm, a) if nt == 3 else orc.cubic_eval(*mm, a)
    term = 1
    for k in range(nc):
        term = term * int(fin[k]) % GL_P
    assert term == claim and tr_v.state == tr.state
    for k in range(nc):
        assert int(fin[k]) == prover.eval_h_gpu(zk.p3.to_device(cols[k]), r)


def test_reference_cuda_prover_same_bytes(orc, ref, zk, prover):
    """The reference's own p3sg::sc_prove_gpu on this GPU gives the same transcript."""
    if not ref.gpu_available():
        pytest.skip("reference shim sees no GPU")
    for functor, nt, par in [(0, 3, []), (1, 5, []), (2, 4, [12345]), (3, 4, [7, 9])]:
        nc = zk.p3.FUNCTOR_NC[functor]
        cols = lcg_cols(orc, 1 << 18, nc, 4242 + functor)
        st0 = orc.tr_init("vs-ref")
        st1, m0, r0, _ = ref.sc_prove_gpu(st0, "t", functor, nt, cols, par)
        tr = zk.Transcript("vs-ref")
        r, m, fin = prover.sc_prove_gpu(tr, "t", dev(zk, cols), functor, nt, par)
        assert (m == m0).all() and (r == r0).all() and tr.state == st1


def test_argument_errors(zk, prover):
    cols = dev(zk, [np.arange(8, dtype=np.uint64)] * 2)
    tr = zk.Transcript("err")
    with pytest.raises(zk.ZkhError):
        prover.sc_prove_gpu(tr, "t", cols, 1, 4)          # nc does not match the summand
    with pytest.raises(zk.ZkhError):
        prover.sc_prove_gpu(tr, "t", cols, 0, 7)          # nt out of range
    with pytest.raises(zk.ZkhError):
        prover.sc_prove_gpu(tr, "t" * 60, cols, 0, 3)     # tag too long
    with pytest.raises(zk.ZkhError):
        prover.sc_prove_gpu(tr, "t", cols, 0, 4)          # combination not built
    assert tr.state == zk.Transcript("err").state          # a failed call leaves the transcript alone


def test_vector_kernels(orc, zk, prover):
    for v in [0, 1, 2, 5, 13, 14, 15, 21]:
        z, s = orc.lcg(v, 500 + v)
        c, _ = orc.lcg(1 << v, s)
        eq = zk.p3.to_host(prover.build_eq_gpu(z))
        assert (eq == orc.build_eq(z)).all()
        assert prover.eval_h_gpu(zk.p3.to_device(c), z) == orc.mle_eval(c, z)
    for logn in [1, 2, 3, 10, 20]:
        f, s = orc.lcg(1 << logn, 600 + logn)
        a = int(orc.lcg(1, s)[0][0])
        out = prover.bind(zk.p3.to_device(f), a)
        prover.sync()
        assert (zk.p3.to_host(out) == orc.bind_lsb(f, a)).all()
    with pytest.raises(zk.ZkhError):
        prover.bind(zk.p3.to_device(np.arange(6, dtype=np.uint64)), 1)
