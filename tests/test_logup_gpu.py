"""Parity of the CUDA logUp path (histogram, batched inversion, combine, GKR fractional-sum prover)."""
import numpy as np
import pytest

from conftest import dig

pytestmark = pytest.mark.gpu
GL_P = 0xFFFFFFFF00000001


def test_logup_primitives_golden(golden, orc, zk, prover):
    import torch
    g = golden["logup"]
    A, _ = orc.lcg(g["n"], g["seed"])
    A_dev = zk.p3.to_device(A)
    assert dig(zk.p3.to_host(prover.inv_all_add(A_dev, g["beta"]))) == g["inv_digest"]
    rev = zk.p3.to_device(A[::-1].copy())
    out = prover.combine([A_dev, rev], g["beta"])
    torch.cuda.synchronize()
    assert dig(zk.p3.to_host(out)) == g["combine_digest"]


@pytest.mark.parametrize("n", [1, 2, 15, 16, 17, 255, 4097, 1 << 16, (1 << 20) + 3])
def test_inv_all_add_sizes(orc, zk, prover, n):
    A, s = orc.lcg(n, 800 + n % 97)
    beta = int(orc.lcg(1, s)[0][0])
    got = zk.p3.to_host(prover.inv_all_add(zk.p3.to_device(A), beta))
    assert (got == orc.inv_all_add(A, beta)).all()


def test_inv_all_add_zero_denominator(zk, prover):
    A = np.array([5, 7, 11, 13], dtype=np.uint64)
    with pytest.raises(zk.ZkhError) as ei:
        prover.inv_all_add(zk.p3.to_device(A), GL_P - 11)
    assert ei.value.code == -4


@pytest.mark.parametrize("M,n", [(1, 10), (16, 1000), (1 << 10, 1 << 16), (1 << 15, 1 << 18), (1 << 16, 1 << 20), (1 << 20, 1 << 18),
                                 (1 << 16, (1 << 20) + 3), (1 << 17, 1 << 19), (3 * (1 << 15) + 5, 1 << 18), (1 << 18, 1 << 18)])
def test_histogram(orc, zk, prover, M, n):
    import torch
    rng = np.random.default_rng(M + n)
    # skewed like the lookup workload: Gaussian around the table centre, clipped
    idx = np.clip(np.rint(rng.normal(M / 2, max(M / 64, 1), n)), 0, M - 1).astype(np.uint32)
    idx_dev = torch.from_numpy(idx.view(np.int32)).cuda()
    cnt = zk.p3.to_host(prover.histogram(idx_dev, M))
    assert (cnt == orc.histogram(idx, M)).all() and int(cnt.sum()) == n
    if M > 1:
        idx[n // 2] = M
        with pytest.raises(zk.ZkhError) as ei:
            prover.histogram(torch.from_numpy(idx.view(np.int32)).cuda(), M)
        assert ei.value.code == -4


@pytest.mark.parametrize("M", [1 << 16, 1 << 18])
def test_histogram_hot_bin_and_uniform(orc, zk, prover, M):
    """Every index on one row (the padding members of a merged lookup) and uniformly spread indices: the two extremes of
    contention for the bins held in shared memory."""
    import torch
    n = (1 << 21) + 5
    for idx in (np.full(n, M - 7, dtype=np.uint32), np.random.default_rng(M).integers(0, M, n).astype(np.uint32)):
        cnt = zk.p3.to_host(prover.histogram(torch.from_numpy(idx.view(np.int32)).cuda(), M))
        assert (cnt == orc.histogram(idx, M)).all() and int(cnt.sum()) == n


def test_gkr_golden(golden, orc, ref_or_none, zk, prover):
    for g in golden["gkr"]:
        L, cl = g["L"], g["combine_last"]
        p, s2 = orc.lcg(1 << L, g["seed"])
        q, _ = orc.lcg(1 << L, s2)
        tr = zk.Transcript("gkr-golden")
        pf, rfin, cpq = prover.gkr_prove(tr, "lug-gA", zk.p3.to_device(p), zk.p3.to_device(q), cl)
        assert tr.state.hex() == g["state"] and dig(pf) == g["proof_digest"]
        assert [int(x) for x in rfin] == g["rfin"]
        if cl:
            assert list(cpq) == g["cpq"]
        st0 = orc.tr_init("gkr-golden")
        assert orc.gkr_verify(st0, "lug-gA", L, pf, cl)[0]
        if ref_or_none:
            assert ref_or_none.gkr_verify(st0, "lug-gA", L, pf, cl)[0]


@pytest.mark.parametrize("L", [1, 2, 3, 4, 8, 11, 12, 13, 14, 16, 18])
@pytest.mark.parametrize("combine_last", [True, False])
def test_gkr_matches_oracle(orc, zk, prover, L, combine_last):
    p, s = orc.lcg(1 << L, 900 + L)
    q, _ = orc.lcg(1 << L, s)
    st0 = orc.tr_init("gkr")
    st1, want, rf0, cpq0 = orc.gkr_prove(st0, "lug-gT", p, q, combine_last)
    p_dev, q_dev = zk.p3.to_device(p), zk.p3.to_device(q)
    tr = zk.Transcript("gkr")
    pf, rfin, cpq = prover.gkr_prove(tr, "lug-gT", p_dev, q_dev, combine_last)
    assert pf == want and tr.state == st1 and (rfin == rf0).all()
    if combine_last:
        assert cpq == cpq0
    assert (zk.p3.to_host(p_dev) == p).all() and (zk.p3.to_host(q_dev) == q).all()


def test_gkr_lookup_shaped_at_scale(orc, ref_or_none, zk, prover):
    """logUp A-side shape at 2^20: leaves (1, A_i + beta); the root satisfies P/Q = sum 1/(A_i+beta),
    the proof verifies and the leaf claims are the MLEs at the final point."""
    L = 20
    A, s = orc.lcg(1 << L, 4242)
    beta = int(orc.lcg(1, s)[0][0])
    q = ((A.astype(object) + beta) % GL_P).astype(np.uint64)
    p = np.ones(1 << L, dtype=np.uint64)
    p_dev, q_dev = zk.p3.to_device(p), zk.p3.to_device(q)
    tr = zk.Transcript("lookup")
    pf, rfin, (cp, cq) = prover.gkr_prove(tr, "lug-gA", p_dev, q_dev, True)
    P, Q = (int(x) for x in np.frombuffer(pf[:16], dtype=np.uint64))
    inv = zk.p3.to_host(prover.inv_all_add(zk.p3.to_device(A), beta))
    S = int(np.sum(inv.astype(object)) % GL_P)
    assert P * pow(Q, GL_P - 2, GL_P) % GL_P == S
    st0 = orc.tr_init("lookup")
    ok, st1, rf, out4 = orc.gkr_verify(st0, "lug-gA", L, pf, True)
    assert ok and st1 == tr.state and (rf == rfin).all() and (int(out4[0]), int(out4[2])) == (cp, cq)
    assert cp == prover.eval_h_gpu(p_dev, rfin) and cq == prover.eval_h_gpu(q_dev, rfin)
    if ref_or_none:
        assert ref_or_none.gkr_verify(st0, "lug-gA", L, pf, True)[0]


def test_gkr_zero_denominator(zk, prover):
    p = zk.p3.to_device(np.ones(8, dtype=np.uint64))
    q = zk.p3.to_device(np.array([1, 2, 3, 0, 5, 6, 7, 8], dtype=np.uint64))
    tr = zk.Transcript("z")
    with pytest.raises(zk.ZkhError) as ei:
        prover.gkr_prove(tr, "t", p, q)
    assert ei.value.code == -4


def test_reference_cuda_gkr_same_bytes(orc, ref, zk, prover):
    if not ref.gpu_available():
        pytest.skip("reference shim sees no GPU")
    for L in (14, 18):
        p, s = orc.lcg(1 << L, 31 + L)
        q, _ = orc.lcg(1 << L, s)
        st0 = orc.tr_init("vs-ref")
        st1, want, rf0, cpq0 = ref.gkr_prove(st0, "lug-gA", p, q, True, gpu=True)
        tr = zk.Transcript("vs-ref")
        pf, rfin, cpq = prover.gkr_prove(tr, "lug-gA", zk.p3.to_device(p), zk.p3.to_device(q), True)
        assert pf == want and tr.state == st1 and (rfin == rf0).all() and cpq == cpq0
