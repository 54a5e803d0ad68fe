"""Parity of the CUDA batched opening (p3bo::prove_class, non-zk) with the oracle restatement, the
reference's host-only verifier and the reference's own CUDA prover."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
GL_P = 0xFFFFFFFF00000001


def make_ledger(orc, v, ncols, T, k, seed):
    cols, s = [], seed
    for _ in range(ncols):
        a, s = orc.lcg(1 << v, s)
        cols.append(a)
    pts, s = orc.lcg(T * v, s)
    pts = pts.reshape(T, v)
    rng = np.random.default_rng(seed)
    ent_col = [int(rng.integers(0, ncols)) for _ in range(k)]
    ent_col[:ncols] = list(range(ncols))[:k]
    zid = [int(rng.integers(0, T)) for _ in range(k)]
    zid[:T] = list(range(T))[:k]
    return cols, pts, ent_col, zid


@pytest.mark.parametrize("v,R,Q,ncols,T,k", [(1, 1, 20, 1, 1, 1), (2, 1, 24, 3, 2, 4), (3, 1, 24, 2, 2, 3),
                                             (6, 2, 24, 5, 3, 9), (8, 1, 32, 4, 4, 7), (11, 1, 24, 6, 5, 12),
                                             (13, 2, 24, 3, 7, 10)])
def test_prove_class_matches_oracle(orc, ref_or_none, zk, prover, v, R, Q, ncols, T, k):
    cols, pts, ent_col, zid = make_ledger(orc, v, ncols, T, k, 100 + v)
    dcols = [zk.p3.to_device(c) for c in cols]
    roots_c = [prover.commit_gpu_rootonly(d, R) for d in dcols]
    assert roots_c[0] == orc.merkle_root(orc.rs_encode(cols[0], R))
    roots = [roots_c[c] for c in ent_col]
    y = [orc.mle_eval(cols[c], pts[t]) for c, t in zip(ent_col, zid)]
    st0 = orc.tr_init("main")
    want, st1 = orc.bo_prove_class(st0, pts, [cols[c] for c in ent_col], roots, zid, R, Q, "tf-bo3")
    tr = zk.Transcript("main")
    got = prover.prove_class(tr, pts, [(dcols[c], roots_c[c], t) for c, t in zip(ent_col, zid)], R, Q, "tf-bo3")
    assert got == want and tr.state == st1
    ok, st2 = orc.bo_verify_class(st0, pts, roots, zid, y, R, Q, "tf-bo3", got)
    assert ok and st2 == st1
    if ref_or_none:
        ok, st3 = ref_or_none.bo_verify_class(st0, pts, roots, zid, y, R, Q, "tf-bo3", got)
        assert ok and st3 == st1
        bad = bytearray(got)
        bad[16] ^= 1
        assert not ref_or_none.bo_verify_class(st0, pts, roots, zid, y, R, Q, "tf-bo3", bytes(bad))[0]
        y2 = list(y)
        y2[-1] = (y2[-1] + 1) % GL_P
        assert not ref_or_none.bo_verify_class(st0, pts, roots, zid, y2, R, Q, "tf-bo3", got)[0]
    for d, c in zip(dcols, cols):
        assert (zk.p3.to_host(d) == c).all()


def test_prove_class_at_scale_verifies(orc, ref_or_none, zk, prover):
    """A class of 2^18-row columns with 12 claims at 4 points: accepted by the verifiers."""
    v, R, Q, ncols, T, k = 18, 1, 24, 6, 4, 12
    cols, pts, ent_col, zid = make_ledger(orc, v, ncols, T, k, 77)
    dcols = [zk.p3.to_device(c) for c in cols]
    roots_c = [prover.commit_gpu_rootonly(d, R) for d in dcols]
    roots = [roots_c[c] for c in ent_col]
    y = [prover.eval_h_gpu(dcols[c], pts[t]) for c, t in zip(ent_col, zid)]
    tr = zk.Transcript("main")
    pf = prover.prove_class(tr, pts, [(dcols[c], roots_c[c], t) for c, t in zip(ent_col, zid)], R, Q, "itf-bo0")
    st0 = orc.tr_init("main")
    ok, st1 = orc.bo_verify_class(st0, pts, roots, zid, y, R, Q, "itf-bo0", pf)
    assert ok and st1 == tr.state
    if ref_or_none:
        assert ref_or_none.bo_verify_class(st0, pts, roots, zid, y, R, Q, "itf-bo0", pf)[0]


def test_reference_cuda_prove_class_same_bytes(orc, ref, zk, prover):
    if not ref.gpu_available():
        pytest.skip("reference shim sees no GPU")
    v, R, Q, ncols, T, k = 12, 1, 24, 5, 3, 8
    cols, pts, ent_col, zid = make_ledger(orc, v, ncols, T, k, 555)
    dcols = [zk.p3.to_device(c) for c in cols]
    roots_c = [prover.commit_gpu_rootonly(d, R) for d in dcols]
    roots = [roots_c[c] for c in ent_col]
    st0 = orc.tr_init("main")
    want, st1, _ms = ref.bo_prove_class(st0, pts, [cols[c] for c in ent_col], roots, zid, R, Q, "tf-bo1")
    tr = zk.Transcript("main")
    got = prover.prove_class(tr, pts, [(dcols[c], roots_c[c], t) for c, t in zip(ent_col, zid)], R, Q, "tf-bo1")
    assert got == want and tr.state == st1


def test_prove_class_argument_errors(orc, zk, prover):
    col = zk.p3.to_device(orc.lcg(8, 1)[0])
    tr = zk.Transcript("e")
    pts = np.zeros((1, 3), dtype=np.uint64)
    with pytest.raises(zk.ZkhError):
        prover.prove_class(tr, pts, [(col, b"\\0" * 32, 1)], 1, 24, "x")   # point index out of range
    with pytest.raises(zk.ZkhError):
        prover.prove_class(tr, pts, [(col, b"\\0" * 32, 0)], 0, 24, "x")   # rate


@pytest.mark.parametrize("v,R,ncols,T,k", [(2, 1, 2, 2, 3), (9, 2, 4, 3, 8), (14, 1, 5, 4, 11)])
def test_kept_commitments_give_the_same_proof(orc, zk, prover, v, R, ncols, T, k):
    """Columns committed with their codeword and tree kept resident open to the same bytes as recomputed ones;
    a class may mix kept and recomputed columns."""
    Q = 24
    cols, pts, ent_col, zid = make_ledger(orc, v, ncols, T, k, 300 + v)
    dcols = [zk.p3.to_device(c) for c in cols]
    plain_roots = [prover.commit_gpu_rootonly(d, R) for d in dcols]
    tr0 = zk.Transcript("main")
    want = prover.prove_class(tr0, pts, [(dcols[c], plain_roots[c], t) for c, t in zip(ent_col, zid)], R, Q, "tf-bo1")
    prover.keep_trees = True
    try:
        kept_roots = [prover.commit_gpu_rootonly(d, R) if i % 2 == 0 or ncols < 3 else plain_roots[i] for i, d in enumerate(dcols)]
        assert kept_roots == plain_roots
        tr1 = zk.Transcript("main")
        got = prover.prove_class(tr1, pts, [(dcols[c], kept_roots[c], t) for c, t in zip(ent_col, zid)], R, Q, "tf-bo1")
        assert got == want and tr1.state == tr0.state
    finally:
        prover.keep_trees = False
        prover.release_kept()
    tr2 = zk.Transcript("main")
    assert prover.prove_class(tr2, pts, [(dcols[c], plain_roots[c], t) for c, t in zip(ent_col, zid)], R, Q, "tf-bo1") == want
