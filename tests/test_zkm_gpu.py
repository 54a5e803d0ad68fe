"""Hiding mode on CUDA: the zk matmul proof equals the CPU engine's bytes, is accepted by the reference's verifier with its zk
switch on, and equals the reference's own zk prover byte for byte (same master seed, same draw order)."""
import numpy as np
import pytest

from imm_helpers import matmul_instance
from lu_helpers import _Arr
from zkm_helpers import ref_zk, OracleZkEngine, ref_imm_prove_zk, ref_imm_verify_zk, ref_irs_prove_zk, ref_irs_verify_zk

pytestmark = pytest.mark.gpu
GL_P = 0xFFFFFFFF00000001


def commit3(zk, eng, zc, x, w, y, dims, R, wrap):
    zkm = zk.zkm
    lj, lk, li = dims
    X = zkm.commit_col(eng, zc, wrap(x), R)
    W = zkm.commit_col(eng, zc, wrap(w), R)
    Y = zkm.commit_col(eng, zc, wrap(y), R, mask=zkm.linked_y_mask(eng, zc, X, W, lj, lk, li))
    return X, W, Y


@pytest.mark.parametrize("dims,sblind_min", [((3, 2, 3), 22), ((4, 3, 3), 22), ((3, 2, 3), 5), ((4, 4, 2), 8)])
def test_zk_matmul_equals_cpu_engine(orc, ref_or_none, zk, prover, dims, sblind_min):
    R, Q, seed = 1, 24, 31
    lj, lk, li = dims
    x, w, y = matmul_instance(orc, lj, lk, li, seed)
    out = []
    for eng, wrap in ((OracleZkEngine(orc), _Arr), (prover, zk.p3.to_device)):
        zc = zk.zkm.ZkCtx(seed=seed, Q=Q, sblind_min=sblind_min)
        X, W, Y = commit3(zk, eng, zc, x, w, y, dims, R, wrap)
        tr = zk.Transcript("imm-t")
        pf = zk.zkm.imm_prove(eng, zc, tr, X, W, Y, lj, lk, li, R, Q)
        out.append((pf, tr.state, [X.root, W.root, Y.root]))
    assert out[0][2] == out[1][2] and out[0][1] == out[1][1] and out[0][0] == out[1][0]
    if ref_or_none:
        ok, st = ref_imm_verify_zk(ref_or_none, zk.Transcript("imm-t").state, out[1][2], lj, lk, li, R, Q, out[1][0], sblind_min)
        assert ok and st == out[1][1]


@pytest.mark.parametrize("dims,sblind_min", [((4, 3, 5), 22), ((6, 6, 5), 22), ((6, 6, 5), 12), ((8, 7, 6), 22)])
def test_zk_matmul_equals_reference_prover(orc, ref, zk, prover, dims, sblind_min):
    """Merged blinds below the structured threshold, structured blinds above: same bytes as p3imm::prove with zk on."""
    R, Q, seed = 1, 24, 0xC0FFEE
    lj, lk, li = dims
    x, w, y = matmul_instance(orc, lj, lk, li, 3)
    st0 = zk.Transcript("imm-t").state
    want, st_ref, roots_ref, _ = ref_imm_prove_zk(ref, st0, x, w, lj, lk, li, R, Q, seed, sblind_min)
    assert len(want) > 0
    zc = zk.zkm.ZkCtx(seed=seed, Q=Q, sblind_min=sblind_min)
    X, W, Y = commit3(zk, prover, zc, x, w, y, dims, R, zk.p3.to_device)
    assert [X.root, W.root, Y.root] == roots_ref
    tr = zk.Transcript("imm-t")
    pf = zk.zkm.imm_prove(prover, zc, tr, X, W, Y, lj, lk, li, R, Q)
    assert tr.state == st_ref and pf == want
    ok, st = ref_imm_verify_zk(ref, st0, roots_ref, lj, lk, li, R, Q, pf, sblind_min)
    assert ok and st == tr.state


def test_blinded_zero_check_matches_python_evaluation(orc, zk, prover):
    from conftest import lcg_cols
    logn, nc = 6, 5
    cols = lcg_cols(orc, 1 << logn, nc, 99)
    terms = [(3, (1, 2)), (7, (3, 4, 4)), (5, (2,), True)]
    rng = np.random.default_rng(1)
    table = [[int(v) for v in rng.integers(1, GL_P, 7, dtype=np.uint64)] for _ in range(logn)]
    tr1, tr2 = zk.Transcript("zb"), zk.Transcript("zb")
    a = prover.sc_prove_zc_blind(tr1, "t", [zk.p3.to_device(c) for c in cols], terms, 17, table)
    b = OracleZkEngine(orc).sc_prove_zc_blind(tr2, "t", [_Arr(c) for c in cols], terms, 17, table)
    assert tr1.state == tr2.state and a[3] == b[3] and all((np.asarray(u) == np.asarray(v)).all() for u, v in zip(a[:3], b[:3]))


def _acc(le, sf, rng, seed):
    from irs_helpers import lift
    r = np.random.default_rng(seed)
    win = (1 << 19) if rng == 1 else (1 << 15)
    return lift(r.integers(-(win - 2) << sf, (win - 2) << sf, 1 << le))


@pytest.mark.parametrize("le,sf,rng,sblind_min", [(4, 16, 2, 22), (5, 20, 2, 22), (5, 16, 2, 6)])
def test_zk_rescale_equals_cpu_engine(orc, zk, prover, le, sf, rng, sblind_min):
    from irs_helpers import irs_tables
    R, Q = 1, 24
    acc = _acc(le, sf, rng, le + sf)
    out = []
    for eng, wrap in ((OracleZkEngine(orc), _Arr), (prover, zk.p3.to_device)):
        zc = zk.zkm.ZkCtx(seed=9, Q=Q, sblind_min=sblind_min)
        T = irs_tables(zk, sf)
        X = zk.zkm.commit_col(eng, zc, wrap(acc), R)
        yo, L, iL, iY = eng.irs_witness(X.dev[:1 << le] if eng is prover else _Arr(acc), sf, rng)
        Y = zk.zkm.commit_col(eng, zc, yo, R)
        tr = zk.Transcript("irs-t")
        pf = zk.zkm.irs_prove(eng, zc, tr, T, X, Y, (L, iL, iY), le, sf, rng, R, Q)
        out.append((pf, tr.state, X.root, Y.root))
    assert out[0][2:] == out[1][2:] and out[0][1] == out[1][1] and out[0][0] == out[1][0]


@pytest.mark.parametrize("le,sf,rng,sblind_min", [(6, 16, 1, 22), (10, 16, 1, 22), (12, 20, 2, 22), (12, 16, 1, 10), (16, 16, 1, 22)])
def test_zk_rescale_equals_reference_prover(orc, ref, zk, prover, le, sf, rng, sblind_min):
    """Same bytes as p3irs::prove with the zk switch on: limb commitments, the merged range lookups with their mask-leaf
    streams, the blinded zero-check, the flush and the blinded batched openings."""
    from irs_helpers import irs_tables
    R, Q, seed = 1, 24, 0xFEED
    acc = _acc(le, sf, rng, 5)
    st0 = zk.Transcript("irs-t").state
    want, st_ref, roots_ref, _ = ref_irs_prove_zk(ref, st0, acc, le, sf, rng, R, Q, seed, sblind_min)
    assert len(want) > 0
    zc = zk.zkm.ZkCtx(seed=seed, Q=Q, sblind_min=sblind_min)
    T = irs_tables(zk, sf)
    X = zk.zkm.commit_col(prover, zc, zk.p3.to_device(acc), R)
    yo, L, iL, iY = prover.irs_witness(X.dev[:1 << le], sf, rng)
    Y = zk.zkm.commit_col(prover, zc, yo, R)
    assert [X.root, Y.root] == roots_ref
    tr = zk.Transcript("irs-t")
    pf = zk.zkm.irs_prove(prover, zc, tr, T, X, Y, (L, iL, iY), le, sf, rng, R, Q)
    assert tr.state == st_ref and pf == want
    ok, st = ref_irs_verify_zk(ref, st0, X.root, Y.root, le, sf, rng, R, Q, pf, sblind_min)
    assert ok and st == tr.state


def _ref_verify3_zk(ref, name, st, roots, le, R, Q, proof):
    from ig_helpers import ref_verify3
    ref_zk(ref, True, Q, 1, 22)
    try:
        return ref_verify3(ref, name, st, roots, le, R, Q, proof)
    finally:
        ref_zk(ref, False)


def test_zk_residual_add_and_swiglu_accepted_by_reference_verifier(orc, ref, zk, prover):
    """p3iadd and p3iswg in hiding mode (blinded zero-check + merged lookups into the 2^20-row window and SILU tables); the
    same host logic runs on the CPU engine in minutes, so it lives in the GPU suite."""
    from ig_helpers import ref_table
    from irs_helpers import lift
    import torch
    R, Q, le = 1, 24, 6
    _dev32 = lambda a: torch.from_numpy(np.ascontiguousarray(a).astype(np.int32)).cuda()
    zkm, ig = zk.zkm, zk.ig
    eng, _Arr = prover, zk.p3.to_device
    T = ig.build_tables(zk.load_library(), 64, 12)
    r = np.random.default_rng(3)
    a, b = r.integers(-(1 << 17), 1 << 17, 1 << le), r.integers(-(1 << 17), 1 << 17, 1 << le)
    zc = zkm.ZkCtx(seed=21, Q=Q)
    A, B = zkm.commit_col(eng, zc, _Arr(lift(a)), R), zkm.commit_col(eng, zc, _Arr(lift(b)), R)
    OUT = zkm.commit_col(eng, zc, _Arr(lift(a + b)), R)
    tr = zk.Transcript("iad-t")
    pf = zkm.iadd_prove(eng, zc, tr, T, A, B, OUT, _dev32((a + b + ig.ABND).astype(np.uint32)), le, R, Q)
    st0 = zk.Transcript("iad-t").state
    ok, st = _ref_verify3_zk(ref, "ref_iadd_verify", st0, [A.root, B.root, OUT.root], le, R, Q, pf)
    assert ok and st == tr.state
    assert not _ref_verify3_zk(ref, "ref_iadd_verify", st0, [B.root, A.root, OUT.root], le, R, Q, pf)[0]
    # SwiGLU product
    g, u = lift(r.integers(-(1 << 18), 1 << 18, 1 << le)), lift(r.integers(-(1 << 17), 1 << 17, 1 << le))
    sil, rem, mo, idxG, idxR, idxM = ig.iswg_witness(g, u, T)
    zc = zkm.ZkCtx(seed=22, Q=Q)
    G, U, MO = (zkm.commit_col(eng, zc, _Arr(x), R) for x in (g, u, mo))
    tr = zk.Transcript("isw-t")
    pf = zkm.iswg_prove(eng, zc, tr, T, G, U, MO, (_Arr(sil), _Arr(rem), _dev32(idxG), _dev32(idxR), _dev32(idxM)), le, R, Q)
    st0 = zk.Transcript("isw-t").state
    ok, st = _ref_verify3_zk(ref, "ref_iswg_verify", st0, [G.root, U.root, MO.root], le, R, Q, pf)
    assert ok and st == tr.state
    bad = bytearray(pf)
    bad[len(pf) // 2] ^= 1
    assert not _ref_verify3_zk(ref, "ref_iswg_verify", st0, [G.root, U.root, MO.root], le, R, Q, bytes(bad))[0]


def _with_zk(ref, fn):
    ref_zk(ref, True, 24, 1, 22)
    try:
        return fn()
    finally:
        ref_zk(ref, False)


def test_zk_rope_accepted_by_reference_verifier(orc, ref, zk, prover):
    import ctypes as C
    import torch
    R, Q, (lseq, ldh, lnh) = 1, 24, (3, 3, 1)
    zkm, ig = zk.zkm, zk.ig
    T = ig.build_tables(zk.load_library(), 64, 12)
    dev, d32 = zk.p3.to_device, lambda a: torch.from_numpy(np.ascontiguousarray(a).astype(np.int32)).cuda()
    g = np.random.default_rng(11)
    ld, lT = ldh + lnh, lseq
    le = lT + ld
    ct = g.integers(-(1 << 14), (1 << 14) + 1, (1 << lseq, 1 << (ldh - 1))).astype(np.int32)
    sn = g.integers(-(1 << 14), (1 << 14) + 1, (1 << lseq, 1 << (ldh - 1))).astype(np.int32)
    q = ig.lift(g.integers(-(1 << 17), 1 << 17, 1 << le))
    y, rem, iR, iY, Cc, S2 = ig.irope_witness(q, ct, sn, lseq, ldh, lT, ld)
    zc = zkm.ZkCtx(seed=41, Q=Q)
    Qc, Y = zkm.commit_col(prover, zc, dev(q), R), zkm.commit_col(prover, zc, dev(y), R)
    tr = zk.Transcript("irope")
    pf = zkm.irope_prove(prover, zc, tr, T, (dev(ig.lift(Cc)), dev(ig.lift(S2)), ldh), Qc, Y, (dev(rem), d32(iR), d32(iY)), lT, ld, R, Q)

    def verify(proof):
        s = (C.c_uint8 * 32)(*zk.Transcript("irope").state)
        ok = ref.lib.ref_irope_verify(s, ct.ctypes.data_as(C.c_void_p), sn.ctypes.data_as(C.c_void_p), C.c_uint32(lseq),
                                      C.c_uint32(ldh), Qc.root, Y.root, C.c_uint32(lT), C.c_uint32(ld), C.c_uint32(R), C.c_uint32(Q),
                                      bytes(proof), C.c_size_t(len(proof)))
        return bool(ok), bytes(s)
    ok, st = _with_zk(ref, lambda: verify(pf))
    assert ok and st == tr.state
    bad = bytearray(pf)
    bad[len(pf) // 2] ^= 1
    assert not _with_zk(ref, lambda: verify(bad))[0]


def test_zk_rmsnorm_accepted_by_reference_verifier(orc, ref, zk, prover):
    """The row column M carries a LINKED mask (CEPS + row sums of squares of X's first mask slice): with a fresh mask instead,
    the hiding row-sum binding fails and the reference refuses the proof."""
    import ctypes as C
    import torch
    R, Q, (lT, ld) = 1, 24, (3, 4)
    zkm, ig = zk.zkm, zk.ig
    T = ig.build_tables(zk.load_library(), 1 << ld, 12)
    dev, d32 = zk.p3.to_device, lambda a: torch.from_numpy(np.ascontiguousarray(a).astype(np.int32)).cuda()
    g = np.random.default_rng(34)
    le = lT + ld
    x = ig.lift(g.integers(-(1 << 17), 1 << 17, 1 << le))
    gains = ig.lift(g.integers(1 << 15, 1 << 17, 1 << ld))
    w = ig.irms_witness(x, gains, T, lT, ld)
    wit = dict(w)
    wit["db"] = [dev(c) for c in w["db"]]
    wit["de"] = [dev(c) for c in w["de"]]
    for k in ("idxE4", "idxM16", "idxMS", "idxISQ", "idxLR1", "idxRW", "idxW", "idxRY", "idxY"):
        wit[k] = d32(w[k])
    wit["idxL"] = [d32(i) for i in w["idxL"]]
    zc = zkm.ZkCtx(seed=43, Q=Q)
    X, G, Y = (zkm.commit_col(prover, zc, dev(a), R) for a in (x, gains, w["y"]))
    tr = zk.Transcript("irms")
    pf = zkm.irms_prove(prover, zc, tr, T, X, G, Y, wit, lT, ld, R, Q)

    def verify(proof):
        s = (C.c_uint8 * 32)(*zk.Transcript("irms").state)
        ok = ref.lib.ref_irms_verify(s, X.root, G.root, Y.root, C.c_uint32(lT), C.c_uint32(ld), C.c_uint32(R), C.c_uint32(Q),
                                     bytes(proof), C.c_size_t(len(proof)))
        return bool(ok), bytes(s)
    ok, st = _with_zk(ref, lambda: verify(pf))
    assert ok and st == tr.state
    bad = bytearray(pf)
    bad[len(pf) // 3] ^= 1
    assert not _with_zk(ref, lambda: verify(bad))[0]


def test_zk_softmax_accepted_by_reference_verifier(orc, ref, zk, prover):
    """Causal softmax rows in hiding mode: the first mask slice of the row sums S is linked to the row sums of EE's."""
    import ctypes as C
    import torch
    R, Q, (la, lseq) = 1, 24, (1, 3)
    zkm, ig = zk.zkm, zk.ig
    T = ig.build_tables(zk.load_library(), 64, 12)
    dev, d32 = zk.p3.to_device, lambda a: torch.from_numpy(np.ascontiguousarray(a).astype(np.int32)).cuda()
    g = np.random.default_rng(17)
    le = la + 2 * lseq
    z = ig.lift(g.integers(-2000, 2000, 1 << le))
    w = ig.ismx_witness(z, T, la, lseq)
    wit = {"xe": [dev(c) for c in w["xe"]], "xb": [dev(c) for c in w["xb"]], "idxDM": d32(w["idxDM"]),
           "idxL": [d32(i) for i in w["idxL"]], "idxMX": d32(w["idxMX"])}
    zc = zkm.ZkCtx(seed=47, Q=Q)
    Z, P = zkm.commit_col(prover, zc, dev(z), R), zkm.commit_col(prover, zc, dev(w["p"]), R)
    tr = zk.Transcript("ismx")
    pf = zkm.ismx_prove(prover, zc, tr, T, Z, P, wit, la, lseq, R, Q)

    def verify(proof):
        s = (C.c_uint8 * 32)(*zk.Transcript("ismx").state)
        ok = ref.lib.ref_ismx_verify(s, Z.root, P.root, C.c_uint32(la), C.c_uint32(lseq), C.c_uint32(R), C.c_uint32(Q), bytes(proof),
                                     C.c_size_t(len(proof)))
        return bool(ok), bytes(s)
    ok, st = _with_zk(ref, lambda: verify(pf))
    assert ok and st == tr.state
    bad = bytearray(pf)
    bad[len(pf) // 3] ^= 1
    assert not _with_zk(ref, lambda: verify(bad))[0]


@pytest.mark.parametrize("dims", [(4, 8, 2, 4, 16, 1), (8, 16, 2, 8, 32, 2)])
def test_zk_integer_layer_equals_reference_prover(orc, ref, zk, prover, dims):
    """The whole decoder layer in hiding mode (p3itf with the zk switch on): 26 + 2A blinded sub-proofs, linked accumulator
    masks, merged lookups over mask-interleaved trees, blinded openings.  Accepted by the reference's layer verifier and, with
    the same master seed, the bytes of the reference's own zk layer prover."""
    from ig_helpers import layer_inputs, ref_itf_prove, ref_itf_verify
    from test_itf_gpu import device_col
    R, Q, seed = 1, 24, 0xABCDEF
    ig, zkm = zk.ig, zk.zkm
    c = ig.Config(*dims)
    T = ig.build_tables(zk.load_library(), c.d, c.btop)
    x0, Wt = layer_inputs(ig, c, 5)
    w = ig.itf_build_witness(c, x0, Wt, T)
    col = device_col(zk)
    zc = zkm.ZkCtx(seed=seed, Q=Q)
    o = zkm.itf_commit_all(prover, zc, c, w, Wt, R, col)
    tr = zk.Transcript("itf-layer")
    pf = zkm.itf_prove(prover, zc, tr, c, w, o, Wt, T, R, Q, col)
    wroots = [x.root for x in o["w"]] + [o["g1"].root, o["g2"].root]
    st0 = zk.Transcript("itf-layer").state
    ok, st = _with_zk(ref, lambda: ref_itf_verify(ref, st0, c, x0, o["x0"].root, wroots, Wt, w["out"], R, Q, pf))
    assert ok and st == tr.state, getattr(ref, "last_why", "")
    bad = bytearray(pf)
    bad[len(pf) // 2] ^= 1
    assert not _with_zk(ref, lambda: ref_itf_verify(ref, st0, c, x0, o["x0"].root, wroots, Wt, w["out"], R, Q, bytes(bad)))[0]
    ref_zk(ref, True, Q, seed, 22)
    try:
        rpf, rst, grid, ms = ref_itf_prove(ref, st0, c, x0, Wt, R, Q)
    finally:
        ref_zk(ref, False)
    assert (grid == w["out"]).all()
    assert rst == tr.state and rpf == pf
    # codewords and salted trees kept in HBM for the openings (within a byte budget): the same proof
    zc = zkm.ZkCtx(seed=seed, Q=Q, keep_bytes=1 << 28)
    o2 = zkm.itf_commit_all(prover, zc, c, w, Wt, R, col)
    assert o2["x0"].tree is not None
    tr2 = zk.Transcript("itf-layer")
    assert zkm.itf_prove(prover, zc, tr2, c, w, o2, Wt, T, R, Q, col) == pf and tr2.state == tr.state


@pytest.mark.parametrize("logn,rounds,with_table", [(6, 3, True), (5, 5, True), (7, 1, False), (4, 3, False), (9, 8, True)])
def test_partial_zero_check_matches_python_evaluation(orc, zk, prover, logn, rounds, with_table):
    """A chain stopped before its last variables: messages, challenges, what every column still holds, the blind's prefix."""
    from conftest import lcg_cols
    nc = 4
    cols = lcg_cols(orc, 1 << logn, nc, 5 * logn + rounds)
    terms = [(3, (1, 2)), (7, (3,)), (5, (2,), True)]
    rng = np.random.default_rng(rounds)
    table = [[int(v) for v in rng.integers(1, GL_P, 7, dtype=np.uint64)] for _ in range(rounds)] if with_table else None
    tr1, tr2 = zk.Transcript("zp"), zk.Transcript("zp")
    a = prover.sc_prove_zc_partial(tr1, "t", [zk.p3.to_device(c) for c in cols], terms, 17, rounds, table, 12345)
    b = OracleZkEngine(orc).sc_prove_zc_partial(tr2, "t", [_Arr(c) for c in cols], terms, 17, rounds, table, 12345)
    assert tr1.state == tr2.state and a[3] == b[3]
    assert all((np.asarray(u) == np.asarray(v)).all() for u, v in zip(a[:3], b[:3]))


@pytest.mark.parametrize("dims,sblind_min", [((3, 2, 3), 5), ((5, 4, 4), 9), ((0, 4, 4), 6)])
def test_factored_matmul_chain_equals_materialised_chain_on_cuda(orc, zk, prover, dims, sblind_min):
    R, Q, seed = 1, 24, 77
    lj, lk, li = dims
    x, w, y = matmul_instance(orc, lj, lk, li, seed)
    out = []
    for materialise in (True, False):
        zc = zk.zkm.ZkCtx(seed=seed, Q=Q, sblind_min=sblind_min)
        zc.materialise = materialise
        X, W, Y = commit3(zk, prover, zc, x, w, y, dims, R, zk.p3.to_device)
        tr = zk.Transcript("imm-t")
        out.append((zk.zkm.imm_prove(prover, zc, tr, X, W, Y, lj, lk, li, R, Q), tr.state))
    assert out[0] == out[1]
