"""Integer-layer gadgets (zk_hillclimb_b200.ig) on CPU: the host logic over an oracle-backed engine produces
proofs the reference's own host-only verifiers accept, ending on the same transcript state; tampered proofs
are rejected; the function tables equal the reference's build_tables."""
import numpy as np
import pytest

from ig_helpers import OracleGadgetEngine, arr, commit, ref_table, ref_verify3


@pytest.fixture(scope="module")
def tables(zk):
    return zk.ig.build_tables(zk.load_library(), 64, 12)


def test_function_tables_equal_reference(ref, zk, tables):
    for which, name in ((0, "EXPT"), (1, "SILU"), (2, "ISQ"), (3, "EXP4")):
        cols, tid = ref_table(ref, which)
        assert tables[name]["id"] == tid, name
        for a, b in zip(tables[name]["cols"], cols):
            assert (a == b).all()


def tamper_rejected(ref, name, st0, roots, le, R, Q, pf):
    for off in (5, 4 + 7 * 8, len(pf) // 2, len(pf) - 11):
        bad = bytearray(pf)
        bad[off] ^= 1
        assert not ref_verify3(ref, name, st0, roots, le, R, Q, bytes(bad))[0]


@pytest.mark.parametrize("le", [5, 8])
def test_iadd(orc, ref, zk, tables, le):
    R, Q = 1, 24
    ig = zk.ig
    eng = OracleGadgetEngine(orc)
    g = np.random.default_rng(le)
    a, b = g.integers(-(1 << 18), 1 << 18, 1 << le), g.integers(-(1 << 18), 1 << 18, 1 << le)
    a[0], b[0] = (1 << 18) - 1, 1 << 18                    # top of the window
    out, idxO = ig.iadd_witness(ig.lift(a), ig.lift(b))
    A, B, O = (commit(eng, arr(eng, x), R) for x in (ig.lift(a), ig.lift(b), out))
    tr = zk.Transcript("iadd")
    pf = ig.iadd_prove(eng, tr, tables, A, B, O, arr(eng, idxO), le, R, Q)
    st0 = zk.Transcript("iadd").state
    ok, st = ref_verify3(ref, "ref_iadd_verify", st0, [A[1], B[1], O[1]], le, R, Q, pf)
    assert ok and st == tr.state
    tamper_rejected(ref, "ref_iadd_verify", st0, [A[1], B[1], O[1]], le, R, Q, pf)
    with pytest.raises(ValueError):
        ig.iadd_witness(ig.lift(np.array([1 << 18])), ig.lift(np.array([1 << 18])))


@pytest.mark.parametrize("le", [5, 7])
def test_iswg(orc, ref, zk, tables, le):
    R, Q = 1, 24
    ig = zk.ig
    eng = OracleGadgetEngine(orc)
    g = np.random.default_rng(100 + le)
    gv, uv = g.integers(-(1 << 19), 1 << 19, 1 << le), g.integers(-(1 << 15), 1 << 15, 1 << le)
    gv[:2] = (-(1 << 19), (1 << 19) - 1)
    sil, rem, mo, iG, iR, iM = ig.iswg_witness(ig.lift(gv), ig.lift(uv), tables)
    G, U, MO = (commit(eng, arr(eng, x), R) for x in (ig.lift(gv), ig.lift(uv), mo))
    tr = zk.Transcript("iswg")
    pf = ig.iswg_prove(eng, tr, tables, G, U, MO, (arr(eng, sil), arr(eng, rem), arr(eng, iG), arr(eng, iR), arr(eng, iM)), le, R, Q)
    st0 = zk.Transcript("iswg").state
    ok, st = ref_verify3(ref, "ref_iswg_verify", st0, [G[1], U[1], MO[1]], le, R, Q, pf)
    assert ok and st == tr.state
    tamper_rejected(ref, "ref_iswg_verify", st0, [G[1], U[1], MO[1]], le, R, Q, pf)


@pytest.mark.parametrize("lseq,ldh,lnh", [(2, 2, 1), (3, 3, 1)])
def test_irope(orc, ref, zk, tables, lseq, ldh, lnh):
    import ctypes as C
    R, Q = 1, 24
    ig = zk.ig
    eng = OracleGadgetEngine(orc)
    g = np.random.default_rng(7 + lseq)
    ld, lT = ldh + lnh, lseq
    le = lT + ld
    ct = g.integers(-(1 << 14), (1 << 14) + 1, (1 << lseq, 1 << (ldh - 1))).astype(np.int32)
    sn = g.integers(-(1 << 14), (1 << 14) + 1, (1 << lseq, 1 << (ldh - 1))).astype(np.int32)
    q = ig.lift(g.integers(-(1 << 17), 1 << 17, 1 << le))
    y, rem, iR, iY, Cc, S2 = ig.irope_witness(q, ct, sn, lseq, ldh, lT, ld)
    Qc, Y = commit(eng, arr(eng, q), R), commit(eng, arr(eng, y), R)
    pub = (arr(eng, ig.lift(Cc)), arr(eng, ig.lift(S2)), ldh)
    tr = zk.Transcript("irope")
    pf = ig.irope_prove(eng, tr, tables, pub, Qc, Y, (arr(eng, rem), arr(eng, iR), arr(eng, iY)), lT, ld, R, Q)

    def verify(proof):
        s = (C.c_uint8 * 32)(*zk.Transcript("irope").state)
        ok = ref.lib.ref_irope_verify(s, ct.ctypes.data_as(C.c_void_p), sn.ctypes.data_as(C.c_void_p), C.c_uint32(lseq),
                                      C.c_uint32(ldh), Qc[1], Y[1], C.c_uint32(lT), C.c_uint32(ld), C.c_uint32(R), C.c_uint32(Q),
                                      bytes(proof), C.c_size_t(len(proof)))
        return bool(ok), bytes(s)
    ok, st = verify(pf)
    assert ok and st == tr.state
    for off in (3, 50, len(pf) // 2, len(pf) - 11):
        bad = bytearray(pf)
        bad[off] ^= 1
        assert not verify(bad)[0]


@pytest.mark.parametrize("lT,ld", [(2, 3), (3, 4)])
def test_irms(orc, ref, zk, lT, ld):
    R, Q = 1, 24
    ig = zk.ig
    T = ig.build_tables(zk.load_library(), 1 << ld, 12)          # ISQ depends on the row width d
    eng = OracleGadgetEngine(orc)
    g = np.random.default_rng(lT * 10 + ld)
    le = lT + ld
    x = ig.lift(g.integers(-(1 << 17), 1 << 17, 1 << le))
    gains = ig.lift(g.integers(1 << 15, 1 << 17, 1 << ld))
    w = ig.irms_witness(x, gains, T, lT, ld)
    X, G, Y = commit(eng, arr(eng, x), R), commit(eng, arr(eng, gains), R), commit(eng, arr(eng, w["y"]), R)
    wit = dict(w)
    wit["db"] = [arr(eng, c) for c in w["db"]]
    wit["de"] = [arr(eng, c) for c in w["de"]]
    for k in ("idxE4", "idxM16", "idxMS", "idxISQ", "idxLR1", "idxRW", "idxW", "idxRY", "idxY"):
        wit[k] = arr(eng, w[k])
    wit["idxL"] = [arr(eng, i) for i in w["idxL"]]
    tr = zk.Transcript("irms")
    pf = ig.irms_prove(eng, tr, T, X, G, Y, wit, lT, ld, R, Q)
    import ctypes as C

    def verify(proof):
        s = (C.c_uint8 * 32)(*zk.Transcript("irms").state)
        ok = ref.lib.ref_irms_verify(s, X[1], G[1], Y[1], C.c_uint32(lT), C.c_uint32(ld), C.c_uint32(R), C.c_uint32(Q),
                                     bytes(proof), C.c_size_t(len(proof)))
        return bool(ok), bytes(s)
    ok, st = verify(pf)
    assert ok and st == tr.state
    for off in (9, 8 + 32 * 21 + 3, len(pf) // 3, len(pf) - 11):
        bad = bytearray(pf)
        bad[off] ^= 1
        assert not verify(bad)[0]


@pytest.mark.parametrize("la,lseq", [(1, 2), (0, 3)])
def test_ismx(orc, ref, zk, tables, la, lseq):
    import ctypes as C
    R, Q = 1, 24
    ig = zk.ig
    eng = OracleGadgetEngine(orc)
    g = np.random.default_rng(la * 10 + lseq)
    le = la + 2 * lseq
    z = ig.lift(g.integers(-2000, 2000, 1 << le))
    w = ig.ismx_witness(z, tables, la, lseq)
    Z, P = commit(eng, arr(eng, z), R), commit(eng, arr(eng, w["p"]), R)
    wit = {"xe": [arr(eng, c) for c in w["xe"]], "xb": [arr(eng, c) for c in w["xb"]], "idxDM": arr(eng, w["idxDM"]),
           "idxL": [arr(eng, i) for i in w["idxL"]], "idxMX": arr(eng, w["idxMX"])}
    tr = zk.Transcript("ismx")
    pf = ig.ismx_prove(eng, tr, tables, Z, P, wit, la, lseq, R, Q)

    def verify(proof):
        s = (C.c_uint8 * 32)(*zk.Transcript("ismx").state)
        ok = ref.lib.ref_ismx_verify(s, Z[1], P[1], C.c_uint32(la), C.c_uint32(lseq), C.c_uint32(R), C.c_uint32(Q), bytes(proof),
                                     C.c_size_t(len(proof)))
        return bool(ok), bytes(s)
    ok, st = verify(pf)
    assert ok and st == tr.state
    for off in (9, 8 + 32 * 9 + 3, len(pf) // 3, len(pf) - 11):
        bad = bytearray(pf)
        bad[off] ^= 1
        assert not verify(bad)[0]
