"""The CPU oracle against the golden vectors minted from the reference's host code
(tests/golden/make_golden.py), and against the reference itself where its shim is built."""
import hashlib

import numpy as np
import pytest

from conftest import dig, lcg_cols

GL_P = 0xFFFFFFFF00000001


def test_field(golden, orc):
    for a, b, s, d, m, inv in golden["field"]:
        assert orc.gl_add(a, b) == s == (a + b) % GL_P
        assert orc.gl_sub(a, b) == d == (a - b) % GL_P
        assert orc.gl_mul(a, b) == m == (a * b) % GL_P
        if a:
            assert orc.gl_inv(a) == inv == pow(a, GL_P - 2, GL_P)
    for l, w in enumerate(golden["roots_of_unity"], start=1):
        assert orc.gl_root_of_unity(l) == w
        assert pow(w, 1 << l, GL_P) == 1 and pow(w, 1 << (l - 1), GL_P) != 1


def test_sha_and_transcript(golden, orc):
    for m, h in golden["sha256"]:
        m = bytes.fromhex(m)
        assert orc.sha256(m).hex() == h == hashlib.sha256(m).hexdigest()
    blk, h = golden["compress64"]
    assert orc.compress64(bytes.fromhex(blk)).hex() == h
    tr = golden["transcript"]
    st = orc.tr_init("p3-golden")
    assert st.hex() == tr[0]
    for label, n, sthex, a, ix in tr[1:]:
        data = bytes((len(label) * 11 + j) & 0xFF for j in range(n))
        st = orc.tr_absorb(st, label, data)
        st, a2 = orc.tr_chal(st)
        st, ix2 = orc.tr_idx(st, 1 << 21)
        assert (st.hex(), a2, ix2) == (sthex, a, ix)


def test_multilinear_helpers(golden, orc):
    e = golden["eq"]
    z, s1 = orc.lcg(e["v"], e["seed"])
    c, _ = orc.lcg(1 << e["v"], s1)
    eq = orc.build_eq(z)
    assert dig(eq) == e["eq_digest"]
    assert orc.eval_h(c, eq) == e["eval_h"] == orc.mle_eval(c, z)
    lg = golden["lagrange"]
    t = [int(x) for x in orc.lcg(6, lg["seed"])[0]]
    assert orc.quad_eval(*t[:4]) == lg["quad"]
    assert orc.cubic_eval(*t[:5]) == lg["cubic"]
    assert orc.quartic_eval(t[:5], t[5]) == lg["quartic"]


def test_encode_merkle_fold(golden, orc):
    for e in golden["encode"]:
        v, R = e["v"], e["R"]
        cc, _ = orc.lcg(1 << v, e["seed"])
        cw = orc.rs_encode(cc, R)
        assert dig(cw) == e["cw_digest"]
        assert dig(orc.rs_encode_horner(cc, R)) == e["cw_digest"]
        assert orc.merkle_root(cw).hex() == e["root"]
        assert dig(orc.merkle_build(cw)) == e["tree_digest"]
        w, beta = orc.gl_root_of_unity(v + R), int(cc[0])
        assert dig(orc.fold(cw, w, beta, True)) == e["fold_mle_digest"]
        assert dig(orc.fold(cw, w, beta, False)) == e["fold_fri_digest"]


def test_ntt_roundtrip_and_naive_dft(orc):
    # the reference's own NTT pins: naive DFT at n=8, round trip at 2^16 (p3_commit_bench.cu:17-56)
    x, _ = orc.lcg(8, 7)
    w = orc.gl_root_of_unity(3)
    naive = [sum(int(x[j]) * pow(w, j * k, GL_P) for j in range(8)) % GL_P for k in range(8)]
    assert [int(t) for t in orc.ntt(x)] == naive
    y, _ = orc.lcg(1 << 16, 99)
    assert (orc.ntt(orc.ntt(y), inverse=True) == y).all()


def test_basefold_open(golden, orc):
    for b in golden["basefold"]:
        v, R, Q = b["v"], b["R"], b["Q"]
        cc, s2 = orc.lcg(1 << v, b["seed"])
        zz, _ = orc.lcg(v, s2)
        y = orc.mle_eval(cc, zz)
        assert y == b["y"]
        pf = orc.bf_prove_eval(cc, zz, y, R, Q, orc.rs_encode(cc, R))
        assert len(pf) == b["proof_len"] and dig(pf) == b["proof_digest"]
        assert pf[12:44].hex() == b["root0"]
        assert orc.bf_verify_eval(pf)
        # the reference's tamper battery (p3_basefold_selftest.cu:55-71), on the serialised proof
        for off in (12 + v * 32, 12 + v * 32 + v * 24, len(pf) - 8 - v * 8, 12 + v * 56 + (8 << R) + 3):
            bad = bytearray(pf)
            bad[off] ^= 1
            assert not orc.bf_verify_eval(bytes(bad))
        wrong = orc.bf_prove_eval(cc, zz, (y + 1) % GL_P, R, Q, orc.rs_encode(cc, R))
        assert not orc.bf_verify_eval(wrong)


def test_gkr(golden, orc):
    for g in golden["gkr"]:
        L, cl = g["L"], g["combine_last"]
        p, s2 = orc.lcg(1 << L, g["seed"])
        q, _ = orc.lcg(1 << L, s2)
        st0 = orc.tr_init("gkr-golden")
        st1, pf, rfin, cpq = orc.gkr_prove(st0, "lug-gA", p, q, cl)
        assert st1.hex() == g["state"] and dig(pf) == g["proof_digest"]
        assert [int(x) for x in rfin] == g["rfin"]
        if cl:
            assert list(cpq) == g["cpq"]
            assert cpq[0] == orc.mle_eval(p, rfin) and cpq[1] == orc.mle_eval(q, rfin)
        ok, st2, rf2, out4 = orc.gkr_verify(st0, "lug-gA", L, pf, cl)
        assert ok and st2 == st1 and (rf2 == rfin).all()
        if L > 1:
            bad = bytearray(pf)
            bad[-1] ^= 1
            assert not orc.gkr_verify(st0, "lug-gA", L, bytes(bad), cl)[0]


def test_sumcheck(golden, orc):
    from oracle import F_LOGUP, F_PROD2, F_PROD3
    fid = {"logup": (F_LOGUP, 4), "prod2": (F_PROD2, 2), "prod3": (F_PROD3, 3)}
    st0 = orc.tr_init("sc-golden")
    for s in golden["sumcheck"]:
        f, nc = fid[s["kind"]]
        cols = lcg_cols(orc, 1 << s["logn"], nc, s["seed"])
        for nthreads in (1, 4):
            st1, m, r, fin = orc.sumcheck(st0, s["tag"], f, s["nt"], cols, s["par"], nthreads)
            assert st1.hex() == s["state"] and dig(m) == s["msgs_digest"]
            assert [int(x) for x in r] == s["chals"]
        # the bound columns are the MLEs at the challenge point
        for k in range(nc):
            assert int(fin[k]) == orc.mle_eval(cols[k], r)


def test_logup_primitives(golden, orc):
    g = golden["logup"]
    A, _ = orc.lcg(g["n"], g["seed"])
    inv = orc.inv_all_add(A, g["beta"])
    assert dig(inv) == g["inv_digest"]
    assert dig(orc.combine([A, A[::-1].copy()], g["beta"])) == g["combine_digest"]
    idx = (A % np.uint64(1 << 10)).astype(np.uint32)
    cnt = orc.histogram(idx, 1 << 10)
    assert int(cnt.sum()) == len(idx) and (cnt == np.bincount(idx, minlength=1 << 10)).all()
    with pytest.raises(IndexError):
        orc.histogram(idx, 16)
    with pytest.raises(ZeroDivisionError):
        orc.inv_all_add(np.array([5, 7], dtype=np.uint64), GL_P - 7)


def _bo_inputs(orc, b):
    s, cols = b["seed"], []
    for _ in range(b["ncols"]):
        a, s = orc.lcg(1 << b["v"], s)
        cols.append(a)
    pts, s = orc.lcg(b["T"] * b["v"], s)
    return cols, pts.reshape(b["T"], b["v"])


def test_batchopen(golden, orc, ref_or_none):
    for b in golden["batchopen"]:
        v, R, Q = b["v"], b["R"], b["Q"]
        cols, pts = _bo_inputs(orc, b)
        roots_c = [orc.merkle_root(orc.rs_encode(c, R)) for c in cols]
        roots = [roots_c[c] for c in b["ent_col"]]
        st0 = orc.tr_init("bo-golden")
        pf, st1 = orc.bo_prove_class(st0, pts, [cols[c] for c in b["ent_col"]], roots, b["zid"], R, Q, "tf-bo0")
        assert dig(pf) == b["proof_digest"] and len(pf) == b["proof_len"] and st1.hex() == b["state"]
        assert b["y"] == [orc.mle_eval(cols[c], pts[t]) for c, t in zip(b["ent_col"], b["zid"])]
        for verifier in [orc] + ([ref_or_none] if ref_or_none else []):
            ok, st2 = verifier.bo_verify_class(st0, pts, roots, b["zid"], b["y"], R, Q, "tf-bo0", pf)
            assert ok and st2 == st1
            for off in (16, len(pf) // 3, len(pf) - 7):
                bad = bytearray(pf)
                bad[off] ^= 1
                assert not verifier.bo_verify_class(st0, pts, roots, b["zid"], b["y"], R, Q, "tf-bo0", bytes(bad))[0]


def test_oracle_equals_reference_live(orc, ref):
    """Where the reference shim is built (it needs the reference tree), compare directly on fresh inputs."""
    rng = np.random.default_rng(5)
    x = (rng.integers(0, 2**63, 64, dtype=np.uint64) * 2) % np.uint64(GL_P)
    for a, b in zip(x[:32], x[32:]):
        a, b = int(a), int(b)
        assert orc.gl_mul(a, b) == ref.gl_mul(a, b)
    c, s = orc.lcg(1 << 7, 42)
    z, _ = orc.lcg(7, s)
    cw = orc.rs_encode(c, 2)
    assert (cw == ref.rs_encode_horner(c, 2)).all()
    y = orc.mle_eval(c, z)
    pf = orc.bf_prove_eval(c, z, y, 2, 24, cw, "seed-live")
    assert pf == ref.bf_prove_eval(c, z, y, 2, 24, cw, "seed-live")
    assert ref.bf_verify_eval(pf, "seed-live") and not ref.bf_verify_eval(pf, "other-seed")


def test_hawkeye_constraint_sumchecks_reference_live(golden, orc, ref):
    """The fp8 gadget's quartic zero-checks have the reference's host loop itself as their oracle
    (p3hwl::sc5_prove over F_dp .. F_do through oracle/_ref): it must reproduce the committed vectors."""
    from oracle import HW_SHAPE
    for gv in golden["hawkeye_sumcheck"]:
        nc, nlam = HW_SHAPE[gv["functor"]]
        assert (nc, nlam) == (gv["nc"], gv["nlam"])
        s, cols = gv["seed"], []
        for _ in range(nc):
            a, s = orc.lcg(1 << gv["logn"], s)
            cols.append(a)
        lam, s = orc.lcg(nlam, s)
        st, m, r = ref.sc5_prove_lam(ref.tr_init("hw-golden"), gv["tag"], gv["functor"], cols, lam)
        assert st.hex() == gv["state"] and dig(m) == gv["msgs_digest"] and [int(x) for x in r] == gv["chals"]
