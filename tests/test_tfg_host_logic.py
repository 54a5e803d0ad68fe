"""bf16 gadgets of the fp8 transformer layer through the host logic in zk_hillclimb_b200.tfg on CPU: the pinned table
artefact equals the reference generator's, and every gadget's proof is accepted by the reference's host-only verifier."""
import hashlib
import os
import sys

import numpy as np
import pytest

from hwl_helpers import host_col
from ig_helpers import OracleGadgetEngine
from tfg_helpers import bf16_add_cases, bf16_patterns, load_art, ref_swg_verify, ref_verify3, ref_verify_roots

ART_LD6_SHA256 = "72ca8b6045cf1ff65d2386e6026884b3d9e2759c7c69cd5298f8e61ae8583223"


def test_artefact_digest(zk):
    """The ld = 6 artefact file (the bytes the reference's loader reads) is pinned by its digest."""
    assert hashlib.sha256(zk.tfart.art_bytes(zk.tfart.build_art(6))).hexdigest() == ART_LD6_SHA256


def test_artefact_equals_reference_generator(zk):
    """Where the reference tree is present, its own Python generator gives the same tables."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = os.path.join(os.environ.get("ZKH_REFERENCE") or os.path.join(os.path.dirname(root), "reference"), "zkllm-src")
    if not os.path.exists(os.path.join(src, "transformer_ref.py")):
        pytest.skip("reference tree not present")
    sys.path.insert(0, src)
    try:
        import contextlib
        import io
        with contextlib.redirect_stdout(io.StringIO()):
            import transformer_ref as R
    finally:
        sys.path.remove(src)
    art = zk.tfart.build_art(6)
    for k, ref in (("mul_mo", R.MUL_MO), ("mul_einc", R.MUL_EINC), ("rsq_mr", R.RSQ_MR), ("rsq_hb", R.RSQ_HB), ("rcp_mr", R.RCP_MR),
                   ("rcp_hb", R.RCP_HB), ("exp_tab", R.EXP_TAB), ("silu_tab", R.SILU_TAB), ("qe4m3", R.QE4M3)):
        assert (np.asarray(art[k]).astype(np.int64) == np.asarray(ref).astype(np.int64)).all(), k
    for ld in (4, 7, 11):
        emin, epsa = R.epsa_table(ld)
        a = zk.tfart.build_art(ld)
        assert emin == a["EMIN"] and (epsa == a["epsa"]).all()


@pytest.mark.parametrize("ln", [1, 5])
def test_swiglu_accepted_by_reference_verifier(orc, ref, zk, ln):
    R, Q = 1, 24
    tfg = zk.tfg
    art = load_art(ref, zk)
    T = tfg.swg_tables(art)
    rng = np.random.default_rng(ln)
    gate, up = bf16_patterns(rng, 1 << ln, 2.0), bf16_patterns(rng, 1 << ln, 1.0)
    wt = tfg.swg_witness(gate, up, art)
    eng = OracleGadgetEngine(orc)
    ops = tfg.swg_commit_operands(eng, wt, R, host_col)
    tr = zk.Transcript("swg")
    pf = tfg.swg_prove(eng, tr, wt, T, ops, R, Q, host_col)
    roots3 = [ops[k][1] for k in ("GATE", "UP", "M")]
    st0 = zk.Transcript("swg").state
    ok, st = ref_swg_verify(ref, st0, roots3, 1 << ln, R, Q, pf)
    assert ok and st == tr.state
    assert not ref_swg_verify(ref, st0, roots3[1:] + roots3[:1], 1 << ln, R, Q, pf)[0]
    for off in (40, len(pf) // 2, len(pf) - 9):
        bad = bytearray(pf)
        bad[off] ^= 1
        assert not ref_swg_verify(ref, st0, roots3, 1 << ln, R, Q, bytes(bad))[0]


def _bf16_add_numpy(a, b):
    """float32 addition of bf16 values rounded back to bf16 (RNE): an independent check of the replay on in-domain rows"""
    fa = (a.astype(np.uint32) << 16).view(np.float32)
    fb = (b.astype(np.uint32) << 16).view(np.float32)
    s = (fa + fb).view(np.uint32).astype(np.uint64)
    return ((s + 0x7FFF + ((s >> 16) & 1)) >> 16).astype(np.uint16)


@pytest.mark.parametrize("ln", [1, 6])
def test_bf16_add_accepted_by_reference_verifier(orc, ref, zk, ln):
    R, Q = 1, 24
    tfg = zk.tfg
    T = tfg.bfa_tables()
    a, b = bf16_add_cases(np.random.default_rng(10 + ln), 1 << ln)
    wt = tfg.bfa_witness(a, b)
    both = ((a & 0x7F80) != 0) & ((b & 0x7F80) != 0) & ((wt["O"] & 0x7F80) != 0)      # no flushed operands / results
    assert (wt["O"][both] == _bf16_add_numpy(a, b)[both]).all()
    eng = OracleGadgetEngine(orc)
    ops = tfg.bfa_commit_operands(eng, wt, R, host_col)
    tr = zk.Transcript("bfa")
    pf = tfg.bfa_prove(eng, tr, wt, T, ops, R, Q, host_col)
    roots3 = [ops[k][1] for k in ("X1", "X2", "OUT")]
    st0 = zk.Transcript("bfa").state
    ok, st = ref_verify3(ref, "ref_bfa_verify", st0, roots3, 1 << ln, R, Q, pf)
    assert ok and st == tr.state
    assert not ref_verify3(ref, "ref_bfa_verify", st0, roots3[::-1], 1 << ln, R, Q, pf)[0]
    bad = bytearray(pf)
    bad[len(pf) // 2] ^= 1
    assert not ref_verify3(ref, "ref_bfa_verify", st0, roots3, 1 << ln, R, Q, bytes(bad))[0]


@pytest.mark.parametrize("B,ld", [(1, 3), (3, 4), (4, 6)])
def test_quantize_accepted_by_reference_verifier(orc, ref, zk, B, ld):
    R, Q = 1, 24
    tfg = zk.tfg
    art = load_art(ref, zk)
    T = tfg.qnt_tables(art)
    rng = np.random.default_rng(B * 10 + ld)
    x = bf16_patterns(rng, B << ld, 3.0).reshape(B, 1 << ld)
    x[0] = (x[0] & 0x8000)                                   # an all-zero row: the phantom floor is the row maximum
    if B > 2:
        x[2] = bf16_patterns(rng, 1 << ld, 1e-12)            # tiny row
    wt = tfg.qnt_witness(x.reshape(-1), B, ld, art)
    # scale = 2^(E-8-127), codes decode to x / scale on the e4m3 grid for a sample of elements
    assert wt["S"][0] == (1 << 23)
    eng = OracleGadgetEngine(orc)
    ops = tfg.qnt_commit_operands(eng, wt, R, host_col)
    tr = zk.Transcript("qnt")
    pf = tfg.qnt_prove(eng, tr, wt, T, ops, R, Q, host_col)
    roots3 = [ops[k][1] for k in ("X", "CODES", "SCALES")]
    st0 = zk.Transcript("qnt").state
    ok, st = ref_verify_roots(ref, "ref_qnt_verify", st0, roots3, (B, ld), R, Q, pf)
    assert ok and st == tr.state
    assert not ref_verify_roots(ref, "ref_qnt_verify", st0, roots3[::-1], (B, ld), R, Q, pf)[0]
    bad = bytearray(pf)
    bad[len(pf) // 3] ^= 1
    assert not ref_verify_roots(ref, "ref_qnt_verify", st0, roots3, (B, ld), R, Q, bytes(bad))[0]


def _rope_tables(zk, seq, dh):
    """bf16 cos / sin tables of the llama rotation, theta = 10000 (seq x dh/2 patterns)."""
    half = dh // 2
    ang = np.arange(seq, dtype=np.float64)[:, None] * (10000.0 ** (-np.arange(half, dtype=np.float64) / half))[None, :]
    to_bf = np.vectorize(zk.tfart.bf_from_f64, otypes=[np.uint16])
    return to_bf(np.cos(ang)).reshape(-1), to_bf(np.sin(ang)).reshape(-1)


@pytest.mark.parametrize("seq,dh", [(2, 4), (4, 8)])
def test_rope_accepted_by_reference_verifier(orc, ref, zk, seq, dh):
    R, Q = 1, 24
    tfg = zk.tfg
    art = load_art(ref, zk)
    T = tfg.rope_tables(art)
    cos, sin = _rope_tables(zk, seq, dh)
    q = bf16_patterns(np.random.default_rng(seq + dh), seq * dh, 1.0)
    wt = tfg.rope_witness(q, cos, sin, seq, dh, art)
    nzq = (q[:dh] & 0x7F80) != 0
    assert (wt["OUT"][:dh][nzq] == q[:dh][nzq]).all()             # position 0: cos = 1, sin = +0
    eng = OracleGadgetEngine(orc)
    ops = tfg.rope_commit_operands(eng, wt, R, host_col)
    tr = zk.Transcript("rope")
    pf = tfg.rope_prove(eng, tr, wt, T, ops, R, Q, host_col)
    roots2 = [ops["Q"][1], ops["OUT"][1]]
    st0 = zk.Transcript("rope").state
    ok, st = ref_verify_roots(ref, "ref_rope_verify", st0, roots2, (seq, dh), R, Q, pf, pre=(cos, sin))
    assert ok and st == tr.state
    assert not ref_verify_roots(ref, "ref_rope_verify", st0, roots2, (seq, dh), R, Q, pf, pre=(sin, cos))[0]
    bad = bytearray(pf)
    bad[len(pf) // 3] ^= 1
    assert not ref_verify_roots(ref, "ref_rope_verify", st0, roots2, (seq, dh), R, Q, bytes(bad), pre=(cos, sin))[0]


@pytest.mark.parametrize("B,ld", [(1, 4), (3, 6)])
def test_rmsnorm_accepted_by_reference_verifier(orc, ref, zk, B, ld):
    R, Q = 1, 24
    tfg = zk.tfg
    art = load_art(ref, zk, ld)
    T = tfg.rms_tables(art)
    rng = np.random.default_rng(B + ld)
    x = bf16_patterns(rng, B << ld, 1.5).reshape(B, 1 << ld)
    if B > 1:
        x[1] = x[1] & 0x8000                                  # zero row: eps dominates
    g = bf16_patterns(rng, 1 << ld, 0.1, zeros=0.0)
    g = ((g.astype(np.uint32) << 16).view(np.float32) + np.float32(1.0)).view(np.uint32) >> 16
    wt = tfg.rms_witness(x.reshape(-1), g.astype(np.uint16), B, art)
    # float check on an ordinary row: y ~ x * g / rms(x) within bf16 rounding of three steps
    xf = (x[0].astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    gf = (g.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    yf = (wt["Y"][:1 << ld].astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    want = xf * gf / np.sqrt((xf * xf).mean() + 1e-6)
    assert np.allclose(yf, want, rtol=0.03, atol=1e-30)
    eng = OracleGadgetEngine(orc)
    ops = tfg.rms_commit_operands(eng, wt, R, host_col)
    tr = zk.Transcript("rms")
    pf = tfg.rms_prove(eng, tr, wt, T, art, ops, R, Q, host_col)
    roots3 = [ops[k][1] for k in ("X", "G", "Y")]
    st0 = zk.Transcript("rms").state
    ok, st = ref_verify_roots(ref, "ref_rms_verify", st0, roots3, (B, ld), R, Q, pf)
    assert ok and st == tr.state
    assert not ref_verify_roots(ref, "ref_rms_verify", st0, roots3[::-1], (B, ld), R, Q, pf)[0]
    bad = bytearray(pf)
    bad[len(pf) // 3] ^= 1
    assert not ref_verify_roots(ref, "ref_rms_verify", st0, roots3, (B, ld), R, Q, bytes(bad))[0]


@pytest.mark.parametrize("B,ln", [(2, 2), (4, 3)])
def test_softmax_accepted_by_reference_verifier(orc, ref, zk, B, ln):
    R, Q = 1, 24
    tfg = zk.tfg
    art = load_art(ref, zk)
    T = tfg.smx_tables(art)
    n = 1 << ln
    rng = np.random.default_rng(B + ln)
    s = bf16_patterns(rng, B * n, 2.0).reshape(B, n)
    msk = (np.arange(n)[None, :] <= (np.arange(B)[:, None] % n)).astype(np.uint8)        # causal rows
    if B > 2:
        msk[B - 1] = 0                                                                      # a row with every lane masked
    wt = tfg.smx_witness(s.reshape(-1), msk.reshape(-1), B, ln, art)
    pf32 = (wt["P"].astype(np.uint32) << 16).view(np.float32).reshape(B, n)
    sf = (s.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    for b in range(B):
        if msk[b].any():
            e = np.where(msk[b] != 0, np.exp(sf[b] - sf[b][msk[b] != 0].max()), 0.0)
            assert np.allclose(pf32[b], e / e.sum(), rtol=0.04, atol=1e-3)
        else:
            assert (wt["P"].reshape(B, n)[b] == 0).all()
    eng = OracleGadgetEngine(orc)
    ops = tfg.smx_commit_operands(eng, wt, R, host_col)
    tr = zk.Transcript("smx")
    pf = tfg.smx_prove(eng, tr, wt, T, art, ops, R, Q, host_col)
    roots2 = [ops["S"][1], ops["P"][1]]
    st0 = zk.Transcript("smx").state
    ok, st = ref_verify_roots(ref, "ref_smx_verify", st0, roots2, (B, n, 23), R, Q, pf, pre=(msk.reshape(-1),))
    assert ok and st == tr.state
    bad_mask = msk.copy()
    bad_mask[0, n - 1] ^= 1
    assert not ref_verify_roots(ref, "ref_smx_verify", st0, roots2, (B, n, 23), R, Q, pf, pre=(bad_mask.reshape(-1),))[0]
    bad = bytearray(pf)
    bad[len(pf) // 3] ^= 1
    assert not ref_verify_roots(ref, "ref_smx_verify", st0, roots2, (B, n, 23), R, Q, bytes(bad), pre=(msk.reshape(-1),))[0]
