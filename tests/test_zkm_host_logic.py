"""Hiding mode, host logic on the CPU engine: the zk matmul proof (masked salted commitments, Libra-blinded chain, blinded
batched openings) is accepted by the reference's verifier with its zk switch on, and rejects what it must."""
import numpy as np
import pytest

from imm_helpers import matmul_instance
from lu_helpers import _Arr
from zkm_helpers import OracleZkEngine, ref_imm_verify_zk, ref_irs_verify_zk, ref_zk

GL_P = 0xFFFFFFFF00000001


def test_seed_stream_and_mask_sizes_match_reference(ref, zk):
    import ctypes as C
    try:
        ref.lib.ref_zk_next_seed.restype = C.c_uint64
        ref_zk(ref, True, 24, 77)
        zc = zk.zkm.ZkCtx(seed=77, Q=24)
        assert [zc.next_seed() for _ in range(6)] == [int(ref.lib.ref_zk_next_seed()) for _ in range(6)]
        assert [zc.e_of(v) for v in range(0, 14)] == [int(ref.lib.ref_zk_e_of(C.c_uint32(v))) for v in range(0, 14)]
    finally:
        ref_zk(ref, False)


def zk_matmul(orc, zk, lj, lk, li, seed, R, sblind_min=22):
    zkm = zk.zkm
    eng = OracleZkEngine(orc)
    zc = zkm.ZkCtx(seed=seed, Q=24, sblind_min=sblind_min)
    x, w, y = matmul_instance(orc, lj, lk, li, seed)
    X = zkm.commit_col(eng, zc, _Arr(x), R)
    W = zkm.commit_col(eng, zc, _Arr(w), R)
    Y = zkm.commit_col(eng, zc, _Arr(y), R, mask=zkm.linked_y_mask(eng, zc, X, W, lj, lk, li))
    return eng, zc, X, W, Y


@pytest.mark.parametrize("lj,lk,li,sblind_min", [(3, 2, 3, 22), (2, 3, 2, 22), (4, 3, 3, 22), (3, 2, 3, 5), (4, 4, 2, 8)])
def test_zk_matmul_accepted_by_reference_verifier(orc, ref, zk, lj, lk, li, sblind_min):
    R, Q = 1, 24
    eng, zc, X, W, Y = zk_matmul(orc, zk, lj, lk, li, 11 + lj, R, sblind_min)
    tr = zk.Transcript("imm-t")
    pf = zk.zkm.imm_prove(eng, zc, tr, X, W, Y, lj, lk, li, R, Q)
    st0 = zk.Transcript("imm-t").state
    roots = [X.root, W.root, Y.root]
    ok, st = ref_imm_verify_zk(ref, st0, roots, lj, lk, li, R, Q, pf, sblind_min)
    assert ok and st == tr.state
    # the plain verifier does not read a hiding proof, a swapped statement and flipped bytes are refused
    assert not ref_imm_verify_zk(ref, st0, [W.root, X.root, Y.root], lj, lk, li, R, Q, pf, sblind_min)[0]
    for off in (20, len(pf) // 3, len(pf) - 50):
        bad = bytearray(pf)
        bad[off] ^= 1
        assert not ref_imm_verify_zk(ref, st0, roots, lj, lk, li, R, Q, bytes(bad), sblind_min)[0]


def test_unlinked_y_mask_is_refused(orc, ref, zk):
    """Y committed with a fresh mask instead of the product of the operands' masks: the hiding claim algebra breaks."""
    R, Q, (lj, lk, li) = 1, 24, (3, 2, 3)
    eng, zc, X, W, _ = zk_matmul(orc, zk, lj, lk, li, 5, R)
    y = matmul_instance(orc, lj, lk, li, 5)[2]
    Y = zk.zkm.commit_col(eng, zc, _Arr(y), R)
    tr = zk.Transcript("imm-t")
    pf = zk.zkm.imm_prove(eng, zc, tr, X, W, Y, lj, lk, li, R, Q)
    assert not ref_imm_verify_zk(ref, zk.Transcript("imm-t").state, [X.root, W.root, Y.root], lj, lk, li, R, Q, pf)[0]


def test_zprng_at_vectorised_matches_restatement(orc):
    eng = OracleZkEngine(orc)
    got = eng.zk_fill_at(0x1234567, 50, 7).a
    assert [int(x) for x in got] == [orc.zprng_at(0x1234567, 7 + i) for i in range(50)]


@pytest.mark.parametrize("le,sf,rng,sblind_min", [(4, 16, 2, 22), (5, 20, 2, 22), (3, 14, 2, 22), (4, 16, 0, 22), (5, 16, 2, 6)])
def test_zk_rescale_accepted_by_reference_verifier(orc, ref, zk, le, sf, rng, sblind_min):
    """Rescale in hiding mode: masked limb commitments, merged range lookups over mask-interleaved fraction trees, blinded
    zero-check, blinded openings.  (The 2^20-row window table runs in the GPU suite; it takes a minute per case here.)"""
    from irs_helpers import irs_tables, lift
    R, Q = 1, 24
    zkm = zk.zkm
    eng = OracleZkEngine(orc)
    zc = zkm.ZkCtx(seed=9, Q=Q, sblind_min=sblind_min)
    r = np.random.default_rng(le + sf)
    win = (1 << 19) if rng == 1 else (1 << 15)
    acc = lift(r.integers(-(win - 2) << sf, (win - 2) << sf, 1 << le))
    T = irs_tables(zk, sf)
    X = zkm.commit_col(eng, zc, _Arr(acc), R)
    yo, L, iL, iY = eng.irs_witness(_Arr(acc), sf, rng)
    Y = zkm.commit_col(eng, zc, yo, R)
    tr = zk.Transcript("irs-t")
    pf = zkm.irs_prove(eng, zc, tr, T, X, Y, (L, iL, iY), le, sf, rng, R, Q)
    st0 = zk.Transcript("irs-t").state
    ok, st = ref_irs_verify_zk(ref, st0, X.root, Y.root, le, sf, rng, R, Q, pf, sblind_min)
    assert ok and st == tr.state
    assert not ref_irs_verify_zk(ref, st0, Y.root, X.root, le, sf, rng, R, Q, pf, sblind_min)[0]
    for off in (40, len(pf) // 2, len(pf) - 60):
        bad = bytearray(pf)
        bad[off] ^= 1
        assert not ref_irs_verify_zk(ref, st0, X.root, Y.root, le, sf, rng, R, Q, bytes(bad), sblind_min)[0]



@pytest.mark.parametrize("lj,lk,li,sblind_min", [(3, 2, 3, 5), (4, 4, 2, 8), (2, 3, 4, 4), (0, 3, 3, 4), (3, 0, 3, 4)])
def test_factored_matmul_chain_equals_materialised_chain(orc, ref, zk, lj, lk, li, sblind_min):
    """Structured blinds: the chain split over the index groups (three short product chains on partially evaluated operands
    and the slice rounds) gives the proof bytes of the chain over the materialised product domain."""
    R, Q = 1, 24
    out = []
    for materialise in (True, False):
        eng, zc, X, W, Y = zk_matmul(orc, zk, lj, lk, li, 11 + lj, R, sblind_min)
        zc.materialise = materialise
        tr = zk.Transcript("imm-t")
        out.append((zk.zkm.imm_prove(eng, zc, tr, X, W, Y, lj, lk, li, R, Q), tr.state, [X.root, W.root, Y.root]))
    assert out[0] == out[1]
    ok, st = ref_imm_verify_zk(ref, zk.Transcript("imm-t").state, out[1][2], lj, lk, li, R, Q, out[1][0], sblind_min)
    assert ok and st == out[1][1]
