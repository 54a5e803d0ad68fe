"""The rescale gadget's host logic (zk_hillclimb_b200.p3.irs_prove / lu_flush) on CPU.

The per-GPU engine is replaced by a stand-in built on the oracle (test infrastructure); the proof must
be accepted by the reference's own host-only verifier (p3irs::verify through oracle/_ref), ending on the
same transcript state, and tampered proofs must be rejected."""
import numpy as np
import pytest

from irs_helpers import OracleIrsEngine, irs_tables, lift, ref_irs_verify, ref_irs_witness, rescale_witness
from lu_helpers import _Arr


def instance(le, sf, rng, seed):
    g = np.random.default_rng(seed)
    win = (1 << 19) if rng == 1 else (1 << 15)
    ymax = win if rng else (1 << 20)
    y = g.integers(-ymax, ymax, 1 << le)
    y[:2] = (-ymax, ymax - 1)
    acc = (y << sf) + g.integers(-(1 << (sf - 1)), 1 << (sf - 1), 1 << le)
    return acc


@pytest.mark.parametrize("sf,rng", [(16, 1), (14, 2), (23, 1), (32, 0)])
def test_rescale_witness_matches_reference(ref, sf, rng):
    le = 9
    acc = instance(le, sf, rng, sf)
    y, L, iL, iY = rescale_witness(acc, sf, rng)
    nl, ry, rL, riL, riY = ref_irs_witness(ref, lift(acc), le, sf, rng)
    assert nl == len(L) and (ry == y).all()
    for a, b in zip(L + iL, rL + riL):
        assert (a == b).all()
    if rng:
        assert (iY == riY).all()


@pytest.mark.parametrize("le,sf,rng", [(6, 16, 1), (7, 14, 2), (6, 23, 1), (5, 32, 0), (8, 20, 2)])
def test_irs_prove_accepted_by_reference_verifier(orc, ref, zk, le, sf, rng):
    R, Q = 1, 24
    eng = OracleIrsEngine(orc)
    acc = _Arr(lift(instance(le, sf, rng, 7 * le + sf)))
    y, L, iL, iY = eng.irs_witness(acc, sf, rng)
    X = (acc, eng.commit_gpu_rootonly(acc, R))
    Y = (y, eng.commit_gpu_rootonly(y, R))
    tr = zk.Transcript("irs-main")
    pf = zk.p3.irs_prove(eng, tr, irs_tables(zk, sf), X, Y, (L, iL, iY), le, sf, rng, R, Q)
    ok, st = ref_irs_verify(ref, zk.Transcript("irs-main").state, X[1], Y[1], le, sf, rng, R, Q, pf)
    assert ok and st == tr.state
    for off in (20, 16 + 32 + 5, len(pf) // 2, len(pf) - 9):
        bad = bytearray(pf)
        bad[off] ^= 1
        assert not ref_irs_verify(ref, zk.Transcript("irs-main").state, X[1], Y[1], le, sf, rng, R, Q, bytes(bad))[0]
    # wrong public parameters
    assert not ref_irs_verify(ref, zk.Transcript("irs-main").state, X[1], Y[1], le, sf, 1 if rng != 1 else 2, R, Q, pf)[0]


def test_lu_flush_groups_by_table_and_size(orc, ref, zk):
    """Two gadgets sharing one ledger and one lookup queue: their limb lookups into the same table merge
    into one instance (subgroups by size), as in p3lu::lu_flush; the reference verifier is run per gadget
    through its own tail, so here the merged flush is checked for shape and self-consistency."""
    R, Q = 1, 24
    eng = OracleIrsEngine(orc)
    ledger, luq = zk.p3.Ledger(), []
    tr = zk.Transcript("irs-two")
    tabs = irs_tables(zk, 16)
    for le, seed in ((5, 1), (6, 2), (5, 3)):
        acc = _Arr(lift(instance(le, 16, 1, seed)))
        y, L, iL, iY = eng.irs_witness(acc, 16, 1)
        X = (acc, eng.commit_gpu_rootonly(acc, R))
        Y = (y, eng.commit_gpu_rootonly(y, R))
        zk.p3.irs_prove(eng, tr, tabs, X, Y, (L, iL, iY), le, 16, 1, R, Q, ledger=ledger, luq=luq)
    assert len(luq) == 6
    groups = zk.p3.lu_flush(eng, tr, luq, ledger, R)
    assert len(groups) == 2 and not luq                 # R16 and RS20, one merged instance each
    import struct
    for g, m in zip(groups, (16, 20)):
        gm, gc, gns = struct.unpack_from("<III", g)
        assert (gm, gc, gns) == (m, 1, 2)               # subgroups: 2^5 rows (2 members), 2^6 rows (1 member)
    sizes = sorted(c[0] for c in ledger.cls)
    assert sizes == [5, 6, 16, 20]
    for v, pts, ents, ys in ledger.cls:
        for (col, root, zid), yv in zip(ents, ys):
            assert orc.mle_eval(col.a, pts[zid]) == yv
