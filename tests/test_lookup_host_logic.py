"""The merged-lookup host logic (zk_hillclimb_b200.p3.prove_super) on CPU.

The per-GPU engine is replaced by a stand-in built on the oracle (test infrastructure); the proof
it produces must be accepted by the reference's own host-only verifier (p3lu::verify_super through
oracle/_ref), with the same transcript state and the same opening-ledger claims."""
import numpy as np
import pytest

from lu_helpers import OracleLookupEngine, _Arr, make_lookup, table_id, verify_with_reference


def build_groups(orc, subs, R):
    groups, roots_flat, committed = [], b"", b""
    for n, members in subs:
        mem = []
        for cols, idx in members:
            roots = [orc.merkle_root(orc.rs_encode(cc, R)) for cc in cols]
            mem.append(([_Arr(cc) for cc in cols], roots, _Arr(idx)))
            roots_flat += b"".join(roots)
            committed += b"\x01" * len(cols)
        groups.append((n, mem))
    return groups, roots_flat, committed


@pytest.mark.parametrize("m,shapes", [(4, [(5, 1)]), (6, [(7, 3), (5, 2)]), (3, [(4, 5)])])
def test_prove_super_accepted_by_reference_verifier(orc, ref, zk, m, shapes):
    R, Q = 1, 24
    tcols, subs = make_lookup(orc, m, shapes, 11 + m)
    groups, roots_flat, committed = build_groups(orc, subs, R)
    tr = zk.Transcript("lu-main")
    pf, claims, cnt = zk.p3.prove_super(OracleLookupEngine(orc), tr, [_Arr(t) for t in tcols], table_id(tcols), groups, R)
    meta = [(n, len(mm)) for n, mm in groups]
    ok, st, vclaims = verify_with_reference(ref, zk.Transcript("lu-main").state, tcols, meta, roots_flat, committed, R, Q, pf)
    assert ok and st == tr.state
    mine = sorted((c[1], np.asarray(c[2], dtype=np.uint64).tobytes(), c[3]) for c in claims)
    theirs = sorted((c[0], c[1].tobytes(), c[2]) for c in vclaims)
    assert mine == theirs
    # every claimed value is the column's MLE at the claimed point
    for col, _root, pt, y in claims:
        assert orc.mle_eval(col.a, pt) == y
    assert int(cnt.a.sum()) == sum((1 << ((k - 1).bit_length() + n)) for n, k in meta)
    for off in (50, len(pf) // 2, len(pf) - 3):
        bad = bytearray(pf)
        bad[off] ^= 1
        assert not verify_with_reference(ref, zk.Transcript("lu-main").state, tcols, meta, roots_flat, committed, R, Q, bytes(bad))[0]


def test_prove_super_rejects_row_outside_table(orc, zk):
    tcols, subs = make_lookup(orc, 4, [(5, 1)], 3)
    groups, _, _ = build_groups(orc, subs, 1)
    cols, roots, idx = groups[0][1][0]
    forged = cols[0].a.copy()
    forged[7] = (int(forged[7]) + 1) % 0xFFFFFFFF00000001      # row 7 is no longer a table row
    groups[0][1][0] = ([_Arr(forged), cols[1]], roots, idx)
    with pytest.raises(ValueError, match="witness not in table"):
        zk.p3.prove_super(OracleLookupEngine(orc), zk.Transcript("x"), [_Arr(t) for t in tcols], table_id(tcols), groups, 1)
    bad_idx = idx.a.copy()
    bad_idx[0] = 1 << 4
    groups[0][1][0] = (cols, roots, _Arr(bad_idx))
    with pytest.raises(IndexError):
        zk.p3.prove_super(OracleLookupEngine(orc), zk.Transcript("x"), [_Arr(t) for t in tcols], table_id(tcols), groups, 1)
