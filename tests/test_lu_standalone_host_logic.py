"""The standalone lookup (p3lu::prove_v, non-zk, per-instance openings) host logic on CPU: byte-identical
to the reference's own host prover and accepted by its verifier; tampered proofs and rows outside the
table are rejected."""
import numpy as np
import pytest

from irs_helpers import OracleStandaloneLuEngine, ref_lu_prove_v, ref_lu_verify_v
from lu_helpers import _Arr, make_lookup


@pytest.mark.parametrize("m,n,committed", [(4, 5, [1, 1]), (6, 4, [1, 1]), (5, 7, [1, 0]), (3, 3, [0, 1])])
def test_lu_prove_matches_reference_prover_and_verifier(orc, ref, zk, m, n, committed):
    R, Q = 1, 24
    tcols, subs = make_lookup(orc, m, [(n, 1)], 40 + m + n)
    cols, idx = subs[0][1][0]
    eng = OracleStandaloneLuEngine(orc)
    W = [(_Arr(c), eng.commit_gpu_rootonly(_Arr(c), R) if k else None) for c, k in zip(cols, committed)]
    tr = zk.Transcript("lu-standalone")
    pf, rA = zk.p3.lu_prove(eng, tr, W, _Arr(idx), zk.p3.make_table(tcols), R, Q, "lut")
    rpf, rst, rroots, rrA = ref_lu_prove_v(ref, zk.Transcript("lu-standalone").state, tcols, cols, committed, idx, R, Q, "lut", 0)
    assert rpf == pf and rst == tr.state and (rrA == np.asarray(rA, dtype=np.uint64)).all()
    roots = [w[1] if w[1] is not None else b"\0" * 32 for w in W]
    ok, st, vrA, yv = ref_lu_verify_v(ref, zk.Transcript("lu-standalone").state, tcols, roots, committed, R, Q, "lut", pf)
    assert ok and st == tr.state and (vrA[:n] == np.asarray(rA, dtype=np.uint64)).all()
    for k, (c, com) in enumerate(zip(cols, committed)):      # virtual columns: the caller binds y_virt
        if not com:
            assert int(yv[0]) == orc.mle_eval(c, np.asarray(rA, dtype=np.uint64))
    for off in (13, 12 + 96 + 3, len(pf) // 2, len(pf) - 5):
        bad = bytearray(pf)
        bad[off] ^= 1
        assert not ref_lu_verify_v(ref, zk.Transcript("lu-standalone").state, tcols, roots, committed, R, Q, "lut", bytes(bad))[0]


def test_lu_prove_rejects_row_outside_table(orc, zk):
    tcols, subs = make_lookup(orc, 4, [(5, 1)], 3)
    cols, idx = subs[0][1][0]
    eng = OracleStandaloneLuEngine(orc)
    forged = cols[0].copy()
    forged[3] = (int(forged[3]) + 1) % 0xFFFFFFFF00000001
    W = [(_Arr(forged), eng.commit_gpu_rootonly(_Arr(forged), 1)), (_Arr(cols[1]), eng.commit_gpu_rootonly(_Arr(cols[1]), 1))]
    with pytest.raises(ValueError, match="witness not in table"):
        zk.p3.lu_prove(eng, zk.Transcript("x"), W, _Arr(idx), zk.p3.make_table(tcols), 1, 24, "lut")
