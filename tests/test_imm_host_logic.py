"""The integer matmul gadget's host logic (zk_hillclimb_b200.p3.imm_prove) on CPU over an
oracle-backed engine: the proof must be accepted by the reference's own verifier (p3imm::verify,
host-only) with the same final transcript state, and its messages must equal the reference
algorithm's (a cubic sumcheck over the three materialised broadcast columns)."""
import struct

import numpy as np
import pytest

from imm_helpers import OracleImmEngine, matmul_instance, ref_imm_verify
from lu_helpers import _Arr


@pytest.mark.parametrize("lj,lk,li", [(3, 2, 2), (4, 3, 1), (2, 4, 3), (5, 5, 4)])
def test_imm_prove_accepted_by_reference_verifier(orc, ref, zk, lj, lk, li):
    R, Q = 1, 24
    X, W, Y = matmul_instance(orc, lj, lk, li, 7 + lj)
    roots = [orc.merkle_root(orc.rs_encode(c, R)) for c in (X, W, Y)]
    tr = zk.Transcript("imm")
    pf = zk.p3.imm_prove(OracleImmEngine(orc), tr, (_Arr(X), roots[0]), (_Arr(W), roots[1]), (_Arr(Y), roots[2]),
                         lj, lk, li, R, Q)
    ok, st = ref_imm_verify(ref, zk.Transcript("imm").state, roots, lj, lk, li, R, Q, pf)
    assert ok and st == tr.state
    for off in (12, 12 + 40 * (lj + lk + li) + 3, len(pf) - 9):
        bad = bytearray(pf)
        bad[off] ^= 1
        assert not ref_imm_verify(ref, zk.Transcript("imm").state, roots, lj, lk, li, R, Q, bytes(bad))[0]


def test_factored_messages_equal_the_materialised_cubic_sumcheck(orc, zk):
    """The reference's algorithm, restated: build EQ, Xb, Wb over u = j | k<<lj | i<<(lj+lk)
    (zkllm-src/p3_int_gadgets.cuh:574-593) and run the 5-point cubic sumcheck on them."""
    from oracle import F_PROD3
    lj, lk, li, R, Q = 3, 3, 2, 1, 24
    X, W, Y = matmul_instance(orc, lj, lk, li, 5)
    roots = [orc.merkle_root(orc.rs_encode(c, R)) for c in (X, W, Y)]
    tr = zk.Transcript("imm")
    pf = zk.p3.imm_prove(OracleImmEngine(orc), tr, (_Arr(X), roots[0]), (_Arr(W), roots[1]), (_Arr(Y), roots[2]),
                         lj, lk, li, R, Q)
    lt = lj + lk + li
    mine = np.frombuffer(pf[12:12 + 40 * lt], dtype=np.uint64).reshape(lt, 5)
    # replay the transcript head to get z, then the reference's columns
    st = orc.tr_init("imm")
    st = orc.tr_absorb(st, "imm-dims", struct.pack("<III", lj, lk, li))
    for lab, r in zip(("imm-X", "imm-W", "imm-Y"), roots):
        st = orc.tr_absorb(st, lab, r)
    z = []
    for _ in range(lk + li):
        st, a = orc.tr_chal(st)
        z.append(a)
    st = orc.tr_absorb(st, "hwl-y", struct.pack("<Q", orc.mle_eval(Y, np.array(z, dtype=np.uint64))))
    eqv = orc.build_eq(np.array(z, dtype=np.uint64))
    u = np.arange(1 << lt)
    j, k, i = u & ((1 << lj) - 1), (u >> lj) & ((1 << lk) - 1), u >> (lj + lk)
    cols = [eqv[k | (i << lk)], X[j | (i << lj)], W[k | (j << lk)]]
    _, m, r, _ = orc.sumcheck(st, "imm-sc", F_PROD3, 5, cols)
    assert (m == mine).all()
