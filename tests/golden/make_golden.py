"""Generate tests/golden/p3_golden.json from the UNMODIFIED reference.

Run in a checkout that has the reference tree (oracle/Makefile `ref` target builds
oracle/_ref/libp3ref.so from it):

    make -C oracle ref && python tests/golden/make_golden.py

Inputs come from the LCG the reference's own selftests use
(zkllm-src/p3_basefold_selftest.cu:12-13) with the seeds recorded in the file, so
the tests can regenerate every input without the reference.  Outputs are the
reference's host code paths: field ops, SHA-256 / transcript, eq / Lagrange
helpers, Horner RS encode, host Merkle, fold, Basefold prove_eval, GKR prove,
and the host sumcheck loops (p3lu::sc_prove, p3hwl::sc5_prove).
Large outputs are stored as SHA-256 digests of their little-endian bytes.
"""
import hashlib
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
from oracle import GL_P, Oracle, Reference  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "p3_golden.json")


def dig(a):
    if isinstance(a, np.ndarray):
        a = np.ascontiguousarray(a).tobytes()
    return hashlib.sha256(bytes(a)).hexdigest()


def main():
    ref, orc = Reference(), Oracle()   # the oracle is used ONLY for its LCG input generator
    g = {"generator": "tests/golden/make_golden.py", "source": "reference host paths via oracle/_ref"}
    seed = 0xBEEF1234

    def lcg(n, s):
        return orc.lcg(n, s)

    # ---- field ----
    edge = [0, 1, 2, GL_P - 1, GL_P - 2, 0xFFFFFFFF, 0x100000000, 0xFFFFFFFF00000000, 0xFFFFFFFE00000001]
    vals, _ = lcg(40, seed)
    vals = edge + [int(x) for x in vals]
    fld = []
    for i, a in enumerate(vals):
        b = vals[(i * 7 + 3) % len(vals)]
        fld.append([a, b, ref.gl_add(a, b), ref.gl_sub(a, b), ref.gl_mul(a, b),
                    ref.gl_inv(a) if a else 0])
    g["field"] = fld
    g["roots_of_unity"] = [ref.gl_root_of_unity(l) for l in range(1, 33)]

    # ---- sha / transcript ----
    msgs = [bytes((i * 37 + j) & 0xFF for j in range(n)) for i, n in enumerate([0, 1, 8, 55, 56, 64, 119, 200])]
    g["sha256"] = [[m.hex(), ref.sha256(m).hex()] for m in msgs]
    blk = bytes(range(64))
    g["compress64"] = [blk.hex(), ref.compress64(blk).hex()]
    st = ref.tr_init("p3-golden")
    trace = [st.hex()]
    for label, n in [("z", 24), ("y", 8), ("root", 32), ("sc", 24), ("imm-sc", 40), ("final", 16)]:
        data = bytes((len(label) * 11 + j) & 0xFF for j in range(n))
        st = ref.tr_absorb(st, label, data)
        st, a = ref.tr_chal(st)
        st, ix = ref.tr_idx(st, 1 << 21)
        trace.append([label, n, st.hex(), a, ix])
    g["transcript"] = trace

    # ---- multilinear helpers ----
    z, s1 = lcg(9, seed + 1)
    c, s1 = lcg(512, s1)
    eq = ref.build_eq(z)
    g["eq"] = {"seed": seed + 1, "v": 9, "eq_digest": dig(eq), "eval_h": ref.eval_h(c, eq)}
    t, _ = lcg(6, seed + 2)
    t = [int(x) for x in t]
    g["lagrange"] = {"seed": seed + 2, "quad": ref.quad_eval(*t[:4]), "cubic": ref.cubic_eval(*t[:5]),
                     "quartic": ref.quartic_eval(t[:5], t[5])}

    # ---- encode / merkle / fold ----
    enc = []
    for v, R in [(3, 1), (6, 2), (8, 1)]:
        cc, _ = lcg(1 << v, seed + 10 + v)
        cw = ref.rs_encode_horner(cc, R)
        w = ref.gl_root_of_unity(v + R)
        beta = int(cc[0])
        enc.append({"seed": seed + 10 + v, "v": v, "R": R, "cw_digest": dig(cw),
                    "root": ref.merkle_root(cw).hex(), "tree_digest": dig(ref.merkle_build(cw)),
                    "fold_mle_digest": dig(ref.fold(cw, w, beta, True)),
                    "fold_fri_digest": dig(ref.fold(cw, w, beta, False))})
    g["encode"] = enc

    # ---- Basefold opening (same shapes as zkllm-src/p3_basefold_selftest.cu:36-44) ----
    bf = []
    for v, R, Q in [(4, 1, 32), (6, 2, 32), (8, 1, 32), (10, 1, 24)]:
        s = seed + 100 + v
        cc, s2 = lcg(1 << v, s)
        zz, _ = lcg(v, s2)
        cw = ref.rs_encode_horner(cc, R)
        y = ref.eval_h(cc, ref.build_eq(zz))
        pf = ref.bf_prove_eval(cc, zz, y, R, Q, cw)
        assert ref.bf_verify_eval(pf)
        bf.append({"seed": s, "v": v, "R": R, "Q": Q, "y": y, "proof_digest": dig(pf), "proof_len": len(pf),
                   "root0": pf[12:44].hex(), "msg0": [int(x) for x in np.frombuffer(pf[12 + v * 32:12 + v * 32 + 24], dtype=np.uint64)]})
    g["basefold"] = bf

    # ---- GKR ----
    gk = []
    for L, cl in [(1, True), (3, True), (6, False), (10, True)]:
        s = seed + 200 + L
        p, s2 = lcg(1 << L, s)
        q, _ = lcg(1 << L, s2)
        st0 = ref.tr_init("gkr-golden")
        st1, pf, rfin, cpq = ref.gkr_prove(st0, "lug-gA", p, q, cl)
        gk.append({"seed": s, "L": L, "combine_last": cl, "state": st1.hex(), "proof_digest": dig(pf),
                   "rfin": [int(x) for x in rfin], "cpq": list(cpq) if cl else None})
    g["gkr"] = gk

    # ---- host sumcheck loops ----
    sc = []
    n = 9
    s = seed + 300
    cols = []
    for _ in range(4):
        a, s = lcg(1 << n, s)
        cols.append(a)
    lam, beta = int(cols[0][5]), int(cols[1][7])
    st0 = ref.tr_init("sc-golden")
    st1, m, r = ref.lu_sc_prove(st0, "lu-sc", cols[0], cols[1], cols[2], cols[3], lam, beta)
    sc.append({"kind": "logup", "seed": seed + 300, "logn": n, "nt": 4, "par": [lam, beta], "tag": "lu-sc",
               "state": st1.hex(), "msgs_digest": dig(m), "chals": [int(x) for x in r]})
    for f, nc, tag in [(0, 2, "hw-sc"), (1, 3, "imm-sc")]:
        s = seed + 310 + f
        cols = []
        for _ in range(nc):
            a, s = lcg(1 << 13, s)
            cols.append(a)
        st1, m, r = ref.sc5_prove(st0, tag, f, cols)
        sc.append({"kind": "prod%d" % nc, "seed": seed + 310 + f, "logn": 13, "nt": 5, "par": [], "tag": tag,
                   "state": st1.hex(), "msgs_digest": dig(m), "chals": [int(x) for x in r]})
    g["sumcheck"] = sc

    # ---- logUp primitives ----
    A, s = lcg(70000, seed + 400)
    beta = int(A[3])
    g["logup"] = {"seed": seed + 400, "n": 70000, "beta": beta, "inv_digest": dig(ref.inv_all_add(A, beta)),
                  "combine_digest": dig(ref.combine([A, A[::-1].copy()], beta))}

    # ---- batched opening: the reference's prover needs a GPU, its verifier does not.  The vectors
    # are the restatement's proofs, recorded only after the REFERENCE verifier accepted them and
    # rejected a tampered copy (the accepted transcript state is recorded too).
    bo = []
    for v, R, Q, ncols, T, k in [(3, 1, 24, 2, 2, 3), (6, 2, 24, 5, 3, 9), (8, 1, 32, 4, 4, 7)]:
        s = seed + 500 + v
        cols = []
        for _ in range(ncols):
            a, s = lcg(1 << v, s)
            cols.append(a)
        pts, s = lcg(T * v, s)
        pts = pts.reshape(T, v)
        ent_col = [(3 * j + 1) % ncols for j in range(k)]
        zid = [(5 * j + 2) % T for j in range(k)]
        roots_c = [ref.merkle_root(ref.rs_encode_horner(c, R)) for c in cols]
        roots = [roots_c[c] for c in ent_col]
        y = [ref.eval_h(cols[c], ref.build_eq(pts[t])) for c, t in zip(ent_col, zid)]
        st0 = ref.tr_init("bo-golden")
        pf, st1 = orc.bo_prove_class(st0, pts, [cols[c] for c in ent_col], roots, zid, R, Q, "tf-bo0")
        ok, st2 = ref.bo_verify_class(st0, pts, roots, zid, y, R, Q, "tf-bo0", pf)
        assert ok and st2 == st1
        bad = bytearray(pf); bad[20] ^= 1
        assert not ref.bo_verify_class(st0, pts, roots, zid, y, R, Q, "tf-bo0", bytes(bad))[0]
        bo.append({"seed": seed + 500 + v, "v": v, "R": R, "Q": Q, "ncols": ncols, "T": T, "k": k,
                   "ent_col": ent_col, "zid": zid, "y": y, "state": st1.hex(), "proof_digest": dig(pf),
                   "proof_len": len(pf), "accepted_by": "p3bo::verify_class (reference, host)"})
    g["batchopen"] = bo

    # ---- quartic zero-checks of the fp8 gadget: p3hwl::sc5_prove over the reference's own constraint
    # functions F_dp .. F_do (ids 6..11), random columns and coefficients
    from oracle import HW_SHAPE
    hw = []
    for f, (nc, nlam) in sorted(HW_SHAPE.items()):
        for logn in (1, 7):
            s = seed + 600 + 10 * f + logn
            cols = []
            for _ in range(nc):
                a, s = lcg(1 << logn, s)
                cols.append(a)
            lam, s = lcg(nlam, s)
            st0 = ref.tr_init("hw-golden")
            st1, m, r = ref.sc5_prove_lam(st0, "hwl-sc", f, cols, lam)
            hw.append({"functor": f, "nc": nc, "nlam": nlam, "seed": seed + 600 + 10 * f + logn, "logn": logn,
                       "tag": "hwl-sc", "state": st1.hex(), "msgs_digest": dig(m), "chals": [int(x) for x in r]})
    g["hawkeye_sumcheck"] = hw

    with open(OUT, "w") as f:
        json.dump(g, f, indent=1)
    print("wrote", OUT, os.path.getsize(OUT), "bytes")


if __name__ == "__main__":
    main()
