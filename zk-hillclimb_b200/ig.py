"""Integer-layer gadgets of the reference's p3 stack (zkllm-src/p3_int_gadgets.cuh), non-zk, as host logic over
the engine interface of p3.py: every gadget absorbs its operands' roots, commits its witness columns, defers
its lookups into the shared queue, proves one (or more) eq-weighted zero-checks with the programmable
summand engine, and records its opening claims in the shared ledger.  Standalone calls (no ledger given) end
with the lookup flush and the batched openings, as the reference's unit-test mode does.

Witness generation is exact integer arithmetic in numpy on the host (the reference replays its witnesses on
the host as well); columns are then handed to the engine.  Values are signed integers lifted into the field.
"""
import struct

import numpy as np

from .p3 import GL_P, Ledger, claimc, lu_flush, make_table, range_table, tail_prove

ABIT = 19
ABND = 1 << ABIT            # RS20 window [-2^19, 2^19)   (p3_int_gadgets.cuh:69-70)
NEG = lambda x: (GL_P - (x % GL_P)) % GL_P


def lift(a):
    """signed int64 array -> canonical field elements (p3ig::gsig)."""
    a = np.asarray(a, dtype=np.int64)
    return np.where(a < 0, a.astype(np.uint64) + np.uint64(GL_P), a.astype(np.uint64))


def sig(v):
    """canonical field elements -> signed int64 (p3ig::sig64)."""
    v = np.asarray(v, dtype=np.uint64)
    return np.where(v > np.uint64(GL_P >> 1), (v - np.uint64(GL_P)).astype(np.int64), v.astype(np.int64))


def build_tables(lib, d, btop):
    """p3ig::build_tables (zkllm-src/p3_int_gadgets.cuh:75-127).  ``lib``: the loaded C library (the function
    tables come from its host routine zkh_ig_table so that they match the reference's libm results)."""
    T = {"btop": btop, "R16": range_table(16, 0), "R14": range_table(14, 0), "RTOP": range_table(btop, 0),
         "RS16": range_table(16, -(1 << 15)), "RS20": range_table(20, -(1 << 19))}
    for name, kind, rows in (("EXPT", 0, 1 << 17), ("SILU", 1, 1 << 20), ("ISQ", 2, 1 << 16)):
        c0, c1 = np.zeros(rows, dtype=np.uint64), np.zeros(rows, dtype=np.uint64)
        if lib.zkh_ig_table(kind, d, c0.ctypes.data, c1.ctypes.data) != 0:
            raise RuntimeError("zkh_ig_table failed")
        T[name] = make_table([c0, c1])
    er = [min(e, 17) for e in range(32)]                               # EXP4: (4^e, 2^e, floor(2^e / 2)), e capped at 17
    T["EXP4"] = make_table([np.array([1 << (2 * e) for e in er], dtype=np.uint64), np.array([1 << e for e in er], dtype=np.uint64),
                            np.array([(1 << (e - 1)) if e else 0 for e in er], dtype=np.uint64)])
    return T


class Ctx:
    """Shared proving context of composed gadgets (p3lu::XCtx): the opening ledger and the deferred lookups."""

    def __init__(self):
        self.ledger, self.luq = Ledger(), []

    def defer(self, W, idx, tab):
        self.luq.append({"W": W, "idx": idx, "tab": tab})


def _tail(engine, tr, ctx, R, Q, tag):
    """p3ig::tail_prove (zkllm-src/p3_int_gadgets.cuh:186-193): lookup flush, then one batched opening per class."""
    lug = lu_flush(engine, tr, ctx.luq, ctx.ledger, R)
    batches = tail_prove(engine, tr, ctx.ledger, R, Q, tag)
    blob = lambda b: struct.pack("<I", len(b)) + b
    return struct.pack("<I", len(lug)) + b"".join(blob(b) for b in lug) + struct.pack("<I", len(batches)) + b"".join(blob(b) for b in batches)


_EMPTY_TAIL = struct.pack("<II", 0, 0)


def _zerocheck(engine, tr, tag, le, cols, terms, konst):
    """zE <- le challenges; sumcheck of eq(zE, .) * (konst + terms) over `cols`; returns (rE, messages)."""
    zE = np.array([tr.chal() for _ in range(le)], dtype=np.uint64)
    E = engine.build_eq_gpu(zE)
    rE, m, _ = engine.sc_prove_zc(tr, tag, [E] + cols, terms, konst)
    return [int(x) for x in rE], np.ascontiguousarray(m, dtype=np.uint64).tobytes()


# ---------------------------------------------------------------------------------- residual add (p3iadd)
def iadd_witness(a, b):
    """p3iadd::gen_witness (p3_int_gadgets.cuh:681-699): out = a + b, checked against the RS20 window."""
    o = sig(a) + sig(b)
    if ((o < -ABND) | (o >= ABND)).any():
        raise ValueError("iadd: out of range")
    return lift(o), (o + ABND).astype(np.uint32)


def iadd_prove(engine, tr, T, A, B, OUT, idxO, le, R, Q, ctx=None):
    """p3iadd::prove (p3_int_gadgets.cuh:712-737).  A, B, OUT: (column, root); idxO: RS20 row of every output.
    Proof: u32 le | messages le*40 | yA yB yO | tail."""
    own = ctx is None
    ctx = ctx or Ctx()
    tr.absorb("iad-dims", struct.pack("<I", le))
    tr.absorb("iad-A", A[1])
    tr.absorb("iad-B", B[1])
    tr.absorb("iad-O", OUT[1])
    ctx.defer([OUT], idxO, T["RS20"])
    rE, msgs = _zerocheck(engine, tr, "iad-sc", le, [A[0], B[0], OUT[0]], [(1, (1,)), (1, (2,)), (NEG(1), (3,))], 0)
    ys = [claimc(engine, tr, ctx.ledger, c[0], c[1], rE) for c in (A, B, OUT)]
    out = struct.pack("<I", le) + msgs + struct.pack("<QQQ", *ys)
    return out + (_tail(engine, tr, ctx, R, Q, "iad-bo") if own else _EMPTY_TAIL)


# ---------------------------------------------------------------------------------- SwiGLU product (p3iswg)
def iswg_witness(g, u, T):
    """p3iswg::gen_witness (p3_int_gadgets.cuh:1755-1781): sil = SILU[g], mo = round(sil*u / 2^16) with the
    remainder; returns (sil, rem, mo, idxG, idxR, idxM)."""
    gv, uv = sig(g), sig(u)
    if ((gv < -ABND) | (gv >= ABND)).any():
        raise ValueError("iswg: G out of range")
    sil = sig(T["SILU"]["cols"][1][gv + ABND])
    m64 = sil * uv
    mo = (m64 + (1 << 15)) >> 16
    rem = (m64 + (1 << 15)) - (mo << 16)
    if ((mo < -ABND) | (mo >= ABND)).any():
        raise ValueError("iswg: M out of range")
    return (lift(sil), rem.astype(np.uint64), lift(mo), (gv + ABND).astype(np.uint32), rem.astype(np.uint32),
            (mo + ABND).astype(np.uint32))


def iswg_prove(engine, tr, T, G, U, MO, wit, le, R, Q, ctx=None):
    """p3iswg::prove (p3_int_gadgets.cuh:1795-1832).  G, U, MO: (column, root); wit = (sil, rem, idxG, idxR, idxM)
    as engine columns / index arrays.  Proof: u32 le | rSIL rREM | messages | ySIL yU yM yR | tail."""
    own = ctx is None
    ctx = ctx or Ctx()
    sil, rem, idxG, idxR, idxM = wit
    tr.absorb("isw-dims", struct.pack("<I", le))
    tr.absorb("isw-G", G[1])
    tr.absorb("isw-U", U[1])
    tr.absorb("isw-M", MO[1])
    rS, rR = engine.commit_gpu_rootonly(sil, R), engine.commit_gpu_rootonly(rem, R)
    tr.absorb("isw-s", rS)
    tr.absorb("isw-r", rR)
    ctx.defer([G, (sil, rS)], idxG, T["SILU"])
    ctx.defer([(rem, rR)], idxR, T["R16"])
    ctx.defer([MO], idxM, T["RS20"])
    rE, msgs = _zerocheck(engine, tr, "isw-sc", le, [sil, U[0], MO[0], rem],
                          [(1, (1, 2)), (NEG(65536), (3,)), (NEG(1), (4,))], 32768)
    ys = [claimc(engine, tr, ctx.ledger, c, r, rE) for c, r in ((sil, rS), U, MO, (rem, rR))]
    out = struct.pack("<I", le) + rS + rR + msgs + struct.pack("<QQQQ", *ys)
    return out + (_tail(engine, tr, ctx, R, Q, "isw-bo") if own else _EMPTY_TAIL)


# ---------------------------------------------------------------------------------- RoPE (p3irope)
def rope_pub_cols(ct, st, lseq, ldh, ld, le):
    """p3irope::cs_at / pub_col (p3_int_gadgets.cuh:1199-1222): the public cos / signed-sin broadcasts over the
    element domain u = j | (t << ld); ct, st: int arrays [2^lseq][2^(ldh-1)] at scale 2^14."""
    u = np.arange(1 << le, dtype=np.int64)
    j, t = u & ((1 << ld) - 1), u >> ld
    s = t & ((1 << lseq) - 1)
    jj = j & ((1 << ldh) - 1)
    hb = (jj >> (ldh - 1)) & 1
    ti = s * (1 << (ldh - 1)) + (jj & ((1 << (ldh - 1)) - 1))
    ct, st = np.asarray(ct, dtype=np.int64).reshape(-1), np.asarray(st, dtype=np.int64).reshape(-1)
    return ct[ti], np.where(hb == 1, st[ti], -st[ti])


def irope_witness(q, ct, st, lseq, ldh, lT, ld):
    """p3irope::gen_witness (p3_int_gadgets.cuh:1241-1267): y = round((q*C + q_rot*S2) / 2^14) with remainder;
    returns (y, rem, idxR, idxY, C, S2) with C, S2 the public columns as signed ints."""
    le, fb = lT + ld, ldh - 1
    C_, S2 = rope_pub_cols(ct, st, lseq, ldh, ld, le)
    qv = sig(q)
    qf = qv[np.arange(1 << le) ^ (1 << fb)]
    y64 = qv * C_ + qf * S2
    Y = (y64 + (1 << 13)) >> 14
    rem = (y64 + (1 << 13)) - (Y << 14)
    if ((Y < -ABND) | (Y >= ABND)).any():
        raise ValueError("irope: y out of range")
    return lift(Y), rem.astype(np.uint64), (rem & 0x3FFF).astype(np.uint32), (Y + ABND).astype(np.uint32), C_, S2


def irope_prove(engine, tr, T, pub, Qc, Y, wit, lT, ld, R, Q, ctx=None):
    """p3irope::prove (p3_int_gadgets.cuh:1279-1322).  pub = (C, S2) engine columns of the public broadcasts and
    ldh; Qc, Y: (column, root); wit = (rem, idxR, idxY).  Proof: u32 lT, ld, fb | rREM | messages | yQ yQx yY yR | tail."""
    own = ctx is None
    ctx = ctx or Ctx()
    Ccol, Scol, ldh = pub
    rem, idxR, idxY = wit
    le, fb = lT + ld, ldh - 1
    tr.absorb("irp-dims", struct.pack("<III", lT, ld, fb))
    tr.absorb("irp-Q", Qc[1])
    tr.absorb("irp-Y", Y[1])
    rR = engine.commit_gpu_rootonly(rem, R)
    tr.absorb("irp-r", rR)
    ctx.defer([(rem, rR)], idxR, T["R14"])
    ctx.defer([Y], idxY, T["RS20"])
    Qx = engine.flip_bit(Qc[0], fb)
    rE, msgs = _zerocheck(engine, tr, "irp-sc", le, [Qc[0], Qx, Y[0], rem, Ccol, Scol],
                          [(1, (1, 5)), (1, (2, 6)), (NEG(16384), (3,)), (NEG(1), (4,))], 8192)
    rf = list(rE)
    rf[fb] = (1 - rf[fb]) % GL_P
    yQ = claimc(engine, tr, ctx.ledger, Qc[0], Qc[1], rE)
    yQx = claimc(engine, tr, ctx.ledger, Qc[0], Qc[1], rf)
    yY = claimc(engine, tr, ctx.ledger, Y[0], Y[1], rE)
    yR = claimc(engine, tr, ctx.ledger, rem, rR, rE)
    out = struct.pack("<III", lT, ld, fb) + rR + msgs + struct.pack("<QQQQ", yQ, yQx, yY, yR)
    return out + (_tail(engine, tr, ctx, R, Q, "irp-bo") if own else _EMPTY_TAIL)


# ---------------------------------------------------------------------------------- RMSNorm (p3irms)
CEPS = 1 << 14
(B_M, B_MM, B_MS, B_P4, B_P2, B_H2, B_RP, B_L40, B_L41, B_L42, B_D40, B_D41, B_D42, B_R, B_L20, B_D20, B_LR0, B_LR1) = range(18)
NDB, NDE = 18, 3          # per-row columns; per-element witness columns W, remW, remY


def rshu(x, sf):
    return (x + (1 << (sf - 1))) >> sf


def irms_witness(x, g, T, lT, ld):
    """p3irms::gen_witness (p3_int_gadgets.cuh:823-903).  x: 2^(lT+ld) activations, g: 2^ld gains (field elements).
    Returns dict with db (18 row columns), de (W, remW, remY), y and the lookup indices."""
    B, d = 1 << lT, 1 << ld
    xv = sig(x).reshape(B, d)
    gv = sig(g)
    M = CEPS + (xv * xv).sum(axis=1)
    e = np.zeros(B, dtype=np.int64)
    while True:
        big = (M >> (2 * e)) >= (1 << 16)
        if not big.any():
            break
        e += big
    m = M >> (2 * e)
    p4, p2 = np.int64(1) << (2 * e), np.int64(1) << e
    h2 = np.where(e > 0, np.int64(1) << np.maximum(e - 1, 0), 0)
    r4 = M - m * p4
    d4 = p4 - 1 - r4
    RP = T["ISQ"]["cols"][1][m].astype(np.int64)
    Rr = (RP + h2) >> e
    r2 = RP + h2 - (Rr << e)
    d2 = p2 - 1 - r2
    db = [None] * NDB
    db[B_M], db[B_MM], db[B_MS] = M, m, m - (1 << 14)
    db[B_P4], db[B_P2], db[B_H2], db[B_RP] = p4, p2, h2, RP
    db[B_L40], db[B_L41], db[B_L42] = r4 & 0xFFFF, (r4 >> 16) & 0xFFFF, r4 >> 32
    db[B_D40], db[B_D41], db[B_D42] = d4 & 0xFFFF, (d4 >> 16) & 0xFFFF, d4 >> 32
    db[B_R], db[B_L20], db[B_D20] = Rr, r2, d2
    db[B_LR0], db[B_LR1] = Rr & 0xFFFF, Rr >> 16
    w64 = Rr[:, None] * gv[None, :]
    Wv = rshu(w64, 16)
    remW = (w64 + (1 << 15)) - (Wv << 16)
    if ((Wv < -ABND) | (Wv >= ABND)).any():
        raise ValueError("irms: W out of range")
    y64 = Wv * xv
    Yv = rshu(y64, 16)
    remY = (y64 + (1 << 15)) - (Yv << 16)
    if ((Yv < -ABND) | (Yv >= ABND)).any():
        raise ValueError("irms: Y out of range")
    u32 = lambda a: np.asarray(a).reshape(-1).astype(np.uint32)
    idxL = [u32(db[c] & 0xFFFF) if c in (B_L20, B_D20) else u32(db[c]) for c in
            (B_L40, B_L41, B_L42, B_D40, B_D41, B_D42, B_L20, B_D20, B_LR0)]
    return {"db": [lift(c) for c in db], "de": [lift(Wv.reshape(-1)), lift(remW.reshape(-1)), lift(remY.reshape(-1))],
            "y": lift(Yv.reshape(-1)), "idxE4": u32(e), "idxM16": u32(m), "idxMS": u32(m - (1 << 14)), "idxISQ": u32(m),
            "idxL": idxL, "idxLR1": u32(Rr >> 16), "idxRW": u32(remW), "idxW": u32(Wv + ABND), "idxRY": u32(remY),
            "idxY": u32(Yv + ABND)}


def _sumcheck(engine, tr, tag, cols, terms, konst):
    r, m, _ = engine.sc_prove_zc(tr, tag, cols, terms, konst)
    return [int(x) for x in r], np.ascontiguousarray(m, dtype=np.uint64).tobytes()


def irms_terms_rows(lamB):
    """The six per-row constraints of p3irms (p3_int_gadgets.cuh:984-1003) as zero-check terms over [E, 18 row columns],
    batched with powers of lamB.  Returns (terms, constant)."""
    lam = [pow(lamB, j, GL_P) for j in range(6)]
    c = lambda k: 1 + k                        # column index of row column k (column 0 is the eq weight)
    n = lambda x: NEG(x)
    terms = [
        # r0 = M - (MM*P4 + r4),  r4 = L40 + 2^16 L41 + 2^32 L42
        (lam[0], (c(B_M),)), (n(lam[0]), (c(B_MM), c(B_P4))), (n(lam[0]), (c(B_L40),)), (n(lam[0] << 16), (c(B_L41),)),
        (n(lam[0] << 32), (c(B_L42),)),
        # r1 = P4 - 1 - r4 - d4
        (lam[1], (c(B_P4),)), (n(lam[1]), (c(B_L40),)), (n(lam[1] << 16), (c(B_L41),)), (n(lam[1] << 32), (c(B_L42),)),
        (n(lam[1]), (c(B_D40),)), (n(lam[1] << 16), (c(B_D41),)), (n(lam[1] << 32), (c(B_D42),)),
        # r2 = R*P2 + L20 - RP - H2
        (lam[2], (c(B_R), c(B_P2))), (lam[2], (c(B_L20),)), (n(lam[2]), (c(B_RP),)), (n(lam[2]), (c(B_H2),)),
        # r3 = P2 - 1 - L20 - D20
        (lam[3], (c(B_P2),)), (n(lam[3]), (c(B_L20),)), (n(lam[3]), (c(B_D20),)),
        # r4' = R - LR0 - 2^16 LR1
        (lam[4], (c(B_R),)), (n(lam[4]), (c(B_LR0),)), (n(lam[4] << 16), (c(B_LR1),)),
        # r5 = MS + 2^14 - MM
        (lam[5], (c(B_MS),)), (n(lam[5]), (c(B_MM),)),
    ]
    konstB = (-lam[1] - lam[3] + lam[5] * 16384) % GL_P
    return terms, konstB


def irms_terms_elements(lamE):
    """The two per-element constraints (p3_int_gadgets.cuh:1028-1035) over columns 0 E, 1 X, 2 Y, 3 W, 4 RW, 5 RY, 6 Rb, 7 Gb."""
    n = lambda x: NEG(x)
    terms = [(1, (6, 7)), (n(65536), (3,)), (n(1), (4,)), (lamE, (3, 1)), (n(lamE * 65536), (2,)), (n(lamE), (5,))]
    return terms, (32768 + lamE * 32768) % GL_P


def irms_prove(engine, tr, T, X, G, Y, wit, lT, ld, R, Q, ctx=None):
    """p3irms::prove (p3_int_gadgets.cuh:922-1047).  X, Y: (column, root) over 2^(lT+ld) elements, G: gains over 2^ld;
    wit: irms_witness output with db/de as engine columns and index arrays.
    Proof: u32 lT, ld | 18 row roots | 3 element roots | yM yMX | mS | mB yB[18] | mE yE[3] yEX yEY yER yEG | tail."""
    own = ctx is None
    ctx = ctx or Ctx()
    le = lT + ld
    tr.absorb("irm-dims", struct.pack("<II", lT, ld))
    tr.absorb("irm-X", X[1])
    tr.absorb("irm-G", G[1])
    tr.absorb("irm-Y", Y[1])
    CB, CE = [], []
    for c in wit["db"]:
        root = engine.commit_gpu_rootonly(c, R)
        CB.append((c, root))
        tr.absorb("irm-cb", root)
    for c in wit["de"]:
        root = engine.commit_gpu_rootonly(c, R)
        CE.append((c, root))
        tr.absorb("irm-ce", root)
    ctx.defer([CB[B_P4], CB[B_P2], CB[B_H2]], wit["idxE4"], T["EXP4"])
    ctx.defer([CB[B_MM]], wit["idxM16"], T["R16"])
    ctx.defer([CB[B_MS]], wit["idxMS"], T["R16"])
    ctx.defer([CB[B_MM], CB[B_RP]], wit["idxISQ"], T["ISQ"])
    for l, c in enumerate((B_L40, B_L41, B_L42, B_D40, B_D41, B_D42, B_L20, B_D20, B_LR0)):
        ctx.defer([CB[c]], wit["idxL"][l], T["R16"])
    ctx.defer([CB[B_LR1]], wit["idxLR1"], T["R16"])
    ctx.defer([CE[1]], wit["idxRW"], T["R16"])
    ctx.defer([CE[0]], wit["idxW"], T["RS20"])
    ctx.defer([CE[2]], wit["idxRY"], T["R16"])
    ctx.defer([Y], wit["idxY"], T["RS20"])
    # M row-sum binding: sum_j X^2 = M - CEPS, weighted by eq(zb, row)
    zb = [tr.chal() for _ in range(lT)]
    yM = claimc(engine, tr, ctx.ledger, CB[B_M][0], CB[B_M][1], zb)
    EQb = engine.bcast_rows(engine.build_eq_gpu(np.array(zb, dtype=np.uint64)), ld)
    rS, mS = _sumcheck(engine, tr, "irm-scS", [EQb, X[0]], [(1, (1, 1))], 0)
    yMX = claimc(engine, tr, ctx.ledger, X[0], X[1], rS)
    # per-row zero-check
    zB = np.array([tr.chal() for _ in range(lT)], dtype=np.uint64)
    lamB = tr.chal()
    terms, konstB = irms_terms_rows(lamB)
    EB = engine.build_eq_gpu(zB)
    rB, mB = _sumcheck(engine, tr, "irm-scB", [EB] + [cb[0] for cb in CB], terms, konstB)
    yB = [claimc(engine, tr, ctx.ledger, cb[0], cb[1], rB) for cb in CB]
    # per-element zero-check: W = round(R*g / 2^16), Y = round(W*x / 2^16)
    zE = np.array([tr.chal() for _ in range(le)], dtype=np.uint64)
    lamE = tr.chal()
    Rb = engine.bcast_rows(CB[B_R][0], ld)
    Gb = engine.bcast_cols(G[0], lT)
    termsE, konstE = irms_terms_elements(lamE)
    rE, mE = _sumcheck(engine, tr, "irm-scE", [engine.build_eq_gpu(zE), X[0], Y[0], CE[0][0], CE[1][0], CE[2][0], Rb, Gb],
                       termsE, konstE)
    yEX = claimc(engine, tr, ctx.ledger, X[0], X[1], rE)
    yEY = claimc(engine, tr, ctx.ledger, Y[0], Y[1], rE)
    yE = [claimc(engine, tr, ctx.ledger, ce[0], ce[1], rE) for ce in CE]
    yER = claimc(engine, tr, ctx.ledger, CB[B_R][0], CB[B_R][1], rE[ld:le])
    yEG = claimc(engine, tr, ctx.ledger, G[0], G[1], rE[:ld])
    out = struct.pack("<II", lT, ld) + b"".join(cb[1] for cb in CB) + b"".join(ce[1] for ce in CE)
    out += struct.pack("<QQ", yM, yMX) + mS + mB + struct.pack("<18Q", *yB) + mE + struct.pack("<3Q", *yE)
    out += struct.pack("<QQQQ", yEX, yEY, yER, yEG)
    return out + (_tail(engine, tr, ctx, R, Q, "irm-bo") if own else _EMPTY_TAIL)


# ---------------------------------------------------------------------------------- causal softmax (p3ismx)
X_SEL, X_DM, X_EE, X_L0, X_L1, X_L2, X_L3 = range(7)
NXE, NXB = 7, 2           # per-element witness columns; per-row columns MX, S


def ismx_witness(z, T, la, lseq):
    """p3ismx::gen_witness (p3_int_gadgets.cuh:1410-1477): causal row max, EXPT lookups, row sum S,
    P = round(E/S * 2^16) with the bracket remainders in 16-bit limbs.  z: 2^(la+2*lseq) scores."""
    seq, NR = 1 << lseq, 1 << (la + lseq)
    zv = sig(z).reshape(NR, seq)
    i = (np.arange(NR) & (seq - 1))[:, None]
    j = np.arange(seq)[None, :]
    causal = j <= i
    mx = np.where(causal, zv, np.iinfo(np.int64).min).max(axis=1)
    dm = np.where(causal, mx[:, None] - zv, 1 << 16)
    if ((dm < 0) | (dm >= (1 << 17))).any():
        raise ValueError("ismx: DM range")
    E = T["EXPT"]["cols"][1][dm].astype(np.int64)
    S = E.sum(axis=1)
    hit = causal & (dm == 0)
    first = hit & (np.cumsum(hit, axis=1) == 1)
    P = ((1 << 17) * E + S[:, None]) // (2 * S[:, None])
    r1 = (1 << 17) * E + S[:, None] - 2 * P * S[:, None]
    r2 = 2 * S[:, None] - 1 - r1
    flat = lambda a: np.ascontiguousarray(a).reshape(-1)
    xe = [first.astype(np.int64), dm, E, r1 & 0xFFFF, r1 >> 16, r2 & 0xFFFF, r2 >> 16]
    u32 = lambda a: flat(a).astype(np.uint32)
    return {"xe": [lift(flat(c)) for c in xe], "xb": [lift(mx), lift(S)], "p": lift(flat(P)), "idxDM": u32(dm),
            "idxL": [u32(r1 & 0xFFFF), u32(r1 >> 16), u32(r2 & 0xFFFF), u32(r2 >> 16)], "idxMX": (mx + (1 << 15)).astype(np.uint32)}


def causal_mask(la, lseq):
    """p3ismx::mask_col: 1 where key index j <= query index i, over u = j | (i << lseq) | (a << 2 lseq)."""
    u = np.arange(1 << (la + 2 * lseq), dtype=np.int64)
    seq = 1 << lseq
    return ((u & (seq - 1)) <= ((u >> lseq) & (seq - 1))).astype(np.uint64)


def ismx_terms(lamE):
    """The five per-element constraints of p3ismx (p3_int_gadgets.cuh:1604-1622) over columns 0 E, 1 Z, 2.. the seven element
    columns, then P, MX broadcast, S broadcast, causal mask; batched with powers of lamE.  Returns (terms, constant)."""
    lam = [pow(lamE, k, GL_P) for k in range(5)]
    n = NEG
    ce = lambda k: 2 + k
    Zc, Pc, MXb, Sb, MK = 1, 2 + NXE, 3 + NXE, 4 + NXE, 5 + NXE
    terms = [
        (lam[0], (ce(X_SEL), ce(X_SEL))), (n(lam[0]), (ce(X_SEL),)),                                   # SEL^2 - SEL
        (lam[1], (ce(X_SEL), ce(X_DM))),                                                               # SEL * DM
        (lam[2], (ce(X_DM),)), (n(lam[2]), (MK, MXb)), (lam[2], (MK, Zc)), (lam[2] * 65536, (MK,)),    # DM - MK(MX - Z) - (1-MK) 2^16
        (lam[3] * 131072, (ce(X_EE),)), (lam[3], (Sb,)), (n(2 * lam[3]), (Pc, Sb)), (n(lam[3]), (ce(X_L0),)),
        (n(lam[3] * 65536), (ce(X_L1),)),                                                              # 2^17 EE + S - 2 P S - r1
        (lam[4], (ce(X_L2),)), (lam[4] * 65536, (ce(X_L3),)), (lam[4], (ce(X_L0),)), (lam[4] * 65536, (ce(X_L1),)),
        (n(2 * lam[4]), (Sb,)),                                                                        # r2 + r1 + 1 - 2 S
    ]
    konst = (-lam[2] * 65536 + lam[4]) % GL_P
    return terms, konst


def ismx_prove(engine, tr, T, Z, P, wit, la, lseq, R, Q, ctx=None):
    """p3ismx::prove (p3_int_gadgets.cuh:1518-1643).  Z, P: (column, root) over 2^(la + 2 lseq); wit: ismx_witness
    output with xe/xb as engine columns and index arrays.
    Proof: u32 la, lseq | 7 element roots | 2 row roots | mSel ySel | ySrow mS ySE | mE yEZ yE[7] yEP yEMX yES | tail."""
    own = ctx is None
    ctx = ctx or Ctx()
    lr, le = la + lseq, la + 2 * lseq
    tr.absorb("ism-dims", struct.pack("<II", la, lseq))
    tr.absorb("ism-Z", Z[1])
    tr.absorb("ism-P", P[1])
    CE, CB = [], []
    for c in wit["xe"]:
        root = engine.commit_gpu_rootonly(c, R)
        CE.append((c, root))
        tr.absorb("ism-ce", root)
    for c in wit["xb"]:
        CB.append((c, engine.commit_gpu_rootonly(c, R)))
    for cb in CB:
        tr.absorb("ism-cb", cb[1])
    ctx.defer([CE[X_DM], CE[X_EE]], wit["idxDM"], T["EXPT"])
    for l in range(4):
        ctx.defer([CE[X_L0 + l]], wit["idxL"][l], T["R16"])
    ctx.defer([CB[0]], wit["idxMX"], T["RS16"])
    # SEL row sum: sum_j SEL = 1, weighted by eq(zb, row)
    zb = np.array([tr.chal() for _ in range(lr)], dtype=np.uint64)
    rS, mSel = _sumcheck(engine, tr, "ism-scsel", [engine.bcast_rows(engine.build_eq_gpu(zb), lseq), CE[X_SEL][0]], [(1, (1,))], 0)
    ySel = claimc(engine, tr, ctx.ledger, CE[X_SEL][0], CE[X_SEL][1], rS)
    # S row sum: sum_j EE = S
    zb = [tr.chal() for _ in range(lr)]
    ySrow = claimc(engine, tr, ctx.ledger, CB[1][0], CB[1][1], zb)
    rS2, mS = _sumcheck(engine, tr, "ism-scs", [engine.bcast_rows(engine.build_eq_gpu(np.array(zb, dtype=np.uint64)), lseq), CE[X_EE][0]],
                        [(1, (1,))], 0)
    ySE = claimc(engine, tr, ctx.ledger, CE[X_EE][0], CE[X_EE][1], rS2)
    # per-element zero-check
    zE = np.array([tr.chal() for _ in range(le)], dtype=np.uint64)
    lamE = tr.chal()
    terms, konst = ismx_terms(lamE)
    cols = [engine.build_eq_gpu(zE), Z[0]] + [c[0] for c in CE] + [P[0], engine.bcast_rows(CB[0][0], lseq),
                                                                   engine.bcast_rows(CB[1][0], lseq), engine.causal_mask(la, lseq)]
    rE, mE = _sumcheck(engine, tr, "ism-sce", cols, terms, konst)
    yEZ = claimc(engine, tr, ctx.ledger, Z[0], Z[1], rE)
    yE = [claimc(engine, tr, ctx.ledger, c[0], c[1], rE) for c in CE]
    yEP = claimc(engine, tr, ctx.ledger, P[0], P[1], rE)
    rb = rE[lseq:le]
    yEMX = claimc(engine, tr, ctx.ledger, CB[0][0], CB[0][1], rb)
    yES = claimc(engine, tr, ctx.ledger, CB[1][0], CB[1][1], rb)
    out = struct.pack("<II", la, lseq) + b"".join(c[1] for c in CE) + b"".join(c[1] for c in CB)
    out += mSel + struct.pack("<Q", ySel) + struct.pack("<Q", ySrow) + mS + struct.pack("<Q", ySE)
    out += mE + struct.pack("<Q", yEZ) + struct.pack("<7Q", *yE) + struct.pack("<QQQ", yEP, yEMX, yES)
    return out + (_tail(engine, tr, ctx, R, Q, "ism-bo") if own else _EMPTY_TAIL)


# ---------------------------------------------------------------------------------- decoder layer (p3itf)
from .p3 import S_A, S_C, S_I, S_J, imm_prove, irs_prove  # noqa: E402

W_Q, W_K, W_V, W_O, W_G, W_U, W_D = range(7)


class Config:
    """p3itf::Config (zkllm-src/p3_int_layer.cuh:41-62): all dimensions powers of two, nh*dh == d."""

    def __init__(self, seq, d, nh, dh, dff, batch=1):
        self.seq, self.d, self.nh, self.dh, self.dff, self.batch = seq, d, nh, dh, dff, batch
        lg = lambda x: int(x).bit_length() - 1
        self.lseq, self.ld, self.lnh, self.ldh, self.ldff, self.lbb = lg(seq), lg(d), lg(nh), lg(dh), lg(dff), lg(batch)
        if any((1 << l) != v for l, v in ((self.lseq, seq), (self.ld, d), (self.lnh, nh), (self.ldh, dh), (self.ldff, dff),
                                          (self.lbb, batch))) or nh * dh != d:
            raise ValueError("itf: config must be pow2 with nh*dh == d")
        self.lT, self.la = self.lseq + self.lbb, self.lnh + self.lbb
        self.A = batch * nh
        self.tsh = (self.ldh + 1) // 2              # power-of-two softmax temperature
        self.sfz = 24 + self.tsh                    # scores rescale shift
        self.btop = self.sfz - 16                   # width of the top-limb table

    def wshape(self, i):
        return (self.dff if i == W_D else self.d), (self.dff if i in (W_G, W_U) else self.d)


def _consts(bits, val):
    return [(S_C, (val >> t) & 1) for t in range(bits)]


def views_qk(c, h, b):
    """xview_qk / wview_qk / yview_qk (p3_int_layer.cuh:96-122): scores of head h, batch b, Y = RQ_h . RK_h^T."""
    a = b * c.nh + h
    xv = [(S_J, t) for t in range(c.ldh)] + _consts(c.lnh, h) + [(S_A, t) for t in range(c.lseq)] + _consts(c.lbb, b)
    yv = [(S_A, t) for t in range(c.lseq)] + [(S_I, t) for t in range(c.lseq)] + _consts(c.la, a)
    return xv, list(xv), yv


def views_pv(c, h, b):
    """xview_pv / wview_pv / yview_pv (p3_int_layer.cuh:124-148): attention output of head h, batch b."""
    a = b * c.nh + h
    xv = [(S_J, t) for t in range(c.lseq)] + [(S_A, t) for t in range(c.lseq)] + _consts(c.la, a)
    wv = [(S_A, t) for t in range(c.ldh)] + _consts(c.lnh, h) + [(S_J, t) for t in range(c.lseq)] + _consts(c.lbb, b)
    yv = [(S_A, t) for t in range(c.ldh)] + _consts(c.lnh, h) + [(S_I, t) for t in range(c.lseq)] + _consts(c.lbb, b)
    return xv, wv, yv


def _view_idx(view, n_first, n_second, first, second):
    """Element indices of a Y-style or operand-style view for all (second, first) index pairs."""
    f = np.arange(1 << n_first, dtype=np.int64)[None, :]
    s = np.arange(1 << n_second, dtype=np.int64)[:, None]
    idx = np.zeros((1 << n_second, 1 << n_first), dtype=np.int64)
    for t, (src, bit) in enumerate(view):
        b = ((f >> bit) & 1) if src == first else ((s >> bit) & 1) if src == second else (bit if src == S_C else 0)
        idx |= b << t
    return idx


def random_layer_inputs(c, seed, wscale=0.9):
    """Synthetic in-range layer inputs in the style of the reference's layer bench (zkllm-src/p3_int_layer_bench.cu:49-72):
    weights uniform within +-2^16*wscale/sqrt(fan-in), gains around 0.75*2^16, RoPE tables for theta = 10000 at scale
    2^14, activations uniform in +-2^16.  Returns (x0, weights dict)."""
    g = np.random.default_rng(seed)
    wb = max(2, int(round(65536.0 * wscale / np.sqrt(c.d))))
    wbd = max(2, int(round(65536.0 * wscale / np.sqrt(c.dff))))
    Wt = {"w": []}
    for i in range(7):
        K, N = c.wshape(i)
        b = wbd if i == W_D else wb
        Wt["w"].append(lift(g.integers(-(b - 1), b, K * N)))
    Wt["g1"] = lift(49152 + g.integers(-16383, 16384, c.d))
    Wt["g2"] = lift(49152 + g.integers(-16383, 16384, c.d))
    s_ = np.arange(c.seq)[:, None]
    j_ = np.arange(c.dh // 2)[None, :]
    ang = s_ * np.power(10000.0, -2.0 * j_ / c.dh)
    Wt["ct"] = np.rint(np.cos(ang) * 16384.0).astype(np.int32)
    Wt["st"] = np.rint(np.sin(ang) * 16384.0).astype(np.int32)
    x0 = lift(g.integers(-(1 << 16) + 1, 1 << 16, c.seq * c.batch * c.d))
    return x0, Wt


def rs20_idx(v):
    s = sig(v)
    if ((s < -ABND) | (s >= ABND)).any():
        raise ValueError("itf: value out of RS20")
    return (s + ABND).astype(np.uint32)


def irs_witness_host(acc, sf, rng):
    """p3irs::gen_witness in numpy (the layer's witness chain runs on the host): returns (y, limbs, limb indices, y indices)."""
    a = sig(acc)
    H = 1 << (sf - 1)
    y = (a + H) >> sf
    rem = (a + H) - (y << sf)
    win = (1 << 19) if rng == 1 else (1 << 15)
    if rng and ((y < -win) | (y >= win)).any():
        raise ValueError("irs: y out of range (data too large)")
    L = [(rem & 0xFFFF).astype(np.uint64)] + ([(rem >> 16).astype(np.uint64)] if sf > 16 else [])
    return lift(y), L, [l.astype(np.uint32) for l in L], ((y + win).astype(np.uint32) if rng else None)


def itf_build_witness(c, x0, Wt, T):
    """p3itf::build_witness (p3_int_layer.cuh:182-318): the layer computed by the gadget replays themselves.
    Wt = {"w": [7 weight grids K x N row-major], "g1", "g2", "ct", "st"} as field elements / int tables."""
    ld, lT, ldff, lseq, ldh, la = c.ld, c.lT, c.ldff, c.lseq, c.ldh, c.la
    le, lef, lez = ld + lT, ldff + lT, la + 2 * lseq
    w = {"x0": x0, "idxW": [rs20_idx(x) for x in Wt["w"]], "idxG1": rs20_idx(Wt["g1"]), "idxG2": rs20_idx(Wt["g2"]),
         "idxX0": rs20_idx(x0)}
    def mat(X, Wm, K, N):
        # Y[k | i << lk]; |x|, |w| < 2^19 and K <= 2^13 keep every partial sum below 2^53, so the float64 product is exact
        y = sig(X).reshape(-1, K).astype(np.float64) @ sig(Wm).reshape(K, N).astype(np.float64)
        return lift(np.rint(y).astype(np.int64).reshape(-1))
    w["rms1"] = irms_witness(x0, Wt["g1"], T, lT, ld)
    w["h1"] = w["rms1"]["y"]
    w["acc"] = [None] * 7
    for i in (W_Q, W_K, W_V):
        w["acc"][i] = mat(w["h1"], Wt["w"][i], c.d, c.d)
    w["rsq"], w["rsk"], w["rsv"] = (irs_witness_host(w["acc"][i], 16, 1) for i in (W_Q, W_K, W_V))
    w["yq"], w["yk"], w["yv"] = w["rsq"][0], w["rsk"][0], w["rsv"][0]
    w["rpq"] = irope_witness(w["yq"], Wt["ct"], Wt["st"], lseq, ldh, lT, ld)
    w["rpk"] = irope_witness(w["yk"], Wt["ct"], Wt["st"], lseq, ldh, lT, ld)
    w["rq"], w["rk"] = w["rpq"][0], w["rpk"][0]
    sc = np.zeros(1 << lez, dtype=np.int64)
    rq, rk = sig(w["rq"]), sig(w["rk"])
    for b in range(c.batch):
        for h in range(c.nh):
            xv, wv, yv = views_qk(c, h, b)
            Xd = rq[_view_idx(xv, ldh, lseq, S_J, S_A)]                    # [i][j]
            Wd = rk[_view_idx(wv, ldh, lseq, S_J, S_A)]                    # [k][j]
            sc[_view_idx(yv, lseq, lseq, S_A, S_I)] = Xd @ Wd.T            # [i][k]
    w["sc"] = lift(sc)
    w["rsz"] = irs_witness_host(w["sc"], c.sfz, 2)
    w["z"] = w["rsz"][0]
    w["smx"] = ismx_witness(w["z"], T, la, lseq)
    w["p"] = w["smx"]["p"]
    pva = np.zeros(1 << le, dtype=np.int64)
    pp, yv_ = sig(w["p"]), sig(w["yv"])
    for b in range(c.batch):
        for h in range(c.nh):
            xv, wv, yv = views_pv(c, h, b)
            Xd = pp[_view_idx(xv, lseq, lseq, S_J, S_A)]                   # [i][j]
            Wd = yv_[_view_idx(wv, lseq, ldh, S_J, S_A)]                   # [k][j]
            pva[_view_idx(yv, ldh, lseq, S_A, S_I)] = Xd @ Wd.T            # [i][k]
    w["pva"] = lift(pva)
    w["rsat"] = irs_witness_host(w["pva"], 16, 1)
    w["at"] = w["rsat"][0]
    w["acc"][W_O] = mat(w["at"], Wt["w"][W_O], c.d, c.d)
    w["rso"] = irs_witness_host(w["acc"][W_O], 16, 1)
    w["yo"] = w["rso"][0]
    w["res1"], w["idxRes1"] = iadd_witness(x0, w["yo"])
    w["rms2"] = irms_witness(w["res1"], Wt["g2"], T, lT, ld)
    w["h2"] = w["rms2"]["y"]
    for i in (W_G, W_U):
        w["acc"][i] = mat(w["h2"], Wt["w"][i], c.d, c.dff)
    w["rsg"], w["rsu"] = irs_witness_host(w["acc"][W_G], 16, 1), irs_witness_host(w["acc"][W_U], 16, 1)
    w["gg"], w["uu"] = w["rsg"][0], w["rsu"][0]
    w["swg"] = iswg_witness(w["gg"], w["uu"], T)
    w["mo"] = w["swg"][2]
    w["acc"][W_D] = mat(w["mo"], Wt["w"][W_D], c.dff, c.d)
    w["rsd"] = irs_witness_host(w["acc"][W_D], 16, 1)
    w["yd"] = w["rsd"][0]
    w["out"], w["idxOut"] = iadd_witness(w["res1"], w["yd"])
    return w


_CHAIN = ("x0", "h1", "yq", "yk", "yv", "rq", "rk", "sc", "z", "p", "pva", "at", "yo", "res1", "h2", "gg", "uu", "mo", "yd", "out")


def itf_commit_all(engine, w, Wt, R, col):
    """p3itf::commit_all (p3_int_layer.cuh:343-419), non-zk: every chain grid, weight and gain committed once.
    ``col`` uploads a host array into an engine column.  Returns {name: (column, root)}."""
    o = {}
    com = lambda a: (lambda c_: (c_, engine.commit_gpu_rootonly(c_, R)))(col(a))
    for k in _CHAIN:
        o[k] = com(w[k])
    o["g1"], o["g2"] = com(Wt["g1"]), com(Wt["g2"])
    o["w"] = [com(x) for x in Wt["w"]]
    o["acc"] = [com(x) for x in w["acc"]]
    return o


def itf_prove(engine, tr, c, w, o, Wt, T, R, Q, col):
    """p3itf::prove (p3_int_layer.cuh:452-581), non-zk: all sub-proofs in fixed order on one transcript with one
    ledger and one lookup queue, one merged-lookup flush, the public input/output bindings, one batched opening per
    size class.  Returns the serialised TfProof: 6 x u32 dims | 24 + 2A length-prefixed sub-proofs in proving order |
    28 roots | u32 groups (len, GroupProof)* | ioin ioout | u32 batches (len, BatchProof)*."""
    ld, lT, ldff, lseq, ldh, la = c.ld, c.lT, c.ldff, c.lseq, c.ldh, c.la
    le, lef, lez = ld + lT, ldff + lT, la + 2 * lseq
    ctx = Ctx()
    tr.absorb("itf-dims", struct.pack("<6I", c.seq, c.d, c.nh, c.dh, c.dff, c.batch))
    for i in range(7):
        ctx.defer([o["w"][i]], col(w["idxW"][i]), T["RS20"])
    ctx.defer([o["g1"]], col(w["idxG1"]), T["RS20"])
    ctx.defer([o["g2"]], col(w["idxG2"]), T["RS20"])
    ctx.defer([o["x0"]], col(w["idxX0"]), T["RS20"])
    subs = []

    def up(wit):
        return {k: ([col(x) for x in v] if isinstance(v, (list, tuple)) else col(v)) for k, v in wit.items() if k not in ("y", "p")}

    def lift_any(a):                     # host witness: numpy; device witness (ig_dev): torch
        if isinstance(a, np.ndarray):
            return lift(a)
        from . import ig_dev
        return ig_dev.lift(a)

    def rms(name, X, G, Y):
        subs.append(irms_prove(engine, tr, T, X, G, Y, up(w[name]), lT, ld, R, Q, ctx))

    def mm(X, Wc, Y, lj, lk, li, views=None):
        subs.append(imm_prove(engine, tr, X, Wc, Y, lj, lk, li, R, Q, ctx.ledger, views))

    def irs(name, X, Y, lev, sf, rng):
        y, L, iL, iY = w[name]
        subs.append(irs_prove(engine, tr, T, X, Y, ([col(l) for l in L], [col(i) for i in iL], col(iY) if iY is not None else None),
                              lev, sf, rng, R, Q, ctx.ledger, ctx.luq))

    def rope(name, Qc, Y):
        y, rem, iR, iY, Cc, S2 = w[name]
        subs.append(irope_prove(engine, tr, T, (col(lift_any(Cc)), col(lift_any(S2)), ldh), Qc, Y, (col(rem), col(iR), col(iY)), lT, ld, R, Q, ctx))

    rms("rms1", o["x0"], o["g1"], o["h1"])
    for i in (W_Q, W_K, W_V):
        mm(o["h1"], o["w"][i], o["acc"][i], ld, ld, lT)
    irs("rsq", o["acc"][W_Q], o["yq"], le, 16, 1)
    irs("rsk", o["acc"][W_K], o["yk"], le, 16, 1)
    irs("rsv", o["acc"][W_V], o["yv"], le, 16, 1)
    rope("rpq", o["yq"], o["rq"])
    rope("rpk", o["yk"], o["rk"])
    for b in range(c.batch):
        for h in range(c.nh):
            mm(o["rq"], o["rk"], o["sc"], ldh, lseq, lseq, views_qk(c, h, b))
    irs("rsz", o["sc"], o["z"], lez, c.sfz, 2)
    subs.append(ismx_prove(engine, tr, T, o["z"], o["p"], up(w["smx"]), la, lseq, R, Q, ctx))
    for b in range(c.batch):
        for h in range(c.nh):
            mm(o["p"], o["yv"], o["pva"], lseq, ldh, lseq, views_pv(c, h, b))
    irs("rsat", o["pva"], o["at"], le, 16, 1)
    mm(o["at"], o["w"][W_O], o["acc"][W_O], ld, ld, lT)
    irs("rso", o["acc"][W_O], o["yo"], le, 16, 1)
    subs.append(iadd_prove(engine, tr, T, o["x0"], o["yo"], o["res1"], col(w["idxRes1"]), le, R, Q, ctx))
    rms("rms2", o["res1"], o["g2"], o["h2"])
    for i in (W_G, W_U):
        mm(o["h2"], o["w"][i], o["acc"][i], ld, ldff, lT)
    irs("rsg", o["acc"][W_G], o["gg"], lef, 16, 1)
    irs("rsu", o["acc"][W_U], o["uu"], lef, 16, 1)
    sil, rem, mo, iG, iR, iM = w["swg"]
    subs.append(iswg_prove(engine, tr, T, o["gg"], o["uu"], o["mo"], (col(sil), col(rem), col(iG), col(iR), col(iM)), lef, R, Q, ctx))
    mm(o["mo"], o["w"][W_D], o["acc"][W_D], ldff, ld, lT)
    irs("rsd", o["acc"][W_D], o["yd"], le, 16, 1)
    subs.append(iadd_prove(engine, tr, T, o["res1"], o["yd"], o["out"], col(w["idxOut"]), le, R, Q, ctx))
    lug = lu_flush(engine, tr, ctx.luq, ctx.ledger, R)
    z1 = [tr.chal() for _ in range(le)]
    ioin = claimc(engine, tr, ctx.ledger, o["x0"][0], o["x0"][1], z1)
    z2 = [tr.chal() for _ in range(le)]
    ioout = claimc(engine, tr, ctx.ledger, o["out"][0], o["out"][1], z2)
    batches = tail_prove(engine, tr, ctx.ledger, R, Q, "itf-bo")
    blob = lambda b: struct.pack("<I", len(b)) + b
    roots = [o["x0"][1], o["h1"][1]] + [a[1] for a in o["acc"]] + [o[k][1] for k in
             ("yq", "yk", "yv", "rq", "rk", "sc", "z", "p", "pva", "at", "yo", "res1", "h2", "gg", "uu", "mo", "yd", "out")]
    out = struct.pack("<6I", c.seq, c.d, c.nh, c.dh, c.dff, c.batch) + b"".join(blob(s) for s in subs) + b"".join(roots)
    out += struct.pack("<I", len(lug)) + b"".join(blob(b) for b in lug) + struct.pack("<QQ", ioin, ioout)
    return out + struct.pack("<I", len(batches)) + b"".join(blob(b) for b in batches)
