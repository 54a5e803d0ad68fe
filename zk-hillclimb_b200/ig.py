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
