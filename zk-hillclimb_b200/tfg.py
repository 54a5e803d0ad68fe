"""bf16 gadgets of the reference's fp8 transformer layer (zkllm-src/p3_swiglu.cuh and siblings), non-zk, as host logic over
the engine interface of p3.py.  Each gadget: tables from the pinned artefact (tfart.build_art), a witness written as tensor
arithmetic (runs on the GPU or, for small cases, the CPU), commitments, deferred lookups (virtual key columns bound through
the lookup's bind callback), one eq-weighted zero-check whose constraint polynomial is expanded into the term list the
programmable zero-check engine takes, and the opening claims.  Standalone calls end with the lookup flush and the batched
openings, as the reference's unit-test mode does.
"""
import struct

import numpy as np
import torch

from .p3 import GL_P, claimc, commit_cols, lu_flush, make_table


# ---------------------------------------------------------------------------------- constraint polynomials
class Poly(dict):
    """Sparse polynomial over the field in the zero-check's columns: {sorted tuple of column indices: coefficient}."""

    @staticmethod
    def var(i):
        return Poly({(i,): 1})

    @staticmethod
    def const(c):
        return Poly({(): c % GL_P}) if c % GL_P else Poly()

    def __add__(self, o):
        o = o if isinstance(o, Poly) else Poly.const(o)
        out = Poly(self)
        for k, v in o.items():
            out[k] = (out.get(k, 0) + v) % GL_P
            if not out[k]:
                del out[k]
        return out

    __radd__ = __add__

    def __neg__(self):
        return Poly({k: (GL_P - v) % GL_P for k, v in self.items()})

    def __sub__(self, o):
        return self + (-(o if isinstance(o, Poly) else Poly.const(o)))

    def __rsub__(self, o):
        return (-self) + o

    def __mul__(self, o):
        if not isinstance(o, Poly):
            o = Poly.const(o)
        out = Poly()
        for k1, v1 in self.items():
            for k2, v2 in o.items():
                k = tuple(sorted(k1 + k2))
                out[k] = (out.get(k, 0) + v1 * v2) % GL_P
                if not out[k]:
                    del out[k]
        return out

    __rmul__ = __mul__


def boolc(x):
    return x * x - x


def zc_terms(constraints, lam):
    """sum_j lam[j] * constraints[j] as (terms, konst) for Prover.sc_prove_zc; every monomial has 1..3 columns."""
    total = Poly()
    for lj, c in zip(lam, constraints):
        total = total + c * lj
    konst = total.pop((), 0)
    if any(len(k) > 3 for k in total):
        raise ValueError("zero-check constraint of degree > 3")
    return [(v, k) for k, v in total.items()], konst


def _powers(x, n):
    out = [1]
    for _ in range(n - 1):
        out.append(out[-1] * x % GL_P)
    return out


def _inv_or0(t, inverse):
    nz = t != 0
    return torch.where(nz, inverse(torch.where(nz, t, torch.ones_like(t))), torch.zeros_like(t))


def _blob(b):
    return struct.pack("<I", len(b)) + b


def _msgs(m):
    return struct.pack("<I", len(m)) + np.ascontiguousarray(m, dtype=np.uint64).tobytes()


def _u64(vals):
    return np.array(vals, dtype=np.uint64).tobytes()


def _tail(engine, tr, ctx, R, Q, tag, strict=True):
    lug = lu_flush(engine, tr, ctx.luq, ctx.ledger, R, strict)
    batches = [engine.prove_class(tr, np.stack(c[1]), c[2], R, Q, "%s%d" % (tag, i)) for i, c in enumerate(ctx.ledger.cls)]
    return lug, batches


def _ser_tail(lug, batches):
    return (struct.pack("<I", len(lug)) + b"".join(_blob(b) for b in lug),
            struct.pack("<I", len(batches)) + b"".join(_blob(b) for b in batches))


def claim_bind(engine, tr, ledger, cols):
    """Bind callback of a lookup whose virtual key columns are affine in (or broadcasts of) committed columns: claim those
    columns at the lookup point (absorbed like any claim); the values ride in the proof as the member's extra slots.
    cols: (column, root) or (column, root, f) with f mapping the lookup point to the column's point (a sub-range of its
    coordinates for a broadcast column)."""
    def bind(pm, _yv):
        claims, extra = [], []
        for ent in cols:
            c, root = ent[0], ent[1]
            pt = np.ascontiguousarray(ent[2](list(pm)) if len(ent) > 2 else pm, dtype=np.uint64)
            y = engine.eval_h_gpu(c, pt)
            tr.absorb("hwl-y", struct.pack("<Q", y))
            claims.append((c, root, pt, y))
            extra.append(y)
        return claims, extra
    return bind


def range_tab(n, off=0):
    return make_table([np.arange(n, dtype=np.uint64) + np.uint64(off)])


def mul7_tab(art):
    j = np.arange(16384, dtype=np.int64)
    return make_table([128 + (j >> 7), 128 + (j & 127), 128 + art["mul_mo"].astype(np.int64), art["mul_einc"].astype(np.int64)])


def rexp_tab():
    j = np.arange(256)
    return make_table([np.where((j >= 1) & (j <= 254), j, 1)])


# ---------------------------------------------------------------------------------- SwiGLU (p3swg)
(SW_SG, SW_SGS, SW_SGEB, SW_SGMB, SW_SGZ, SW_SGEI, SW_US, SW_UEB, SW_UMB, SW_UZ, SW_UEI, SW_MO, SW_EI, SW_EO) = range(14)
SW_NDS = 14


def swg_tables(art):
    """p3swg::build_tables (p3_swiglu.cuh:46-66)."""
    j = np.arange(65536, dtype=np.int64)
    return {"R128": range_tab(128), "R256": range_tab(256), "MUL7": mul7_tab(art), "REXP": rexp_tab(),
            "SILU": make_table([j, art["silu_tab"].astype(np.int64)])}


def swg_witness(gate, up, art, device="cpu", inverse=None):
    """p3swg::gen_witness (p3_swiglu.cuh:113-160): m = bf16_mul(SILU[gate], up) elementwise on bf16 patterns (uint16
    arrays of 2^ln elements).  Returns the operand pattern columns, the 14 witness columns, the two virtual MUL7 key columns,
    the 7 lookup-index columns and the output patterns."""
    from .hwl import host_inverse
    inverse = inverse or host_inverse
    dev = torch.device(device)
    t64 = lambda a: torch.as_tensor(np.asarray(a).astype(np.int64), device=dev)
    gp, upat = t64(gate), t64(up)
    n = gp.numel()
    if n & (n - 1):
        raise ValueError("swg: n must be pow2")
    sg = t64(art["silu_tab"])[gp]
    sgs, sgeb, sgmb = (sg >> 15) & 1, (sg >> 7) & 255, sg & 127
    us, ueb, umb = (upat >> 15) & 1, (upat >> 7) & 255, upat & 127
    sgz, uz = (sgeb == 0).to(torch.int64), (ueb == 0).to(torch.int64)
    mj = (sgmb << 7) | umb
    mo, ei = 128 + t64(art["mul_mo"])[mj], t64(art["mul_einc"])[mj]
    z2 = (sgz | uz) != 0
    eo = torch.where(z2, torch.ones_like(sgeb), sgeb + ueb - 127 + ei)
    if bool(((eo < 1) | (eo > 254)).any()):
        raise ValueError("swg: mul exp domain")
    m = ((sgs ^ us) << 15) | torch.where(z2, torch.zeros_like(eo), (eo << 7) | (mo - 128))
    ws = [sg, sgs, sgeb, sgmb, sgz, _inv_or0(sgeb, inverse), us, ueb, umb, uz, _inv_or0(ueb, inverse), mo, ei, eo]
    i32 = lambda t: t.to(torch.int32)
    lidx = [i32(gp), i32(sgeb), i32(sgmb), i32(ueb), i32(umb), i32(mj), i32(eo)]
    return {"n": n, "ln": n.bit_length() - 1, "gpat": gp, "upat": upat, "mpat": m, "ws": ws, "sgmf": 128 + sgmb, "umf": 128 + umb,
            "lidx": lidx, "M": m.cpu().numpy().astype(np.uint16)}


def swg_commit_operands(engine, wt, R, col):
    out = {}
    for name, key in (("GATE", "gpat"), ("UP", "upat"), ("M", "mpat")):
        c = col(wt[key])
        out[name] = (c, engine.commit_gpu_rootonly(c, R))
    return out


def swg_constraints():
    """F_sw (p3_swiglu.cuh:172-207) over the columns [E, UP, M, ws[14]] as polynomials in column indices."""
    v = Poly.var
    c = lambda k: v(3 + k)
    z2 = c(SW_SGZ) + c(SW_UZ) - c(SW_SGZ) * c(SW_UZ)
    nz2 = 1 - z2
    sm = c(SW_SGS) + c(SW_US) - 2 * c(SW_SGS) * c(SW_US)
    return [
        c(SW_SG) - (32768 * c(SW_SGS) + 128 * c(SW_SGEB) + c(SW_SGMB)),
        boolc(c(SW_SGS)), boolc(c(SW_SGZ)), c(SW_SGZ) * c(SW_SGEB), c(SW_SGEB) * c(SW_SGEI) - (1 - c(SW_SGZ)),
        v(1) - (32768 * c(SW_US) + 128 * c(SW_UEB) + c(SW_UMB)),
        boolc(c(SW_US)), boolc(c(SW_UZ)), c(SW_UZ) * c(SW_UEB), c(SW_UEB) * c(SW_UEI) - (1 - c(SW_UZ)),
        z2 * (c(SW_EO) - 1),
        nz2 * (c(SW_EO) - (c(SW_SGEB) + c(SW_UEB) + c(SW_EI) - 127)),
        v(2) - (32768 * sm + nz2 * (128 * c(SW_EO) + c(SW_MO) - 128)),
    ]


def swg_prove(engine, tr, wt, T, ops, R, Q, col, ctx=None, strict=True):
    """p3swg::prove (p3_swiglu.cuh:239-312), non-zk.  Returns the serialised SwgProof:
    u32 n | rws[14] | u32 groups (len, GroupProof)* | mE | yE[14] yUP yM | u32 batches (len, BatchProof)*."""
    from .ig import Ctx
    own = ctx is None
    ctx = ctx or Ctx()
    tr.absorb("swg-dims", struct.pack("<I", wt["n"]))
    for name in ("R128", "R256", "MUL7", "REXP", "SILU"):
        tr.absorb("swg-tab", T[name]["id"])
    tr.absorb("swg-G", ops["GATE"][1])
    tr.absorb("swg-U", ops["UP"][1])
    tr.absorb("swg-M", ops["M"][1])
    C = commit_cols(engine, [col(t) for t in wt["ws"]], R)
    for _, root in C:
        tr.absorb("swg-cw", root)
    sgmf, umf = col(wt["sgmf"]), col(wt["umf"])
    specs = [("SILU", [ops["GATE"], C[SW_SG]]), ("R256", [C[SW_SGEB]]), ("R128", [C[SW_SGMB]]), ("R256", [C[SW_UEB]]),
             ("R128", [C[SW_UMB]]), ("MUL7", [(sgmf, None), (umf, None), C[SW_MO], C[SW_EI]]), ("REXP", [C[SW_EO]])]
    for i, (tab, W) in enumerate(specs):
        ent = {"W": W, "idx": col(wt["lidx"][i]), "tab": T[tab]}
        if tab == "MUL7":
            ent["bind"] = claim_bind(engine, tr, ctx.ledger, [C[SW_SGMB], C[SW_UMB]])
        ctx.luq.append(ent)
    zE = [tr.chal() for _ in range(wt["ln"])]
    lam = _powers(tr.chal(), 13)
    terms, konst = zc_terms(swg_constraints(), lam)
    E = engine.build_eq_gpu(np.array(zE, dtype=np.uint64))
    rE, mE, _ = engine.sc_prove_zc(tr, "swg-scE", [E, ops["UP"][0], ops["M"][0]] + [c for c, _ in C], terms, konst)
    rE = [int(x) for x in rE]
    yUP = claimc(engine, tr, ctx.ledger, ops["UP"][0], ops["UP"][1], rE)
    yM = claimc(engine, tr, ctx.ledger, ops["M"][0], ops["M"][1], rE)
    yE = [claimc(engine, tr, ctx.ledger, c, root, rE) for c, root in C]
    lug, batches = _tail(engine, tr, ctx, R, Q, "swg-bo", strict) if own else ([], [])
    sl, sb = _ser_tail(lug, batches)
    return struct.pack("<I", wt["n"]) + b"".join(root for _, root in C) + sl + _msgs(mE) + _u64(yE) + _u64([yUP, yM]) + sb


# ---------------------------------------------------------------------------------- bf16 add block and gadget (p3bfa)
BA_COLS = ("S1 E1 M1 Z1 I1 S2 E2 M2 Z2 I2 SG EH EL MH ML SHS SLS OP KD PWD DR DZ DI DM FAR ZB NZ NNF NN AV CZ AI AN "
           "W PLO PHI PDN PDH PUP U1H U1L U2H U2L QM RR RB RT RTI ZRT L0 QH RUP C CI EO").split()
BA = {name: i for i, name in enumerate(BA_COLS)}
NBA = len(BA_COLS)                       # 55
BT_NAMES = ("R128", "R256", "R512", "D16", "WDA", "RM17", "RMH", "REXP")
# block lookups in flush order: (table, block columns)
BA_LU = [("R256", ("E1",)), ("R256", ("E2",)), ("R128", ("M1",)), ("R128", ("M2",)), ("D16", ("KD", "PWD")), ("R256", ("DR",)),
         ("R128", ("DM",)), ("WDA", ("W", "PLO", "PHI", "PDN", "PDH", "PUP")), ("R512", ("U1H",)), ("R512", ("U1L",)),
         ("R512", ("U2H",)), ("R512", ("U2L",)), ("RM17", ("PDN", "RR")), ("R128", ("QM",)), ("RMH", ("PDH", "RB", "RT")),
         ("REXP", ("EO",))]
N_BA_C = 52


def rm_table(tmax):
    """(2^t, r) for r < 2^t, t = 0..tmax, padded with (1, 0) to a power of two."""
    rows = 2 << tmax
    p, r = np.ones(rows, dtype=np.int64), np.zeros(rows, dtype=np.int64)
    row = 0
    for t in range(tmax + 1):
        p[row:row + (1 << t)] = 1 << t
        r[row:row + (1 << t)] = np.arange(1 << t)
        row += 1 << t
    return make_table([p, r])


def bfa_tables():
    """p3bfa::build_tables (p3_bfadd.cuh:86-124)."""
    T = {"R128": range_tab(128), "R256": range_tab(256), "R512": range_tab(512), "REXP": rexp_tab(), "RM17": rm_table(16)}
    kd = np.where(np.arange(16) < 10, np.arange(16), 0)
    T["D16"] = make_table([kd, 1 << kd])
    w = np.where((np.arange(32) >= 1) & (np.arange(32) <= 18), np.arange(32), 1)
    pdn = 1 << np.maximum(w - 8, 0)
    T["WDA"] = make_table([w, 1 << (w - 1), 1 << w, pdn, pdn >> 1, 1 << np.maximum(8 - w, 0)])
    h, b, x = np.zeros(2048, dtype=np.int64), np.zeros(2048, dtype=np.int64), np.zeros(2048, dtype=np.int64)
    row = 1
    for t in range(10):
        for rb in (0, 1):
            h[row:row + (1 << t)], b[row:row + (1 << t)], x[row:row + (1 << t)] = 1 << t, rb, np.arange(1 << t)
            row += 1 << t
    T["RMH"] = make_table([h, b, x])
    return T


def ba_fill(p1, p2, inverse):
    """p3bfa::ba_fill (p3_bfadd.cuh:167-283) on int64 tensors of bf16 patterns: the canonical bf16 addition replayed with all
    intermediate values.  Returns (55 columns in BA_COLS order, 16 lookup-index columns, output patterns); raises on rows outside
    the gadget's domain (flush / saturate)."""
    from .hwl import enc
    I = torch.int64
    b2i = lambda t: t.to(I)
    one, zero = torch.ones_like(p1), torch.zeros_like(p1)
    shl = torch.bitwise_left_shift
    s1, e1, m1 = (p1 >> 15) & 1, (p1 >> 7) & 255, p1 & 127
    s2, e2, m2 = (p2 >> 15) & 1, (p2 >> 7) & 255, p2 & 127
    z1, z2 = e1 == 0, e2 == 0
    sg = (e2 > e1) | ((e2 == e1) & (m2 > m1))
    pick = lambda a, b: torch.where(sg, b, a)             # hi operand's field
    eh, el = pick(e1, e2), pick(e2, e1)
    mh, ml = 128 + pick(m1, m2), 128 + pick(m2, m1)
    shs, sls = pick(s1, s2), pick(s2, s1)
    op = shs ^ sls
    d = eh - el
    far = d >= 10
    kd = torch.where(far, zero, d)
    pwd = shl(one, kd)
    dr = torch.where(far, d - 10, zero)
    dz = d == 0
    nz = ~z1 & ~z2
    dm = torch.where(nz & dz, mh - ml, zero)
    zb = z1 & z2
    nnf = nz & ~far
    av = torch.where(nnf, mh * pwd + torch.where(op != 0, -ml, ml), zero + 128)
    cz = nnf & (av == 0)
    nn = nnf & ~cz
    an = torch.where((av > 0) & ~cz, av, zero + 128)
    w = zero.clone()
    for j in range(20):
        w += b2i(an >= (1 << j))
    if bool(((w < 1) | (w > 18)).any()):
        raise ValueError("bfa: bitlen window")
    plo, phi = shl(one, w - 1), shl(one, w)
    dn_s, up_s = (w - 8).clamp(min=0), (8 - w).clamp(min=0)
    pdn, pup = shl(one, dn_s), shl(one, up_s)
    pdh = pdn >> 1
    u1, u2 = an - plo, phi - 1 - an
    q = torch.where(w > 8, an >> dn_s, shl(an, up_s))
    rr = an * pup - q * pdn
    rb = b2i((pdh > 0) & (rr >= pdh))
    rt = rr - rb * pdh
    zrt, l0, qh = rt == 0, q & 1, q >> 1
    rup = b2i((rb != 0) & (~zrt | (l0 != 0)))
    qr = q + rup
    c = b2i(qr == 256)
    eo_near = el + w - 8 + c
    if bool((nn & ((eo_near < 1) | (eo_near > 254))).any()):
        raise ValueError("bfa: add exp domain")
    if bool((nz & far & (eh > 254)).any()):
        raise ValueError("bfa: far exp domain")
    eo = torch.where(nn, eo_near, torch.where(nz & far, eh, one))
    out = torch.where(zb, (s1 & s2) << 15,
          torch.where(z1, p2, torch.where(z2, p1, torch.where(far, (shs << 15) | (eh << 7) | (mh - 128),
          torch.where(cz, zero, (shs << 15) | (eo << 7) | (qr - 128 * c - 128))))))
    inv0 = lambda t: _inv_or0(t, inverse)
    v = {"S1": s1, "E1": e1, "M1": m1, "Z1": b2i(z1), "I1": inv0(e1), "S2": s2, "E2": e2, "M2": m2, "Z2": b2i(z2), "I2": inv0(e2),
         "SG": b2i(sg), "EH": eh, "EL": el, "MH": mh, "ML": ml, "SHS": shs, "SLS": sls, "OP": op, "KD": kd, "PWD": pwd, "DR": dr,
         "DZ": b2i(dz), "DI": inv0(d), "DM": dm, "FAR": b2i(far), "ZB": b2i(zb), "NZ": b2i(nz), "NNF": b2i(nnf), "NN": b2i(nn),
         "AV": enc(av), "CZ": b2i(cz), "AI": inv0(enc(av)), "AN": an, "W": w, "PLO": plo, "PHI": phi, "PDN": pdn, "PDH": pdh,
         "PUP": pup, "U1H": u1 >> 9, "U1L": u1 & 511, "U2H": u2 >> 9, "U2L": u2 & 511, "QM": q - 128, "RR": rr, "RB": rb, "RT": rt,
         "RTI": inv0(rt), "ZRT": b2i(zrt), "L0": l0, "QH": qh, "RUP": rup, "C": c, "CI": inv0(enc(qr - 256)), "EO": eo}
    cols = [v[name] for name in BA_COLS]
    rmh = torch.where(pdh == 0, zero, 2 * pdh - 1 + rb * pdh + rt)
    lu = [e1, e2, m1, m2, kd, dr, dm, w, u1 >> 9, u1 & 511, u2 >> 9, u2 & 511, pdn - 1 + rr, q - 128, rmh, eo]
    return cols, [t.to(torch.int32) for t in lu], out


def ba_constraints(c, x1, x2, out):
    """p3bfa::ba_constraints (p3_bfadd.cuh:289-392): the 52 residuals of one add block; c maps a block column name to its
    polynomial variable, x1 / x2 / out are the operand and output pattern variables."""
    nz1, nz2, nfar = 1 - c["Z1"], 1 - c["Z2"], 1 - c["FAR"]
    D = c["EH"] - c["EL"]
    qr256 = c["QM"] + c["RUP"] - 128
    hipat = 32768 * c["SHS"] + 128 * c["EH"] + c["MH"] - 128
    nrpat = 32768 * c["SHS"] + 128 * c["EO"] + c["QM"] + c["RUP"] - 128 * c["C"]
    mux = lambda a, b: a + c["SG"] * (b - a)
    return [
        x1 - (32768 * c["S1"] + 128 * c["E1"] + c["M1"]), boolc(c["S1"]), boolc(c["Z1"]), c["Z1"] * c["E1"], c["E1"] * c["I1"] - nz1,
        x2 - (32768 * c["S2"] + 128 * c["E2"] + c["M2"]), boolc(c["S2"]), boolc(c["Z2"]), c["Z2"] * c["E2"], c["E2"] * c["I2"] - nz2,
        boolc(c["SG"]), c["EH"] - mux(c["E1"], c["E2"]), c["EL"] - mux(c["E2"], c["E1"]),
        c["MH"] - (128 + mux(c["M1"], c["M2"])), c["ML"] - (128 + mux(c["M2"], c["M1"])),
        c["SHS"] - mux(c["S1"], c["S2"]), c["SLS"] - mux(c["S2"], c["S1"]),
        c["OP"] + 2 * c["SHS"] * c["SLS"] - (c["SHS"] + c["SLS"]),
        boolc(c["FAR"]), nfar * (c["KD"] - D), c["FAR"] * c["KD"], c["FAR"] * (D - (c["DR"] + 10)),
        boolc(c["DZ"]), c["DZ"] * D, D * c["DI"] - (1 - c["DZ"]), c["NZ"] * c["DZ"] * (c["MH"] - c["ML"] - c["DM"]),
        c["ZB"] - c["Z1"] * c["Z2"], c["NZ"] - nz1 * nz2, c["NNF"] - c["NZ"] * nfar, c["FAR"] * c["CZ"],
        c["NN"] - c["NNF"] + c["NZ"] * c["CZ"],
        c["NNF"] * (c["AV"] - c["MH"] * c["PWD"] - c["ML"] + 2 * c["OP"] * c["ML"]),
        boolc(c["CZ"]), c["CZ"] * c["AV"], c["AV"] * c["AI"] - (1 - c["CZ"]),
        c["AN"] + c["AV"] * c["CZ"] - (c["AV"] + 128 * c["CZ"]),
        c["AN"] - c["PLO"] - (512 * c["U1H"] + c["U1L"]), c["PHI"] - 1 - c["AN"] - (512 * c["U2H"] + c["U2L"]),
        (c["QM"] + 128) * c["PDN"] + c["RR"] - c["AN"] * c["PUP"], c["RR"] - (c["RB"] * c["PDH"] + c["RT"]),
        c["RT"] * c["RTI"] - (1 - c["ZRT"]), c["ZRT"] * c["RT"], boolc(c["ZRT"]), boolc(c["L0"]),
        c["QM"] + 128 - (2 * c["QH"] + c["L0"]), c["RUP"] + c["RB"] * c["ZRT"] * (1 - c["L0"]) - c["RB"],
        boolc(c["C"]), c["C"] * qr256, qr256 * c["CI"] - (1 - c["C"]),
        c["NN"] * (c["EO"] + 8 - (c["EL"] + c["W"] + c["C"])),
        out - (32768 * c["ZB"] * c["S1"] * c["S2"] + c["Z1"] * nz2 * x2 + nz1 * c["Z2"] * x1 + c["NZ"] * c["FAR"] * hipat
               + c["NN"] * nrpat),
        c["NZ"] * c["FAR"] * (c["EO"] - c["EH"]),
    ]


def bfa_witness(a, b, device="cpu", inverse=None):
    """p3bfa::gen_witness (p3_bfadd.cuh:421-438): out = bf16_add(a, b) elementwise on 2^ln bf16 patterns."""
    from .hwl import host_inverse
    dev = torch.device(device)
    t64 = lambda x: torch.as_tensor(np.asarray(x).astype(np.int64), device=dev)
    x1, x2 = t64(a), t64(b)
    n = x1.numel()
    if n & (n - 1):
        raise ValueError("bfa: n must be pow2")
    ws, lidx, out = ba_fill(x1, x2, inverse or host_inverse)
    return {"n": n, "ln": n.bit_length() - 1, "x1": x1, "x2": x2, "opat": out, "ws": ws, "lidx": lidx,
            "O": out.cpu().numpy().astype(np.uint16)}


def bfa_commit_operands(engine, wt, R, col):
    out = {}
    for name, key in (("X1", "x1"), ("X2", "x2"), ("OUT", "opat")):
        c = col(wt[key])
        out[name] = (c, engine.commit_gpu_rootonly(c, R))
    return out


def bfa_prove(engine, tr, wt, T, ops, R, Q, col, ctx=None, strict=True):
    """p3bfa::prove (p3_bfadd.cuh:447-499), non-zk.  Serialised BfaProof:
    u32 n | rws[55] | u32 groups (len, GroupProof)* | mE | yE[55] yX1 yX2 yOUT | u32 batches (len, BatchProof)*."""
    from .ig import Ctx
    own = ctx is None
    ctx = ctx or Ctx()
    tr.absorb("bfa-dims", struct.pack("<I", wt["n"]))
    for name in BT_NAMES:
        tr.absorb("bfa-tab", T[name]["id"])
    tr.absorb("bfa-X1", ops["X1"][1])
    tr.absorb("bfa-X2", ops["X2"][1])
    tr.absorb("bfa-O", ops["OUT"][1])
    C = commit_cols(engine, [col(t) for t in wt["ws"]], R)
    for _, root in C:
        tr.absorb("bfa-cw", root)
    for i, (tab, names) in enumerate(BA_LU):
        ctx.luq.append({"W": [C[BA[nm]] for nm in names], "idx": col(wt["lidx"][i]), "tab": T[tab]})
    zE = [tr.chal() for _ in range(wt["ln"])]
    lam = _powers(tr.chal(), N_BA_C)
    cv = {name: Poly.var(4 + i) for i, name in enumerate(BA_COLS)}
    terms, konst = zc_terms(ba_constraints(cv, Poly.var(1), Poly.var(2), Poly.var(3)), lam)
    E = engine.build_eq_gpu(np.array(zE, dtype=np.uint64))
    rE, mE, _ = engine.sc_prove_zc(tr, "bfa-scE", [E, ops["X1"][0], ops["X2"][0], ops["OUT"][0]] + [c for c, _ in C], terms, konst)
    rE = [int(x) for x in rE]
    yX = [claimc(engine, tr, ctx.ledger, ops[k][0], ops[k][1], rE) for k in ("X1", "X2", "OUT")]
    yE = [claimc(engine, tr, ctx.ledger, c, root, rE) for c, root in C]
    lug, batches = _tail(engine, tr, ctx, R, Q, "bfa-bo", strict) if own else ([], [])
    sl, sb = _ser_tail(lug, batches)
    return struct.pack("<I", wt["n"]) + b"".join(root for _, root in C) + sl + _msgs(mE) + _u64(yE) + _u64(yX) + sb


# ---------------------------------------------------------------------------------- activation quantisation (p3qnt)
(QD_XS, QD_XEB, QD_XMB, QD_XZ, QD_XEI, QD_SH, QD_SEL, QD_MAG) = range(8)
(QR_E, QR_EDIF, QR_FSEL) = range(3)
Q_EFLOOR = 9


def qnt_tables(art):
    """p3qnt::build_tables (p3_quant.cuh:60-76): R256 and the quantisation table extended with zero rows to dexp < 256."""
    j = np.arange(32768, dtype=np.int64)
    mag = np.zeros(32768, dtype=np.int64)
    mag[:4096] = art["qe4m3"].astype(np.int64)
    return {"R256": range_tab(256), "QEXT": make_table([j >> 7, j & 127, mag])}


def qnt_witness(x, B, ld, art, device="cpu", inverse=None):
    """p3qnt::gen_witness (p3_quant.cuh:143-213): per row of d = 2^ld bf16 patterns, the shared exponent E = max(9, largest
    exponent present), the power-of-two fp32 scale (E - 8) << 23 and the e4m3 code of every element.  x: B*d uint16 patterns.
    Rows are padded to a power of two (at least 2)."""
    from .hwl import host_inverse
    inverse = inverse or host_inverse
    dev = torch.device(device)
    I = torch.int64
    d = 1 << ld
    Bpad = 1 << max(max(B, 2) - 1, 0).bit_length()
    lb = Bpad.bit_length() - 1
    xp = torch.zeros(Bpad, d, dtype=I, device=dev)
    xp[:B] = torch.as_tensor(np.asarray(x).astype(np.int64).reshape(B, d), device=dev)
    xs, xeb, xmb = (xp >> 15) & 1, (xp >> 7) & 255, xp & 127
    xz = xeb == 0
    E = torch.where(xz, torch.zeros_like(xeb), xeb).amax(dim=1).clamp(min=Q_EFLOOR)
    att = ~xz & (xeb == E[:, None])
    sel = att & (att.cumsum(dim=1) == 1)
    fsel = (~att.any(dim=1)).to(I)
    sh = torch.where(xz, torch.zeros_like(xeb), E[:, None] - xeb)
    qe = torch.as_tensor(np.asarray(art["qe4m3"]).astype(np.int64), device=dev)
    mag = torch.where(sh < 32, qe[((sh.clamp(max=31)) << 7) | xmb], torch.zeros_like(sh))
    code = xs * 128 + torch.where(xz, torch.zeros_like(mag), mag)
    scale = (E - 8) << 23
    flat = lambda t: t.reshape(-1).contiguous()
    de = [flat(t) for t in (xs, xeb, xmb, xz.to(I), _inv_or0(xeb, inverse), sh, sel.to(I), mag)]
    db = [E, E - Q_EFLOOR, fsel]
    i32 = lambda t: flat(t).to(torch.int32)
    return {"B": B, "ld": ld, "d": d, "Bpad": Bpad, "lb": lb, "le": lb + ld, "xpat": flat(xp), "cpat": flat(code), "spat": scale,
            "de": de, "db": db, "lidx": [i32(xeb), i32((sh << 7) | xmb), i32(E - Q_EFLOOR)],
            "C": code[:B].cpu().numpy().astype(np.uint8).reshape(-1), "S": scale[:B].cpu().numpy().astype(np.uint32)}


def qnt_commit_operands(engine, wt, R, col):
    out = {}
    for name, key in (("X", "xpat"), ("CODES", "cpat"), ("SCALES", "spat")):
        c = col(wt[key])
        out[name] = (c, engine.commit_gpu_rootonly(c, R))
    return out


def qnt_prove(engine, tr, wt, T, ops, R, Q, col, ctx=None, strict=True):
    """p3qnt::prove (p3_quant.cuh:291-416), non-zk.  Serialised QntProof: u32 B ld | rde[8] rdb[3] | groups |
    mDe yDe[8] yDeX yDeC yDeE | mDb yDb[3] yDbS | yBF | mBind yBSEL | batches."""
    from .ig import Ctx
    from .p3 import F_PROD2
    own = ctx is None
    ctx = ctx or Ctx()
    lg = ctx.ledger
    ld, lb, le = wt["ld"], wt["lb"], wt["le"]
    tr.absorb("qnt-dims", struct.pack("<II", wt["B"], ld))
    tr.absorb("qnt-tab", T["R256"]["id"])
    tr.absorb("qnt-tab", T["QEXT"]["id"])
    tr.absorb("qnt-X", ops["X"][1])
    tr.absorb("qnt-C", ops["CODES"][1])
    tr.absorb("qnt-S", ops["SCALES"][1])
    CDe = commit_cols(engine, [col(t) for t in wt["de"]], R)
    CDb = commit_cols(engine, [col(t) for t in wt["db"]], R)
    for _, root in CDe:
        tr.absorb("qnt-ce", root)
    for _, root in CDb:
        tr.absorb("qnt-cb", root)
    ctx.luq.append({"W": [CDe[QD_XEB]], "idx": col(wt["lidx"][0]), "tab": T["R256"]})
    ctx.luq.append({"W": [CDe[QD_SH], CDe[QD_XMB], CDe[QD_MAG]], "idx": col(wt["lidx"][1]), "tab": T["QEXT"]})
    ctx.luq.append({"W": [CDb[QR_EDIF]], "idx": col(wt["lidx"][2]), "tab": T["R256"]})
    chal_vec = lambda n: [tr.chal() for _ in range(n)]
    eq = lambda z: engine.build_eq_gpu(np.array(z, dtype=np.uint64))
    claim = lambda c, z: claimc(engine, tr, lg, c[0], c[1], z)
    v = Poly.var
    # element domain: columns [E, X, CODES, de[8], E of the row broadcast]
    zE = chal_vec(le)
    lam = _powers(tr.chal(), 11)
    c = lambda k: v(3 + k)
    Ebc, nz = v(11), 1 - c(QD_XZ)
    cons = [v(1) - (32768 * c(QD_XS) + 128 * c(QD_XEB) + c(QD_XMB)), boolc(c(QD_XS)), boolc(c(QD_XZ)), c(QD_XZ) * c(QD_XEB),
            c(QD_XEB) * c(QD_XEI) - nz, nz * (c(QD_SH) + c(QD_XEB) - Ebc), c(QD_XZ) * c(QD_SH), boolc(c(QD_SEL)),
            c(QD_SEL) * c(QD_SH), c(QD_SEL) * c(QD_XZ), v(2) - (128 * c(QD_XS) + nz * c(QD_MAG))]
    terms, konst = zc_terms(cons, lam)
    cols = [eq(zE), ops["X"][0], ops["CODES"][0]] + [t for t, _ in CDe] + [engine.bcast_rows(CDb[QR_E][0], ld)]
    rE, mDe, _ = engine.sc_prove_zc(tr, "qnt-scE", cols, terms, konst)
    rE = [int(x) for x in rE]
    yDeX, yDeC = claim(ops["X"], rE), claim(ops["CODES"], rE)
    yDe = [claim(cd, rE) for cd in CDe]
    yDeE = claim(CDb[QR_E], rE[ld:le])
    # row domain: columns [E, SCALES, db[3]]
    zB = chal_vec(lb)
    lamB = _powers(tr.chal(), 4)
    r_ = lambda k: v(2 + k)
    consB = [boolc(r_(QR_FSEL)), r_(QR_FSEL) * r_(QR_EDIF), r_(QR_E) - (Q_EFLOOR + r_(QR_EDIF)), v(1) - (r_(QR_E) - 8) * (1 << 23)]
    terms, konst = zc_terms(consB, lamB)
    rB, mDb, _ = engine.sc_prove_zc(tr, "qnt-scB", [eq(zB), ops["SCALES"][0]] + [t for t, _ in CDb], terms, konst)
    rB = [int(x) for x in rB]
    yDbS = claim(ops["SCALES"], rB)
    yDb = [claim(cd, rB) for cd in CDb]
    # row binding: sum_i SEL = 1 - FSEL
    z2 = chal_vec(lb)
    yBF = claim(CDb[QR_FSEL], z2)
    rS, mBind, _ = engine.sc_prove_gpu(tr, "qnt-scS", [engine.bcast_rows(eq(z2), ld), CDe[QD_SEL][0]], F_PROD2, 5)
    yBSEL = claim(CDe[QD_SEL], [int(x) for x in rS])
    lug, batches = _tail(engine, tr, ctx, R, Q, "qnt-bo", strict) if own else ([], [])
    sl, sb = _ser_tail(lug, batches)
    out = struct.pack("<II", wt["B"], ld) + b"".join(r for _, r in CDe) + b"".join(r for _, r in CDb) + sl
    out += _msgs(mDe) + _u64(yDe) + _u64([yDeX, yDeC, yDeE]) + _msgs(mDb) + _u64(yDb) + _u64([yDbS, yBF]) + _msgs(mBind) + _u64([yBSEL])
    return out + sb


# ---------------------------------------------------------------------------------- RoPE (p3rope)
RP_FIXED = ("AS AEB AMB AZ AEI BS BEB BMB BZ BEI MOAC EIAC EOAC PAC MOSB EISB EOSB PSB MOCB EICB EOCB PCB MOSA EISA EOSA PSA "
            "NSB").split()
RP = {name: i for i, name in enumerate(RP_FIXED)}
RP_A1, RP_A2 = len(RP_FIXED), len(RP_FIXED) + NBA
NDR = len(RP_FIXED) + 2 * NBA            # 137
N_RP_C = 23 + 2 * N_BA_C


def rope_tables(art):
    """p3rope::build_tables (p3_rope.cuh:88-98): the add block's tables plus MUL7."""
    T = bfa_tables()
    T["MUL7"] = mul7_tab(art)
    return T


def _bf_fields(p):
    eb = (p >> 7) & 255
    return (p >> 15) & 1, eb, p & 127, (eb == 0).to(torch.int64)


def _bf_mul(x, t, art_mo, art_ei, what):
    """canonical bf16 product of decomposed operands (sign, exponent, mantissa, zero flag): (mo, ei, eo, pattern, MUL7 row)"""
    mj = (x[2] << 7) | t[2]
    mo, ei = 128 + art_mo[mj], art_ei[mj]
    z2 = (x[3] | t[3]) != 0
    eo = torch.where(z2, torch.ones_like(mj), x[1] + t[1] - 127 + ei)
    if bool(((eo < 1) | (eo > 254)).any()):
        raise ValueError("%s: mul exp domain" % what)
    pat = ((x[0] ^ t[0]) << 15) | torch.where(z2, torch.zeros_like(eo), (eo << 7) | (mo - 128))
    return mo, ei, eo, pat, mj


def rope_witness(q, cos, sin, seq, dh, art, device="cpu", inverse=None):
    """p3rope::gen_witness (p3_rope.cuh:146-243): llama rotate-half RoPE on bf16 patterns with public bf16 cos / sin tables
    (seq * dh/2 patterns each): four canonical products and two canonical adds per (position, pair)."""
    from .hwl import host_inverse
    inverse = inverse or host_inverse
    dev = torch.device(device)
    t64 = lambda a: torch.as_tensor(np.asarray(a).astype(np.int64), device=dev)
    half = dh // 2
    lp, lh = seq.bit_length() - 1, half.bit_length() - 1
    if (1 << lp) != seq or (1 << lh) != half:
        raise ValueError("rope: dims must be pow2")
    Q = t64(q).reshape(seq, dh)
    ap, bp = Q[:, :half].reshape(-1).contiguous(), Q[:, half:].reshape(-1).contiguous()
    da, db, dc, ds = _bf_fields(ap), _bf_fields(bp), _bf_fields(t64(cos).reshape(-1)), _bf_fields(t64(sin).reshape(-1))
    mo_t, ei_t = t64(art["mul_mo"]), t64(art["mul_einc"])
    pac, psb, pcb, psa = (_bf_mul(x, t, mo_t, ei_t, "rope") for x, t in ((da, dc), (db, ds), (db, dc), (da, ds)))
    nsb = psb[3] ^ 0x8000
    a1, lu1, oa = ba_fill(pac[3], nsb, inverse)
    a2, lu2, ob = ba_fill(pcb[3], psa[3], inverse)
    inv0 = lambda t: _inv_or0(t, inverse)
    ws = [da[0], da[1], da[2], da[3], inv0(da[1]), db[0], db[1], db[2], db[3], inv0(db[1])]
    for m in (pac, psb, pcb, psa):
        ws += [m[0], m[1], m[2], m[3]]
    ws += [nsb] + a1 + a2
    i32 = lambda t: t.to(torch.int32)
    lidx = [i32(da[1]), i32(da[2]), i32(db[1]), i32(db[2]), i32(pac[4]), i32(psb[4]), i32(pcb[4]), i32(psa[4]),
            i32(pac[2]), i32(psb[2]), i32(pcb[2]), i32(psa[2])] + lu1 + lu2
    out = torch.cat([oa.reshape(seq, half), ob.reshape(seq, half)], dim=1).reshape(-1).contiguous()
    return {"seq": seq, "dh": dh, "lp": lp, "lh": lh, "ln": lp + lh, "qpat": Q.reshape(-1).contiguous(), "opat": out, "qa": ap, "qb": bp,
            "oa": oa, "ob": ob, "cf": list(dc), "sf": list(ds), "ws": ws, "lidx": lidx, "amf": 128 + da[2], "bmf": 128 + db[2],
            "cmf": 128 + dc[2], "smf": 128 + ds[2], "OUT": out.cpu().numpy().astype(np.uint16)}


def rope_commit_operands(engine, wt, R, col):
    out = {}
    for name, key in (("Q", "qpat"), ("OUT", "opat")):
        c = col(wt[key])
        out[name] = (c, engine.commit_gpu_rootonly(c, R))
    return out


def rope_constraints():
    """F_rp (p3_rope.cuh:262-318) over [Eq, QA, QB, OA, OB, cos fields s eb mb z, sin fields s eb mb z, ws[137]]."""
    v = Poly.var
    c = lambda name: v(13 + RP[name])
    cons = []
    for x, src in (("A", 1), ("B", 2)):
        cons += [v(src) - (32768 * c(x + "S") + 128 * c(x + "EB") + c(x + "MB")), boolc(c(x + "S")), boolc(c(x + "Z")),
                 c(x + "Z") * c(x + "EB"), c(x + "EB") * c(x + "EI") - (1 - c(x + "Z"))]
    for x, tv, suf in (("A", 5, "AC"), ("B", 9, "SB"), ("B", 5, "CB"), ("A", 9, "SA")):
        TS, TEB, TZ = v(tv), v(tv + 1), v(tv + 3)
        z2 = c(x + "Z") + TZ - c(x + "Z") * TZ
        sg = c(x + "S") + TS - 2 * c(x + "S") * TS
        cons += [z2 * (c("EO" + suf) - 1), (1 - z2) * (c("EO" + suf) - (c(x + "EB") + TEB + c("EI" + suf) - 127)),
                 c("P" + suf) - (32768 * sg + (1 - z2) * (128 * c("EO" + suf) + c("MO" + suf) - 128))]
    sgsb = c("BS") + v(9) - 2 * c("BS") * v(9)
    cons.append(c("NSB") + 65536 * sgsb - (c("PSB") + 32768))
    blk = lambda base: {name: v(13 + base + i) for i, name in enumerate(BA_COLS)}
    cons += ba_constraints(blk(RP_A1), c("PAC"), c("NSB"), v(3))
    cons += ba_constraints(blk(RP_A2), c("PCB"), c("PSA"), v(4))
    return cons


def rope_prove(engine, tr, wt, T, ops, R, Q, col, ctx=None, strict=True):
    """p3rope::prove (p3_rope.cuh:345-459), non-zk.  Serialised RopeProof: u32 lp lh | rws[137] | groups | mE |
    u32 137, yE | yQA yQB yOA yOB | batches."""
    from .ig import Ctx
    own = ctx is None
    ctx = ctx or Ctx()
    lg = ctx.ledger
    lh, ln = wt["lh"], wt["ln"]
    field_bytes = lambda t: t.cpu().numpy().astype(np.uint64).tobytes()
    tr.absorb("rop-dims", struct.pack("<II", wt["lp"], lh))
    for name in BT_NAMES:
        tr.absorb("rop-tab", T[name]["id"])
    tr.absorb("rop-tab", T["MUL7"]["id"])
    for k in range(4):
        tr.absorb("rop-cos", field_bytes(wt["cf"][k]))
        tr.absorb("rop-sin", field_bytes(wt["sf"][k]))
    tr.absorb("rop-Q", ops["Q"][1])
    tr.absorb("rop-O", ops["OUT"][1])
    C = commit_cols(engine, [col(t) for t in wt["ws"]], R)
    for _, root in C:
        tr.absorb("rop-cw", root)
    virt = {k: (col(wt[k]), None) for k in ("amf", "bmf", "cmf", "smf")}
    cc = lambda name: C[RP[name]]
    specs = [("R256", [cc("AEB")], None), ("R128", [cc("AMB")], None), ("R256", [cc("BEB")], None), ("R128", [cc("BMB")], None),
             ("MUL7", [virt["amf"], virt["cmf"], cc("MOAC"), cc("EIAC")], "AMB"), ("MUL7", [virt["bmf"], virt["smf"], cc("MOSB"), cc("EISB")], "BMB"),
             ("MUL7", [virt["bmf"], virt["cmf"], cc("MOCB"), cc("EICB")], "BMB"), ("MUL7", [virt["amf"], virt["smf"], cc("MOSA"), cc("EISA")], "AMB"),
             ("REXP", [cc("EOAC")], None), ("REXP", [cc("EOSB")], None), ("REXP", [cc("EOCB")], None), ("REXP", [cc("EOSA")], None)]
    for base in (RP_A1, RP_A2):
        specs += [(tab, [C[base + BA[nm]] for nm in names], None) for tab, names in BA_LU]
    for i, (tab, W, bindcol) in enumerate(specs):
        ent = {"W": W, "idx": col(wt["lidx"][i]), "tab": T[tab]}
        if bindcol:
            ent["bind"] = claim_bind(engine, tr, lg, [cc(bindcol)])
        ctx.luq.append(ent)
    zE = [tr.chal() for _ in range(ln)]
    lam = _powers(tr.chal(), N_RP_C)
    terms, konst = zc_terms(rope_constraints(), lam)
    cols = [engine.build_eq_gpu(np.array(zE, dtype=np.uint64))] + [col(wt[k]) for k in ("qa", "qb", "oa", "ob")] + \
        [col(t) for t in wt["cf"]] + [col(t) for t in wt["sf"]] + [c for c, _ in C]
    rE, mE, _ = engine.sc_prove_zc(tr, "rop-scE", cols, terms, konst)
    rE = [int(x) for x in rE]
    ins = lambda bit: rE[:lh] + [bit] + rE[lh:]
    claim = lambda c, z: claimc(engine, tr, lg, c[0], c[1], z)
    yQ = [claim(ops["Q"], ins(0)), claim(ops["Q"], ins(1)), claim(ops["OUT"], ins(0)), claim(ops["OUT"], ins(1))]
    yE = [claim(cd, rE) for cd in C]
    lug, batches = _tail(engine, tr, ctx, R, Q, "rop-bo", strict) if own else ([], [])
    sl, sb = _ser_tail(lug, batches)
    return struct.pack("<II", wt["lp"], lh) + b"".join(r for _, r in C) + sl + _msgs(mE) + struct.pack("<I", len(yE)) + _u64(yE) + \
        _u64(yQ) + sb


# ---------------------------------------------------------------------------------- RMSNorm (p3rms)
RMS_DE = "XS XEB XMB XZ XEI SH PW Q RR SEL MO1 EI1 EO1 MO2 EI2 EO2".split()
RMS_DB = "E FSEL EDIF S EPSA WD PLO PHI PDN PUP U1H U1L U2H U2L NR U16 QB PP MR HB TEB".split()
RMS_DW = "GS GEB GMB GZ GEI".split()
RD, RB_, RW = ({n: i for i, n in enumerate(names)} for names in (RMS_DE, RMS_DB, RMS_DW))
RMS_TABS = ("R128", "R256", "R512", "R11", "R12", "R16", "SH512", "RM17", "RM8", "WD24", "EPSAT", "RSQT", "MUL7", "REXP")


def rms_tables(art):
    """p3rms::build_tables (p3_rmsnorm.cuh:95-146); the window of the row sum depends on the row length 2^ld."""
    wmax = 17 + art["ld"]
    if wmax > 30:
        raise ValueError("rms: ld too large (WMAX > 30)")
    j = np.arange(512, dtype=np.int64)
    wd = np.where(np.arange(32) <= wmax, np.arange(32), 0).astype(np.int64)
    j16 = np.arange(65536, dtype=np.int64)
    return {"R128": range_tab(128), "R256": range_tab(256), "R512": range_tab(512), "R11": range_tab(1 << (wmax - 12)),
            "R12": range_tab(4096), "R16": range_tab(65536), "SH512": make_table([j, 1 << np.minimum(j, 16)]),
            "RM17": rm_table(16), "RM8": rm_table(wmax - 16),
            "WD24": make_table([wd, np.where(wd > 0, 1 << np.maximum(wd - 1, 0), 0), 1 << wd, 1 << np.maximum(wd - 16, 0),
                                1 << np.maximum(16 - wd, 0)]),
            "EPSAT": make_table([j, art["epsa"].astype(np.int64)]),
            "RSQT": make_table([32768 + (j16 & 32767), j16 >> 15, 128 + art["rsq_mr"].astype(np.int64), art["rsq_hb"].astype(np.int64)]),
            "MUL7": mul7_tab(art), "REXP": rexp_tab()}


def _bitlen(t, maxbits):
    w = torch.zeros_like(t)
    for j in range(maxbits):
        w += (t >= (1 << j)).to(torch.int64)
    return w


def rms_witness(x, g, B, art, device="cpu", inverse=None):
    """p3rms::gen_witness (p3_rmsnorm.cuh:225-377): canonical RMSNorm of B rows of d = 2^ld bf16 patterns with bf16 gains:
    block-float sum of squares, eps, top-16-bit normalisation, table reciprocal square root, two table multiplies."""
    from .hwl import enc, host_inverse
    inverse = inverse or host_inverse
    dev = torch.device(device)
    I = torch.int64
    t64 = lambda a: torch.as_tensor(np.asarray(a).astype(np.int64), device=dev)
    ld, EMIN = art["ld"], art["EMIN"]
    d = 1 << ld
    Bpad = 1 << max(max(B, 2) - 1, 0).bit_length()
    lb = Bpad.bit_length() - 1
    shl = torch.bitwise_left_shift
    xp = torch.zeros(Bpad, d, dtype=I, device=dev)
    xp[:B] = t64(x).reshape(B, d)
    gp = t64(g)
    gs, geb, gmb, gz = _bf_fields(gp)
    xs, xeb, xmb, xz = _bf_fields(xp)
    pres = xz == 0
    E = torch.where(pres, 2 * xeb, torch.zeros_like(xeb)).amax(dim=1).clamp(min=EMIN)
    att = pres & (2 * xeb == E[:, None])
    sel = att & (att.cumsum(dim=1) == 1)
    fsel = (~att.any(dim=1)).to(I)
    zero, one = torch.zeros_like(xeb), torch.ones_like(xeb)
    sh = torch.where(pres, E[:, None] - 2 * xeb, zero)
    shc = sh.clamp(max=16)
    pw = torch.where(pres, shl(one, shc), one)
    sq = (128 + xmb) * (128 + xmb)
    q = torch.where(pres, sq >> shc, zero)
    rr = torch.where(pres, sq - shl(q, shc), zero)
    S = q.sum(dim=1)
    epsa = t64(art["epsa"])[E.clamp(max=511)]
    Sp = S + epsa
    if bool(((Sp < 1) | (Sp >= (1 << (17 + ld)))).any()):
        raise ValueError("rms: S' window")
    wd = _bitlen(Sp, 40)
    o1 = torch.ones_like(wd)
    plo, phi = shl(o1, wd - 1), shl(o1, wd)
    dn_s, up_s = (wd - 16).clamp(min=0), (16 - wd).clamp(min=0)
    pdn, pup = shl(o1, dn_s), shl(o1, up_s)
    u1, u2 = Sp - plo, phi - 1 - Sp
    nr = torch.where(wd > 16, Sp & (pdn - 1), torch.zeros_like(Sp))
    u16 = torch.where(wd > 16, Sp >> dn_s, shl(Sp, up_s))
    Xexp = E + wd - (284 + ld)
    qb = (Xexp + 400) >> 1
    pp = Xexp + 400 - 2 * qb
    rsj = (pp << 15) | (u16 - 32768)
    mrfull, hb = 128 + t64(art["rsq_mr"])[rsj], t64(art["rsq_hb"])[rsj]
    teb = 318 + hb - qb
    if bool(((teb < 1) | (teb > 254)).any()):
        raise ValueError("rms: rsqrt exp domain")
    mo_t, ei_t = t64(art["mul_mo"]), t64(art["mul_einc"])
    j1 = (xmb << 7) | (mrfull[:, None] - 128)
    mo1, ei1 = 128 + mo_t[j1], ei_t[j1]
    eo1 = torch.where(pres, xeb + teb[:, None] - 127 + ei1, one)
    if bool(((eo1 < 1) | (eo1 > 254)).any()):
        raise ValueError("rms: mul1 exp domain")
    j2 = ((mo1 - 128) << 7) | gmb[None, :]
    mo2, ei2 = 128 + mo_t[j2], ei_t[j2]
    z2 = (xz | gz[None, :]) != 0
    eo2 = torch.where(z2, one, eo1 + geb[None, :] - 127 + ei2)
    if bool(((eo2 < 1) | (eo2 > 254)).any()):
        raise ValueError("rms: mul2 exp domain")
    y = ((xs ^ gs[None, :]) << 15) | torch.where(z2, zero, (eo2 << 7) | (mo2 - 128))
    inv0 = lambda t: _inv_or0(t, inverse)
    flat = lambda t: t.reshape(-1).contiguous()
    de = [flat(t) for t in (xs, xeb, xmb, xz, inv0(xeb), sh, pw, q, enc(rr), sel.to(I), mo1, ei1, eo1, mo2, ei2, eo2)]
    db = [E, fsel, E - EMIN, S, epsa, wd, plo, phi, pdn, pup, u1 >> 12, u1 & 4095, u2 >> 12, u2 & 4095, nr, u16, qb, pp, mrfull, hb, teb]
    dw = [gs, geb, gmb, gz, inv0(geb)]
    i32 = lambda t: flat(t).to(torch.int32)
    lidx = [i32(xeb), i32(xmb), i32(sh), i32(pw - 1 + rr), i32(q), i32(j1), i32(j2), i32(eo1), i32(eo2), i32(geb), i32(gmb),
            i32(E.clamp(max=511)), i32(wd), i32(u1 >> 12), i32(u1 & 4095), i32(u2 >> 12), i32(u2 & 4095), i32(pdn - 1 + nr), i32(rsj),
            i32(E - EMIN), i32(qb), i32(teb)]
    return {"B": B, "ld": ld, "d": d, "Bpad": Bpad, "lb": lb, "le": lb + ld, "xpat": flat(xp), "gpat": gp, "ypat": flat(y), "de": de,
            "db": db, "dw": dw, "xmf": flat(128 + xmb), "mrf": flat(mrfull[:, None].expand(Bpad, d)), "gmf": flat((128 + gmb)[None, :].expand(Bpad, d)),
            "lidx": lidx, "Y": y[:B].cpu().numpy().astype(np.uint16).reshape(-1)}


def rms_commit_operands(engine, wt, R, col):
    out = {}
    for name, key in (("X", "xpat"), ("G", "gpat"), ("Y", "ypat")):
        c = col(wt[key])
        out[name] = (c, engine.commit_gpu_rootonly(c, R))
    return out


def rms_prove(engine, tr, wt, T, art, ops, R, Q, col, ctx=None, strict=True):
    """p3rms::prove (p3_rmsnorm.cuh:527-735), non-zk.  Serialised RmsProof: u32 B ld | rde[16] rdb[21] rdw[5] | groups |
    mDe yDe[16] yDeX yDeY yDeE yDeTEB yDeGS yDeGEB yDeGZ | mDb yDb[21] | mDw yDw[5] yDwG | yBS yBF | mBind yBXZ yBQ yBSEL | batches."""
    from .ig import Ctx
    own = ctx is None
    ctx = ctx or Ctx()
    lg = ctx.ledger
    ld, lb, le = wt["ld"], wt["lb"], wt["le"]
    tr.absorb("rms-dims", struct.pack("<IIII", wt["B"], ld, art["EMIN"], art["eps_bits"]))
    for name in RMS_TABS:
        tr.absorb("rms-tab", T[name]["id"])
    tr.absorb("rms-X", ops["X"][1])
    tr.absorb("rms-G", ops["G"][1])
    tr.absorb("rms-Y", ops["Y"][1])
    commit = lambda cols: commit_cols(engine, [col(t) for t in cols], R)
    CDe, CDb, CDw = commit(wt["de"]), commit(wt["db"]), commit(wt["dw"])
    for label, cd in (("rms-ce", CDe), ("rms-cb", CDb), ("rms-cw", CDw)):
        for _, root in cd:
            tr.absorb(label, root)
    e_, b_, w_ = (lambda n: CDe[RD[n]]), (lambda n: CDb[RB_[n]]), (lambda n: CDw[RW[n]])
    xmf, mrf, gmf = ((col(wt[k]), None) for k in ("xmf", "mrf", "gmf"))
    specs = [("R256", [e_("XEB")]), ("R128", [e_("XMB")]), ("SH512", [e_("SH"), e_("PW")]), ("RM17", [e_("PW"), e_("RR")]),
             ("R16", [e_("Q")]), ("MUL7", [xmf, mrf, e_("MO1"), e_("EI1")]), ("MUL7", [e_("MO1"), gmf, e_("MO2"), e_("EI2")]),
             ("REXP", [e_("EO1")]), ("REXP", [e_("EO2")]), ("R256", [w_("GEB")]), ("R128", [w_("GMB")]),
             ("EPSAT", [b_("E"), b_("EPSA")]), ("WD24", [b_(n) for n in ("WD", "PLO", "PHI", "PDN", "PUP")]), ("R11", [b_("U1H")]),
             ("R12", [b_("U1L")]), ("R11", [b_("U2H")]), ("R12", [b_("U2L")]), ("RM8", [b_("PDN"), b_("NR")]),
             ("RSQT", [b_(n) for n in ("U16", "PP", "MR", "HB")]), ("R512", [b_("EDIF")]), ("R512", [b_("QB")]), ("REXP", [b_("TEB")])]
    for i, (tab, W) in enumerate(specs):
        ent = {"W": W, "idx": col(wt["lidx"][i]), "tab": T[tab]}
        if i == 5:
            ent["bind"] = claim_bind(engine, tr, lg, [e_("XMB"), b_("MR") + (lambda pm: pm[ld:le],)])
        elif i == 6:
            ent["bind"] = claim_bind(engine, tr, lg, [w_("GMB") + (lambda pm: pm[:ld],)])
        ctx.luq.append(ent)
    chal_vec = lambda n: [tr.chal() for _ in range(n)]
    eq = lambda z: engine.build_eq_gpu(np.array(z, dtype=np.uint64))
    claim = lambda c, z: claimc(engine, tr, lg, c[0], c[1], z)
    v = Poly.var
    # element domain: [E, X, Y, de[16], E row, TEB row, GS col, GEB col, GZ col]
    zE = chal_vec(le)
    lam = _powers(tr.chal(), 16)
    c = lambda n: v(3 + RD[n])
    Ebc, TEB, GS, GEB, GZ = (v(19 + k) for k in range(5))
    nz = 1 - c("XZ")
    z2 = c("XZ") + GZ - c("XZ") * GZ
    xmfp = 128 + c("XMB")
    sy = c("XS") + GS - 2 * c("XS") * GS
    cons = [v(1) - (32768 * c("XS") + 128 * c("XEB") + c("XMB")), boolc(c("XS")), boolc(c("XZ")), c("XZ") * c("XEB"),
            c("XEB") * c("XEI") - nz, c("Q") * c("PW") + c("RR") - nz * xmfp * xmfp, nz * (c("SH") + 2 * c("XEB") - Ebc),
            c("XZ") * c("SH"), boolc(c("SEL")), c("SEL") * c("SH"), c("SEL") * c("XZ"),
            nz * (c("EO1") - (c("XEB") + TEB + c("EI1") - 127)), c("XZ") * (c("EO1") - 1), z2 * (c("EO2") - 1),
            (1 - z2) * (c("EO2") - (c("EO1") + GEB + c("EI2") - 127)),
            v(2) - (32768 * sy + (1 - z2) * (128 * c("EO2") + c("MO2") - 128))]
    terms, konst = zc_terms(cons, lam)
    cols = [eq(zE), ops["X"][0], ops["Y"][0]] + [t for t, _ in CDe] + [engine.bcast_rows(b_("E")[0], ld), engine.bcast_rows(b_("TEB")[0], ld),
            engine.bcast_cols(w_("GS")[0], lb), engine.bcast_cols(w_("GEB")[0], lb), engine.bcast_cols(w_("GZ")[0], lb)]
    rE, mDe, _ = engine.sc_prove_zc(tr, "rms-scE", cols, terms, konst)
    rE = [int(x) for x in rE]
    yDeX, yDeY = claim(ops["X"], rE), claim(ops["Y"], rE)
    yDe = [claim(cd, rE) for cd in CDe]
    rb, ri = rE[ld:le], rE[:ld]
    yDeT = [claim(b_("E"), rb), claim(b_("TEB"), rb), claim(w_("GS"), ri), claim(w_("GEB"), ri), claim(w_("GZ"), ri)]
    # row domain: [E, db[21]]
    zB = chal_vec(lb)
    lamB = _powers(tr.chal(), 10)
    r_ = lambda n: v(1 + RB_[n])
    Sp = r_("S") + r_("EPSA")
    consB = [boolc(r_("FSEL")), r_("FSEL") * r_("EDIF"), r_("E") - (art["EMIN"] + r_("EDIF")), boolc(r_("PP")), boolc(r_("HB")),
             r_("E") + r_("WD") + 400 - (2 * r_("QB") + r_("PP") + (284 + ld)), r_("TEB") + r_("QB") - (318 + r_("HB")),
             Sp - r_("PLO") - (4096 * r_("U1H") + r_("U1L")), r_("PHI") - 1 - Sp - (4096 * r_("U2H") + r_("U2L")),
             r_("U16") * r_("PDN") + r_("NR") - Sp * r_("PUP")]
    terms, konst = zc_terms(consB, lamB)
    rB, mDb, _ = engine.sc_prove_zc(tr, "rms-scB", [eq(zB)] + [t for t, _ in CDb], terms, konst)
    rB = [int(x) for x in rB]
    yDb = [claim(cd, rB) for cd in CDb]
    # gain domain: [E, G, dw[5]]
    zW = chal_vec(ld)
    lamW = _powers(tr.chal(), 5)
    consW = [v(1) - (32768 * v(2) + 128 * v(3) + v(4)), boolc(v(2)), boolc(v(5)), v(5) * v(3), v(3) * v(6) - (1 - v(5))]
    terms, konst = zc_terms(consW, lamW)
    rW, mDw, _ = engine.sc_prove_zc(tr, "rms-scW", [eq(zW), ops["G"][0]] + [t for t, _ in CDw], terms, konst)
    rW = [int(x) for x in rW]
    yDwG = claim(ops["G"], rW)
    yDw = [claim(cd, rW) for cd in CDw]
    # row binding: sum_i (1 - XZ) Q = S and sum_i SEL = 1 - FSEL
    z2r = chal_vec(lb)
    yBS, yBF = claim(b_("S"), z2r), claim(b_("FSEL"), z2r)
    lam1, lam2 = tr.chal(), tr.chal()
    terms, konst = zc_terms([(1 - v(1)) * v(2), v(3)], [lam1, lam2])
    rS, mBind, _ = engine.sc_prove_zc(tr, "rms-scS", [engine.bcast_rows(eq(z2r), ld), e_("XZ")[0], e_("Q")[0], e_("SEL")[0]], terms, konst)
    rS = [int(x) for x in rS]
    yB = [claim(e_("XZ"), rS), claim(e_("Q"), rS), claim(e_("SEL"), rS)]
    lug, batches = _tail(engine, tr, ctx, R, Q, "rms-bo", strict) if own else ([], [])
    sl, sb = _ser_tail(lug, batches)
    out = struct.pack("<II", wt["B"], ld) + b"".join(r for cd in (CDe, CDb, CDw) for _, r in cd) + sl
    out += _msgs(mDe) + _u64(yDe) + _u64([yDeX, yDeY] + yDeT) + _msgs(mDb) + _u64(yDb) + _msgs(mDw) + _u64(yDw) + _u64([yDwG])
    out += _u64([yBS, yBF]) + _msgs(mBind) + _u64(yB)
    return out + sb


# ---------------------------------------------------------------------------------- masked softmax (p3smx)
SMX_FIXED = "XM X2M DP DK SEL1 EXV EEB EMB EZ EZI SH2 PW2 Q2 RR2 SEL2 MO3 EI3 EO3".split()
SM = {n: i for i, n in enumerate(SMX_FIXED)}
SM_A = len(SMX_FIXED)
NDE2 = SM_A + NBA                          # 73
SMX_DB = "KMAX MXP E EDIF FSEL S WD PLO PHI PDN PUP U1H U1L U2H U2L NR U16 MRC HBC REB".split()
SB = {n: i for i, n in enumerate(SMX_DB)}
SMX_XT = ("R11", "R12", "R16", "SH512", "WD24", "RM8", "MUL7", "EXPT", "RCPT")
N_SM_DE = 22 + N_BA_C


def smx_tables(art, wmax=23):
    """p3smx::build_tables (p3_softmax.cuh:95-138): the add block's tables plus the denominator / exp / reciprocal tables;
    rows of 2^ln lanes need wmax >= 16 + ln."""
    if not 23 <= wmax <= 30:
        raise ValueError("smx: wmax out of [23,30]")
    T = bfa_tables()
    j = np.arange(512, dtype=np.int64)
    wd = np.where(np.arange(32) <= wmax, np.arange(32), 0).astype(np.int64)
    j16, j15 = np.arange(65536, dtype=np.int64), np.arange(32768, dtype=np.int64)
    T.update({"wmax": wmax, "R11": range_tab(1 << (wmax - 12)), "R12": range_tab(4096), "R16": range_tab(65536),
              "SH512": make_table([j, 1 << np.minimum(j, 16)]),
              "WD24": make_table([wd, np.where(wd > 0, 1 << np.maximum(wd - 1, 0), 0), 1 << wd, 1 << np.maximum(wd - 16, 0),
                                  1 << np.maximum(16 - wd, 0)]),
              "RM8": rm_table(wmax - 16), "MUL7": mul7_tab(art), "EXPT": make_table([j16, art["exp_tab"].astype(np.int64)]),
              "RCPT": make_table([32768 + j15, 128 + art["rcp_mr"].astype(np.int64), art["rcp_hb"].astype(np.int64)])})
    return T


def smx_witness(s, msk, B, ln, art, device="cpu", inverse=None):
    """p3smx::gen_witness (p3_softmax.cuh:213-398): canonical masked softmax of B rows of n = 2^ln bf16 scores (masked lanes
    output +0 and take no part in the maximum or the sum): key-order maximum, one bf16 subtract block, table exp, block-float
    denominator, table reciprocal, table multiply."""
    from .hwl import host_inverse
    inverse = inverse or host_inverse
    dev = torch.device(device)
    I = torch.int64
    t64 = lambda a: torch.as_tensor(np.asarray(a).astype(np.int64), device=dev)
    n = 1 << ln
    Bpad = 1 << max(max(B, 2) - 1, 0).bit_length()
    lb = Bpad.bit_length() - 1
    EMIN = art["sm_emin"]
    shl = torch.bitwise_left_shift
    sp = torch.zeros(Bpad, n, dtype=I, device=dev)
    mk = torch.zeros(Bpad, n, dtype=I, device=dev)
    sp[:B] = t64(s).reshape(B, n)
    mk[:B] = (t64(msk).reshape(B, n) != 0).to(I)
    M = mk != 0
    sgn, eb, mb, _ = _bf_fields(sp)
    key = 32768 - sgn + (1 - 2 * sgn) * (128 * eb + mb)
    kq = torch.where(M, key, torch.full_like(key, -1))
    kmax_all = kq.amax(dim=1)
    emp = kmax_all < 0
    attk = M & (key == kmax_all[:, None])
    sel1 = attk & (attk.cumsum(dim=1) == 1)
    mxp = (sel1.to(I) * sp).sum(dim=1)
    kmax = torch.where(emp, torch.zeros_like(kmax_all), kmax_all)
    zero, one = torch.zeros_like(sp), torch.ones_like(sp)
    xm = torch.where(M, sp, zero)
    x2m = torch.where(M, (mxp ^ 0x8000)[:, None].expand(Bpad, n), zero)
    blk, blu, dp = ba_fill(xm.reshape(-1), x2m.reshape(-1), inverse)
    dp = dp.reshape(Bpad, n)
    dk = torch.where(M, kmax[:, None] - key, zero)
    xv = t64(art["exp_tab"])[dp]
    if bool((((xv >> 15) & 1) != 0).any()):
        raise ValueError("smx: negative exp")
    eeb, emb = (xv >> 7) & 255, xv & 127
    ez = eeb == 0
    pres = M & ~ez
    E = torch.where(pres, eeb + 8, zero).amax(dim=1).clamp(min=EMIN)
    att2 = pres & (eeb + 8 == E[:, None])
    sel2 = att2 & (att2.cumsum(dim=1) == 1)
    fsel = (~att2.any(dim=1)).to(I)
    sh = torch.where(pres, E[:, None] - (eeb + 8), zero)
    shc = sh.clamp(max=16)
    pw = torch.where(pres, shl(one, shc), one)
    sq = (128 + emb) << 8
    q = torch.where(pres, sq >> shc, zero)
    rr = torch.where(pres, sq - shl(q, shc), zero)
    S = q.sum(dim=1)
    wcap = min(max(16 + ln, 23), 30)
    if bool((~emp & ((S < 1) | (S >= (1 << wcap)))).any()):
        raise ValueError("smx: S window")
    Ssafe = torch.where(emp, torch.ones_like(S), S)
    wd = _bitlen(Ssafe, 40)
    o1 = torch.ones_like(wd)
    dn_s, up_s = (wd - 16).clamp(min=0), (16 - wd).clamp(min=0)
    plo, phi, pdn, pup = shl(o1, wd - 1), shl(o1, wd), shl(o1, dn_s), shl(o1, up_s)
    u1, u2 = Ssafe - plo, phi - 1 - Ssafe
    nr = torch.where(wd > 16, Ssafe & (pdn - 1), torch.zeros_like(S))
    u16 = torch.where(wd > 16, Ssafe >> dn_s, shl(Ssafe, up_s))
    ri = u16 - 32768
    mrc, hbc = 128 + t64(art["rcp_mr"])[ri], t64(art["rcp_hb"])[ri]
    reb = 277 + hbc - E - wd
    if bool((~emp & ((reb < 1) | (reb > 254))).any()):
        raise ValueError("smx: recip exp domain")
    # rows without any participating lane: the benign constants of the reference (normalisation gated off)
    gate = lambda t, dflt: torch.where(emp, torch.full_like(t, dflt), t)
    wd, plo, phi, pdn, pup = gate(wd, 1), gate(plo, 1), gate(phi, 2), gate(pdn, 1), gate(pup, 1 << 15)
    u1, u2, nr, u16, mrc, hbc, reb = gate(u1, 0), gate(u2, 0), gate(nr, 0), gate(u16, 32768), gate(mrc, 128), gate(hbc, 1), gate(reb, 1)
    mj = (emb << 7) | (mrc[:, None] - 128)
    mo, ei = 128 + t64(art["mul_mo"])[mj], t64(art["mul_einc"])[mj]
    eo = torch.where(pres, eeb + reb[:, None] - 127 + ei, one)
    if bool(((eo < 1) | (eo > 254)).any()):
        raise ValueError("smx: out exp domain")
    p = torch.where(pres, (eo << 7) | (mo - 128), zero)
    flat = lambda t: t.reshape(-1).contiguous()
    de = [flat(t) for t in (xm, x2m, dp, dk, sel1.to(I), xv, eeb, emb, ez.to(I), _inv_or0(eeb, inverse), sh, pw, q, rr, sel2.to(I), mo, ei, eo)] + blk
    db = [kmax, mxp, E, E - EMIN, fsel, S, wd, plo, phi, pdn, pup, u1 >> 12, u1 & 4095, u2 >> 12, u2 & 4095, nr, u16, mrc, hbc, reb]
    i32 = lambda t: flat(t).to(torch.int32)
    lidx = [i32(dk), i32(dp), i32(eeb), i32(emb), i32(sh), i32(pw - 1 + rr), i32(q), i32(mj), i32(eo),
            i32(E - EMIN), i32(wd), i32(u1 >> 12), i32(u1 & 4095), i32(u2 >> 12), i32(u2 & 4095), i32(pdn - 1 + nr), i32(u16 - 32768),
            i32(reb)] + blu
    return {"B": B, "ln": ln, "n": n, "Bpad": Bpad, "lb": lb, "le": lb + ln, "spat": flat(sp), "ppat": flat(p), "mskc": flat(mk),
            "empc": emp.to(I), "de": de, "db": db, "lidx": lidx, "emf": flat(128 + emb), "mrcf": flat(mrc[:, None].expand(Bpad, n)),
            "P": p[:B].cpu().numpy().astype(np.uint16).reshape(-1)}


def smx_commit_operands(engine, wt, R, col):
    out = {}
    for name, key in (("S", "spat"), ("P", "ppat")):
        c = col(wt[key])
        out[name] = (c, engine.commit_gpu_rootonly(c, R))
    return out


def smx_prove(engine, tr, wt, T, art, ops, R, Q, col, ctx=None, strict=True):
    """p3smx::prove (p3_softmax.cuh:529-713), non-zk.  Serialised SmxProof: u32 B ln | rde[73] rdb[20] | groups | mDe |
    u32 73, yDe | yDeS yDeP yDeKM yDeMX yDeE yDeRB | mDb yDb[20] | yBF yBS | mBind yBSEL1 yBSEL2 yBQ2 | batches."""
    from .ig import Ctx
    own = ctx is None
    ctx = ctx or Ctx()
    lg = ctx.ledger
    ln, lb, le = wt["ln"], wt["lb"], wt["le"]
    if 16 + ln > T["wmax"]:
        raise ValueError("smx: tables too small (need wmax >= 16+ln)")
    tr.absorb("smx-dims", struct.pack("<III", wt["B"], ln, art["sm_emin"]))
    for name in BT_NAMES + SMX_XT:
        tr.absorb("smx-tab", T[name]["id"])
    tr.absorb("smx-msk", wt["mskc"].cpu().numpy().astype(np.uint64).tobytes())
    tr.absorb("smx-S", ops["S"][1])
    tr.absorb("smx-P", ops["P"][1])
    commit = lambda cols: commit_cols(engine, [col(t) for t in cols], R)
    CDe, CDb = commit(wt["de"]), commit(wt["db"])
    for _, root in CDe:
        tr.absorb("smx-ce", root)
    for _, root in CDb:
        tr.absorb("smx-cb", root)
    e_, b_ = (lambda nm: CDe[SM[nm]]), (lambda nm: CDb[SB[nm]])
    emf, mrcf = (col(wt["emf"]), None), (col(wt["mrcf"]), None)
    specs = [("R16", [e_("DK")]), ("EXPT", [e_("DP"), e_("EXV")]), ("R256", [e_("EEB")]), ("R128", [e_("EMB")]),
             ("SH512", [e_("SH2"), e_("PW2")]), ("RM17", [e_("PW2"), e_("RR2")]), ("R16", [e_("Q2")]),
             ("MUL7", [emf, mrcf, e_("MO3"), e_("EI3")]), ("REXP", [e_("EO3")]), ("R512", [b_("EDIF")]),
             ("WD24", [b_(nm) for nm in ("WD", "PLO", "PHI", "PDN", "PUP")]), ("R11", [b_("U1H")]), ("R12", [b_("U1L")]),
             ("R11", [b_("U2H")]), ("R12", [b_("U2L")]), ("RM8", [b_("PDN"), b_("NR")]), ("RCPT", [b_("U16"), b_("MRC"), b_("HBC")]),
             ("REXP", [b_("REB")])]
    specs += [(tab, [CDe[SM_A + BA[nm]] for nm in names]) for tab, names in BA_LU]
    for i, (tab, W) in enumerate(specs):
        ent = {"W": W, "idx": col(wt["lidx"][i]), "tab": T[tab]}
        if i == 7:
            ent["bind"] = claim_bind(engine, tr, lg, [e_("EMB"), b_("MRC") + (lambda pm: pm[ln:le],)])
        ctx.luq.append(ent)
    chal_vec = lambda k: [tr.chal() for _ in range(k)]
    eq = lambda z: engine.build_eq_gpu(np.array(z, dtype=np.uint64))
    claim = lambda c, z: claimc(engine, tr, lg, c[0], c[1], z)
    v = Poly.var
    # element domain: [E, S, P, MSK, de[73], KMAX row, MXP row, E row, REB row]
    zE = chal_vec(le)
    lam = _powers(tr.chal(), N_SM_DE)
    c = lambda nm: v(4 + SM[nm])
    cA = {nm: v(4 + SM_A + i) for i, nm in enumerate(BA_COLS)}
    Mv = v(3)
    KM, MX, Eb, RBv = (v(4 + NDE2 + k) for k in range(4))
    nM, MEZ = 1 - Mv, Mv * c("EZ")
    absent = 1 - Mv + MEZ
    mag = 128 * cA["E1"] + cA["M1"]
    key = 32768 - cA["S1"] + mag - 2 * cA["S1"] * mag
    shrel = c("SH2") + c("EEB") + 8 - Eb
    sqv = 256 * (128 + c("EMB"))
    eo3rel = c("EO3") + 127 - (c("EEB") + RBv + c("EI3"))
    pat = 128 * c("EO3") + c("MO3") - 128
    cons = [c("XM") - Mv * v(1), nM * c("X2M"), Mv * (MX - (32768 - 32768 * cA["S2"] + 128 * cA["E2"] + cA["M2"])),
            Mv * (KM - (key + c("DK"))), nM * c("DK"), boolc(c("SEL1")), c("SEL1") * nM, c("SEL1") * c("DK"),
            c("SEL1") * (c("XM") - MX), c("EXV") - (128 * c("EEB") + c("EMB")), boolc(c("EZ")), c("EZ") * c("EEB"),
            c("EEB") * c("EZI") - (1 - c("EZ")), c("SH2") * absent, Mv * shrel - MEZ * shrel,
            c("Q2") * c("PW2") + c("RR2") - (Mv * sqv - MEZ * sqv), boolc(c("SEL2")), c("SEL2") * c("SH2"), c("SEL2") * absent,
            Mv * eo3rel - MEZ * eo3rel, absent * (c("EO3") - 1), v(2) - (Mv * pat - MEZ * pat)]
    cons += ba_constraints(cA, c("XM"), c("X2M"), c("DP"))
    terms, konst = zc_terms(cons, lam)
    cols = [eq(zE), ops["S"][0], ops["P"][0], col(wt["mskc"])] + [t for t, _ in CDe] + \
        [engine.bcast_rows(b_(nm)[0], ln) for nm in ("KMAX", "MXP", "E", "REB")]
    rE, mDe, _ = engine.sc_prove_zc(tr, "smx-scE", cols, terms, konst)
    rE = [int(x) for x in rE]
    yDeS, yDeP = claim(ops["S"], rE), claim(ops["P"], rE)
    yDe = [claim(cd, rE) for cd in CDe]
    rb = rE[ln:le]
    yDeR = [claim(b_(nm), rb) for nm in ("KMAX", "MXP", "E", "REB")]
    # row domain: [E, EMP, db[20]]
    zB = chal_vec(lb)
    lamB = _powers(tr.chal(), 7)
    r_ = lambda nm: v(2 + SB[nm])
    nE = 1 - v(1)
    consB = [boolc(r_("FSEL")), r_("FSEL") * r_("EDIF"), r_("E") - (art["sm_emin"] + r_("EDIF")),
             nE * (r_("S") - r_("PLO") - (4096 * r_("U1H") + r_("U1L"))), nE * (r_("PHI") - 1 - r_("S") - (4096 * r_("U2H") + r_("U2L"))),
             nE * (r_("U16") * r_("PDN") + r_("NR") - r_("S") * r_("PUP")), nE * (r_("REB") + r_("E") + r_("WD") - (277 + r_("HBC")))]
    terms, konst = zc_terms(consB, lamB)
    rB, mDb, _ = engine.sc_prove_zc(tr, "smx-scB", [eq(zB), col(wt["empc"])] + [t for t, _ in CDb], terms, konst)
    rB = [int(x) for x in rB]
    yDb = [claim(cd, rB) for cd in CDb]
    # row binding: sum_j SEL1 = 1 - EMP, sum_j SEL2 = 1 - FSEL, sum_j Q2 = S
    z2 = chal_vec(lb)
    yBF, yBS = claim(b_("FSEL"), z2), claim(b_("S"), z2)
    lam3 = [tr.chal(), tr.chal(), tr.chal()]
    terms, konst = zc_terms([v(1), v(2), v(3)], lam3)
    rS, mBind, _ = engine.sc_prove_zc(tr, "smx-scS", [engine.bcast_rows(eq(z2), ln), e_("SEL1")[0], e_("SEL2")[0], e_("Q2")[0]], terms, konst)
    rS = [int(x) for x in rS]
    yB = [claim(e_("SEL1"), rS), claim(e_("SEL2"), rS), claim(e_("Q2"), rS)]
    lug, batches = _tail(engine, tr, ctx, R, Q, "smx-bo", strict) if own else ([], [])
    sl, sb = _ser_tail(lug, batches)
    out = struct.pack("<II", wt["B"], ln) + b"".join(r for cd in (CDe, CDb) for _, r in cd) + sl
    out += _msgs(mDe) + struct.pack("<I", len(yDe)) + _u64(yDe) + _u64([yDeS, yDeP] + yDeR) + _msgs(mDb) + _u64(yDb)
    out += _u64([yBF, yBS]) + _msgs(mBind) + _u64(yB)
    return out + sb


# ---------------------------------------------------------------------------------- composed fp8 transformer layer (p3tf)
class TfConfig:
    """p3tf::Config (p3_transformer.cuh:93-127): power-of-two shapes; attention instances a = b * nh + h."""

    def __init__(self, seq, d, nh, dh, dff, batch=1):
        self.seq, self.d, self.nh, self.dh, self.dff, self.batch = seq, d, nh, dh, dff, batch
        lg = lambda x: x.bit_length() - 1
        self.lseq, self.ld, self.ldh, self.ldff, self.lnh, self.lbb = lg(seq), lg(d), lg(dh), lg(dff), lg(nh), lg(batch)
        if any((1 << l) != x for l, x in ((self.lseq, seq), (self.ld, d), (self.ldh, dh), (self.ldff, dff), (self.lnh, nh),
                                          (self.lbb, batch))) or nh * dh != d:
            raise ValueError("tf: config must be pow2")
        self.T, self.lT, self.A = seq * batch, self.lseq + self.lbb, batch * nh
        A = self.A
        self.nmm, self.nqn = 7 + 2 * A, 4 + 4 * A
        self.mmWQ, self.mmWK, self.mmWV = 0, 1, 2
        self.mmQK, self.mmPV = (lambda a: 3 + a), (lambda a: 3 + A + a)
        self.mmWO, self.mmWG, self.mmWU, self.mmWD = 3 + 2 * A, 4 + 2 * A, 5 + 2 * A, 6 + 2 * A
        self.qnH1 = 0
        self.qnRQ, self.qnRK = (lambda a: 1 + 2 * a), (lambda a: 2 + 2 * a)
        self.qnPB, self.qnVT = (lambda a: 1 + 2 * A + a), (lambda a: 1 + 3 * A + a)
        self.qnAT, self.qnH2, self.qnSW = 1 + 4 * A, 2 + 4 * A, 3 + 4 * A

    def dims(self):
        return (self.seq, self.d, self.nh, self.dh, self.dff, self.batch)


W_Q, W_K, W_V, W_O, W_G, W_U, W_D = range(7)


def tf_tables(art, smx_wmax=23):
    """p3tf::build_tables (p3_transformer.cuh:506-520)."""
    from . import hwl
    return {"hw": hwl.build_tables(), "rms": rms_tables(art), "qnt": qnt_tables(art), "rope": rope_tables(art),
            "smx": smx_tables(art, smx_wmax), "bfa": bfa_tables(), "swg": swg_tables(art)}


def tf_build_witness(c, x0, W, art, device="cpu", engine=None):
    """p3tf::build_witness (p3_transformer.cuh:238-499): the layer is computed by the gadget replays themselves, each output
    feeding the next input.  x0: T*d bf16 patterns; W: {"w": [(codes N*K uint8, scales N uint32)] * 7, "g1", "g2" (d bf16),
    "cos", "sin" (seq * dh/2 bf16)}.  With ``engine`` (the CUDA prover) the matmul replays run in its witness kernel."""
    from . import hwl
    inverse = None if engine is None else (lambda t: engine.inv_all_add(t.contiguous(), 0))
    kw = {"device": device, "inverse": inverse}
    u16 = lambda a: np.ascontiguousarray(a, dtype=np.uint16)
    seq, d, dh, dff, T, A, nh = c.seq, c.d, c.dh, c.dff, c.T, c.A, c.nh
    w = {"cfg": c, "qn": [None] * c.nqn, "mm": [None] * c.nmm, "rp": [None] * (2 * A), "sm": [None] * A, "mmY": [None] * c.nmm}

    def matmul(i, B, K, N, xq, wcodes, wscales):
        args = (B, K, N, xq["C"], wcodes, xq["S"], wscales)
        w["mm"][i] = hwl.gen_witness_dev(engine, *args) if engine is not None else hwl.gen_witness(*args, device=device)
        w["mmY"][i] = w["mm"][i]["Y"]
        return w["mmY"][i]

    w["rms"] = [rms_witness(u16(x0), W["g1"], T, art, **kw), None]
    w["qn"][c.qnH1] = qnt_witness(w["rms"][0]["Y"], T, c.ld, art, **kw)
    yq, yk, yv = (matmul(i, T, d, d, w["qn"][c.qnH1], *W["w"][wi]) for i, wi in ((c.mmWQ, W_Q), (c.mmWK, W_K), (c.mmWV, W_V)))
    mask = np.tril(np.ones((seq, seq), dtype=np.uint8)).reshape(-1)
    w["smmask"] = mask
    attn = np.zeros((T, d), dtype=np.uint16)
    head = lambda Y, b, h: Y.reshape(T, d)[b * seq:(b + 1) * seq, h * dh:(h + 1) * dh]
    for b in range(c.batch):
        for h in range(nh):
            a = b * nh + h
            w["rp"][2 * a] = rope_witness(head(yq, b, h).reshape(-1), W["cos"], W["sin"], seq, dh, art, **kw)
            w["rp"][2 * a + 1] = rope_witness(head(yk, b, h).reshape(-1), W["cos"], W["sin"], seq, dh, art, **kw)
            w["qn"][c.qnRQ(a)] = qnt_witness(w["rp"][2 * a]["OUT"], seq, c.ldh, art, **kw)
            w["qn"][c.qnRK(a)] = qnt_witness(w["rp"][2 * a + 1]["OUT"], seq, c.ldh, art, **kw)
            sc = matmul(c.mmQK(a), seq, dh, seq, w["qn"][c.qnRQ(a)], w["qn"][c.qnRK(a)]["C"], w["qn"][c.qnRK(a)]["S"])
            w["sm"][a] = smx_witness(sc, mask, seq, c.lseq, art, **kw)
            w["qn"][c.qnPB(a)] = qnt_witness(w["sm"][a]["P"], seq, c.lseq, art, **kw)
            vt = np.ascontiguousarray(head(yv, b, h).T).reshape(-1)
            w["qn"][c.qnVT(a)] = qnt_witness(vt, dh, c.lseq, art, **kw)
            pv = matmul(c.mmPV(a), seq, seq, dh, w["qn"][c.qnPB(a)], w["qn"][c.qnVT(a)]["C"], w["qn"][c.qnVT(a)]["S"])
            attn[b * seq:(b + 1) * seq, h * dh:(h + 1) * dh] = pv.reshape(seq, dh)
    w["qn"][c.qnAT] = qnt_witness(attn.reshape(-1), T, c.ld, art, **kw)
    yo = matmul(c.mmWO, T, d, d, w["qn"][c.qnAT], *W["w"][W_O])
    w["res"] = [bfa_witness(u16(x0), yo, **kw), None]
    w["rms"][1] = rms_witness(w["res"][0]["O"], W["g2"], T, art, **kw)
    w["qn"][c.qnH2] = qnt_witness(w["rms"][1]["Y"], T, c.ld, art, **kw)
    yg = matmul(c.mmWG, T, d, dff, w["qn"][c.qnH2], *W["w"][W_G])
    yu = matmul(c.mmWU, T, d, dff, w["qn"][c.qnH2], *W["w"][W_U])
    w["sw"] = swg_witness(yg, yu, art, **kw)
    w["qn"][c.qnSW] = qnt_witness(w["sw"]["M"], T, c.ldff, art, **kw)
    yd = matmul(c.mmWD, T, dff, d, w["qn"][c.qnSW], *W["w"][W_D])
    w["res"][1] = bfa_witness(w["res"][0]["O"], yd, **kw)
    w["x0"], w["out"] = u16(x0), w["res"][1]["O"]
    return w


def tf_commit_all(engine, w, R, col, x0ext=None):
    """p3tf::commit_all (p3_transformer.cuh:565-727): every chained column is committed once; producer and consumer share
    the (column, root) pair wherever they hold the same values on the same domain.  x0ext: an already committed input
    column (the previous layer's output, or the embedded input of a model)."""
    from . import hwl
    c = w["cfg"]
    A, nh = c.A, c.nh
    com = lambda t: (lambda cc: (cc, engine.commit_gpu_rootonly(cc, R)))(col(t))
    o = {"rms": [None, None], "qn": [None] * c.nqn, "mm": [None] * c.nmm, "rp": [None] * (2 * A), "sm": [None] * A, "res": [None, None],
         "Ymm": [None] * c.nmm}

    def quant(i, X):
        o["qn"][i] = {"X": X, "CODES": com(w["qn"][i]["cpat"]), "SCALES": com(w["qn"][i]["spat"])}

    def matmul(i, X, Wc, XS, WS):
        m = w["mm"][i]
        o["mm"][i] = {"X": X if X is not None else com(m["xcodes"]), "W": Wc if Wc is not None else com(m["wcodes"]), "XS": XS,
                      "WS": WS if WS is not None else com(m["wsb"])}
        o["Ymm"][i] = com(m["dob"][hwl.O_YB])

    o["rms"][0] = rms_commit_operands(engine, w["rms"][0], R, col) if x0ext is None else \
        {"X": x0ext, "G": com(w["rms"][0]["gpat"]), "Y": com(w["rms"][0]["ypat"])}
    quant(c.qnH1, o["rms"][0]["Y"])
    X1 = com(w["mm"][c.mmWQ]["xcodes"])
    for i in (c.mmWQ, c.mmWK, c.mmWV):
        matmul(i, X1, None, o["qn"][c.qnH1]["SCALES"], None)
    for a in range(A):
        for k in (0, 1):
            o["rp"][2 * a + k] = rope_commit_operands(engine, w["rp"][2 * a + k], R, col)
        quant(c.qnRQ(a), o["rp"][2 * a]["OUT"])
        quant(c.qnRK(a), o["rp"][2 * a + 1]["OUT"])
        matmul(c.mmQK(a), None, None, o["qn"][c.qnRQ(a)]["SCALES"], o["qn"][c.qnRK(a)]["SCALES"])
        o["sm"][a] = {"S": o["Ymm"][c.mmQK(a)], "P": com(w["sm"][a]["ppat"])}
        quant(c.qnPB(a), o["sm"][a]["P"])
        quant(c.qnVT(a), com(w["qn"][c.qnVT(a)]["xpat"]))
        matmul(c.mmPV(a), None, None, o["qn"][c.qnPB(a)]["SCALES"], o["qn"][c.qnVT(a)]["SCALES"])
    quant(c.qnAT, com(w["qn"][c.qnAT]["xpat"]))
    matmul(c.mmWO, None, None, o["qn"][c.qnAT]["SCALES"], None)
    o["res"][0] = {"X1": o["rms"][0]["X"], "X2": o["Ymm"][c.mmWO], "OUT": com(w["res"][0]["opat"])}
    o["rms"][1] = {"X": o["res"][0]["OUT"], "G": com(w["rms"][1]["gpat"]), "Y": com(w["rms"][1]["ypat"])}
    quant(c.qnH2, o["rms"][1]["Y"])
    X2 = com(w["mm"][c.mmWG]["xcodes"])
    for i in (c.mmWG, c.mmWU):
        matmul(i, X2, None, o["qn"][c.qnH2]["SCALES"], None)
    o["sw"] = {"GATE": o["Ymm"][c.mmWG], "UP": o["Ymm"][c.mmWU], "M": com(w["sw"]["mpat"])}
    quant(c.qnSW, o["sw"]["M"])
    matmul(c.mmWD, None, None, o["qn"][c.qnSW]["SCALES"], None)
    o["res"][1] = {"X1": o["res"][0]["OUT"], "X2": o["Ymm"][c.mmWD], "OUT": com(w["res"][1]["opat"])}
    return o


def tf_weight_roots(engine, c, W, R, col):
    """p3tf::weight_roots (p3_transformer.cuh:732-752): the public weight-side commitments, from the weights and the canonical
    padding alone: 7 code roots, 7 scale roots, g1, g2."""
    from . import hwl
    roots_c, roots_s = [], []
    for codes, scales in W["w"]:
        N = len(scales)
        K = len(codes) // N
        dd = hwl.Dims(c.T, K, N)
        wc = np.zeros((dd.Npad, dd.Kpad), dtype=np.uint64)
        wc[:N, :K] = np.asarray(codes, dtype=np.uint64).reshape(N, K)
        ws = np.zeros(dd.Npad, dtype=np.uint64)
        ws[:N] = np.asarray(scales, dtype=np.uint64)
        roots_c.append(engine.commit_gpu_rootonly(engine.upload(wc.reshape(-1)), R))
        roots_s.append(engine.commit_gpu_rootonly(engine.upload(ws), R))
    g = [engine.commit_gpu_rootonly(engine.upload(np.asarray(W[k], dtype=np.uint64)), R) for k in ("g1", "g2")]
    return roots_c + roots_s + g


def tf_prove_subs(engine, tr, w, o, T, art, R, Q, col, ctx, strict=True):
    """p3tf::prove_subs (p3_transformer.cuh:826-925): the layer header and every gadget sub-proof in fixed order on the shared
    transcript, ledger and lookup queue.  Returns the serialised sub-proofs in proving order."""
    from . import hwl
    c = w["cfg"]
    A = c.A
    tr.absorb("tf-dims", struct.pack("<6I", *c.dims()))
    subs = []
    rms = lambda i: subs.append(rms_prove(engine, tr, w["rms"][i], T["rms"], art, o["rms"][i], R, Q, col, ctx, strict))
    qn = lambda i: subs.append(qnt_prove(engine, tr, w["qn"][i], T["qnt"], o["qn"][i], R, Q, col, ctx, strict))
    mm = lambda i: subs.append(hwl.prove(engine, tr, w["mm"][i], T["hw"], o["mm"][i], R, Q, col, w["mmY"][i], ctx, strict))
    rms(0)
    qn(c.qnH1)
    for i in (c.mmWQ, c.mmWK, c.mmWV):
        mm(i)
    for a in range(A):
        for k in (0, 1):
            subs.append(rope_prove(engine, tr, w["rp"][2 * a + k], T["rope"], o["rp"][2 * a + k], R, Q, col, ctx, strict))
        qn(c.qnRQ(a))
        qn(c.qnRK(a))
        mm(c.mmQK(a))
        subs.append(smx_prove(engine, tr, w["sm"][a], T["smx"], art, o["sm"][a], R, Q, col, ctx, strict))
        qn(c.qnPB(a))
        qn(c.qnVT(a))
        mm(c.mmPV(a))
    qn(c.qnAT)
    mm(c.mmWO)
    subs.append(bfa_prove(engine, tr, w["res"][0], T["bfa"], o["res"][0], R, Q, col, ctx, strict))
    rms(1)
    qn(c.qnH2)
    mm(c.mmWG)
    mm(c.mmWU)
    subs.append(swg_prove(engine, tr, w["sw"], T["swg"], o["sw"], R, Q, col, ctx, strict))
    qn(c.qnSW)
    mm(c.mmWD)
    subs.append(bfa_prove(engine, tr, w["res"][1], T["bfa"], o["res"][1], R, Q, col, ctx, strict))
    return subs


class Seams:
    """Seam claims on the shared ledger: every claimed value is absorbed like any opening claim and recorded in order."""

    def __init__(self, engine, tr, ledger, strict, who):
        self.engine, self.tr, self.lg, self.strict, self.who, self.vals = engine, tr, ledger, strict, who, []

    def chal_vec(self, n):
        return [self.tr.chal() for _ in range(n)]

    def cl(self, cr, z):
        y = claimc(self.engine, self.tr, self.lg, cr[0], cr[1], z)
        self.vals.append(y)
        return y

    def pair(self, Ac, zA, Bc, zB, what):
        if self.cl(Ac, zA) != self.cl(Bc, zB) and self.strict:
            raise ValueError("%s: seam mismatch: %s" % (self.who, what))

    def codes(self, Cc, Xc, ldr, lk, lb, what):
        """quantiser codes against the padded matmul operand: restriction, then one zero claim per padding subcube"""
        z = self.chal_vec(ldr + lb)
        self.pair(Cc, z, Xc, z[:ldr] + [0] * (lk - ldr) + z[ldr:], what)
        for t in range(ldr, lk):
            zt = self.chal_vec(t + lb)
            if self.cl(Xc, zt[:t] + [1] + [0] * (lk - t - 1) + zt[t:]) != 0 and self.strict:
                raise ValueError("%s: padding not zero: %s" % (self.who, what))


def tf_prove_seams(engine, tr, w, o, ctx, strict=True, bind_in=True, bind_out=True):
    """p3tf::prove_seams (p3_transformer.cuh:931-1006): restriction / zero-padding seams between quantiser codes and matmul
    operands, head slice / transpose / concat seams, and (single layer) the public input / output bindings.  Returns the
    seam values in order."""
    c = w["cfg"]
    nh = c.nh
    S = Seams(engine, tr, ctx.ledger, strict, "tf")
    bits = lambda v, n: [(v >> i) & 1 for i in range(n)]
    slice_pt = lambda z, li, h, b: z[:li] + bits(h, c.lnh) + z[li:] + bits(b, c.lbb)
    lk_of = lambda i: w["mm"][i]["d"].Kpad.bit_length() - 1
    lkH1, lkQK, lkPV, lkSW = lk_of(c.mmWQ), lk_of(c.mmQK(0)), lk_of(c.mmPV(0)), lk_of(c.mmWD)
    if bind_in:
        S.cl(o["rms"][0]["X"], S.chal_vec(c.ld + c.lT))
    S.codes(o["qn"][c.qnH1]["CODES"], o["mm"][c.mmWQ]["X"], c.ld, lkH1, c.lT, "h1 codes")
    for b in range(c.batch):
        for h in range(nh):
            a = b * nh + h
            z = S.chal_vec(c.ldh + c.lseq)
            S.pair(o["rp"][2 * a]["Q"], z, o["Ymm"][c.mmWQ], slice_pt(z, c.ldh, h, b), "rope-q slice")
            z = S.chal_vec(c.ldh + c.lseq)
            S.pair(o["rp"][2 * a + 1]["Q"], z, o["Ymm"][c.mmWK], slice_pt(z, c.ldh, h, b), "rope-k slice")
            S.codes(o["qn"][c.qnRQ(a)]["CODES"], o["mm"][c.mmQK(a)]["X"], c.ldh, lkQK, c.lseq, "qk x codes")
            S.codes(o["qn"][c.qnRK(a)]["CODES"], o["mm"][c.mmQK(a)]["W"], c.ldh, lkQK, c.lseq, "qk w codes")
            z = S.chal_vec(c.lseq + c.ldh)
            zt = z[c.lseq:] + bits(h, c.lnh) + z[:c.lseq] + bits(b, c.lbb)
            S.pair(o["qn"][c.qnVT(a)]["X"], z, o["Ymm"][c.mmWV], zt, "v^T transpose")
            S.codes(o["qn"][c.qnPB(a)]["CODES"], o["mm"][c.mmPV(a)]["X"], c.lseq, lkPV, c.lseq, "pv x codes")
            S.codes(o["qn"][c.qnVT(a)]["CODES"], o["mm"][c.mmPV(a)]["W"], c.lseq, lkPV, c.ldh, "pv w codes")
            z = S.chal_vec(c.ldh + c.lseq)
            S.pair(o["qn"][c.qnAT]["X"], slice_pt(z, c.ldh, h, b), o["Ymm"][c.mmPV(a)], z, "concat half")
    S.codes(o["qn"][c.qnAT]["CODES"], o["mm"][c.mmWO]["X"], c.ld, lkH1, c.lT, "attn codes")
    S.codes(o["qn"][c.qnH2]["CODES"], o["mm"][c.mmWG]["X"], c.ld, lkH1, c.lT, "h2 codes")
    S.codes(o["qn"][c.qnSW]["CODES"], o["mm"][c.mmWD]["X"], c.ldff, lkSW, c.lT, "swiglu codes")
    if bind_out:
        S.cl(o["res"][1]["OUT"], S.chal_vec(c.ld + c.lT))
    return S.vals


def tf_serialize(w, o, subs, lug, seam, batches):
    """Serialised TfProof: 6 x u32 dims | length-prefixed sub-proofs in proving order | roots rX0 rRmsY[2] rCodes[] rScales[]
    rMX[] rMW[] rRopeQ[] rRopeO[] rSmP[] rVtX[] rAtX rRes1 rSwM rOut | per matmul u32 count + bf16 outputs | groups |
    u32 count + seam values | batches."""
    c = w["cfg"]
    root = lambda cr: cr[1]
    out = struct.pack("<6I", *c.dims()) + b"".join(_blob(s) for s in subs)
    out += root(o["rms"][0]["X"]) + root(o["rms"][0]["Y"]) + root(o["rms"][1]["Y"])
    out += b"".join(root(q["CODES"]) for q in o["qn"]) + b"".join(root(q["SCALES"]) for q in o["qn"])
    out += b"".join(root(m["X"]) for m in o["mm"]) + b"".join(root(m["W"]) for m in o["mm"])
    out += b"".join(root(r["Q"]) for r in o["rp"]) + b"".join(root(r["OUT"]) for r in o["rp"])
    out += b"".join(root(s["P"]) for s in o["sm"]) + b"".join(root(o["qn"][c.qnVT(a)]["X"]) for a in range(c.A))
    out += root(o["qn"][c.qnAT]["X"]) + root(o["res"][0]["OUT"]) + root(o["sw"]["M"]) + root(o["res"][1]["OUT"])
    for y in w["mmY"]:
        out += struct.pack("<I", len(y)) + np.ascontiguousarray(y, dtype=np.uint16).tobytes()
    sl, sb = _ser_tail(lug, batches)
    return out + sl + struct.pack("<I", len(seam)) + _u64(seam) + sb


def tf_prove(engine, tr, w, o, T, art, R, Q, col, strict=True, stages=None):
    """p3tf::prove (p3_transformer.cuh:1011-1037), non-zk: all sub-proofs in fixed order on one transcript with one ledger,
    one merged-lookup flush, the composition seams with both public I/O bindings, one batched opening per size class.
    stages: optional dict that receives the wall-clock seconds of the four stages (the engine calls synchronise)."""
    import time
    from .ig import Ctx
    ctx = Ctx()
    t0 = time.perf_counter()
    subs = tf_prove_subs(engine, tr, w, o, T, art, R, Q, col, ctx, strict)
    t1 = time.perf_counter()
    lug = lu_flush(engine, tr, ctx.luq, ctx.ledger, R, strict)
    t2 = time.perf_counter()
    seam = tf_prove_seams(engine, tr, w, o, ctx, strict, True, True)
    t3 = time.perf_counter()
    batches = [engine.prove_class(tr, np.stack(k[1]), k[2], R, Q, "tf-bo%d" % i) for i, k in enumerate(ctx.ledger.cls)]
    if stages is not None:
        stages.update(subs_s=t1 - t0, lookups_s=t2 - t1, seams_s=t3 - t2, openings_s=time.perf_counter() - t3,
                      lookup_groups=len(lug), opening_classes=len(batches))
    return tf_serialize(w, o, subs, lug, seam, batches)


# ---------------------------------------------------------------------------------- multi-layer model (p3mdl)
def mdl_build_witness(c, ids, MW, art, device="cpu", engine=None):
    """p3mdl::build_model_witness (p3_model.cuh:169-229): embedding gather at the public token ids, the chained layers, final
    RMSNorm, quantise, LM-head fp8 matmul -> logits.  MW: {"vocab", "emb" (vocab*d bf16), "layers": [layer weights as for
    tf_build_witness], "gF" (d bf16), "wh": (codes vocab*d uint8, scales vocab uint32)}."""
    from . import hwl
    V, d, T = MW["vocab"], c.d, c.T
    if V & (V - 1):
        raise ValueError("mdl: vocab must be pow2")
    ids = np.asarray(ids, dtype=np.int64)
    if len(ids) != T or (ids >= V).any():
        raise ValueError("mdl: token ids")
    inverse = None if engine is None else (lambda t: engine.inv_all_add(t.contiguous(), 0))
    kw = {"device": device, "inverse": inverse}
    x0 = np.asarray(MW["emb"], dtype=np.uint16).reshape(V, d)[ids].reshape(-1)
    w = {"cfg": c, "vocab": V, "ids": ids.astype(np.uint32), "x0": x0, "lay": []}
    xi = x0
    for LW in MW["layers"]:
        w["lay"].append(tf_build_witness(c, xi, LW, art, device, engine))
        xi = w["lay"][-1]["out"]
    w["rmsF"] = rms_witness(xi, MW["gF"], T, art, **kw)
    w["qnF"] = qnt_witness(w["rmsF"]["Y"], T, c.ld, art, **kw)
    args = (T, d, V, w["qnF"]["C"], MW["wh"][0], w["qnF"]["S"], MW["wh"][1])
    w["mmH"] = hwl.gen_witness_dev(engine, *args) if engine is not None else hwl.gen_witness(*args, device=device)
    w["logits"] = w["mmH"]["Y"]
    return w


def mdl_commit(engine, w, MW, R, col):
    """p3mdl::commit_model (p3_model.cuh:240-296): embedding table, embedded input, the layers chained through shared
    commitments (layer i + 1's input column is layer i's output column), the head."""
    from . import hwl
    c = w["cfg"]
    com = lambda t: (lambda cc: (cc, engine.commit_gpu_rootonly(cc, R)))(col(t))
    up = lambda a: com(torch.as_tensor(np.asarray(a).astype(np.int64)))
    o = {"E": up(MW["emb"]), "X0": up(w["x0"]), "lay": []}
    for li, wl in enumerate(w["lay"]):
        o["lay"].append(tf_commit_all(engine, wl, R, col, o["X0"] if li == 0 else o["lay"][li - 1]["res"][1]["OUT"]))
    o["rmsF"] = {"X": o["lay"][-1]["res"][1]["OUT"], "G": com(w["rmsF"]["gpat"]), "Y": com(w["rmsF"]["ypat"])}
    o["qnF"] = {"X": o["rmsF"]["Y"], "CODES": com(w["qnF"]["cpat"]), "SCALES": com(w["qnF"]["spat"])}
    o["mmH"] = {"X": com(w["mmH"]["xcodes"]), "W": com(w["mmH"]["wcodes"]), "XS": o["qnF"]["SCALES"], "WS": com(w["mmH"]["wsb"])}
    o["YH"] = com(w["mmH"]["dob"][hwl.O_YB])
    return o


def mdl_roots(engine, c, MW, R, col):
    """p3mdl::model_roots (p3_model.cuh:306-327): embedding, final gain, head codes / scales, then 16 roots per layer."""
    from . import hwl
    up = lambda a: engine.commit_gpu_rootonly(engine.upload(np.asarray(a, dtype=np.uint64)), R)
    V = MW["vocab"]
    dd = hwl.Dims(c.T, c.d, V)
    wc = np.zeros((dd.Npad, dd.Kpad), dtype=np.uint64)
    wc[:V, :c.d] = np.asarray(MW["wh"][0], dtype=np.uint64).reshape(V, c.d)
    ws = np.zeros(dd.Npad, dtype=np.uint64)
    ws[:V] = np.asarray(MW["wh"][1], dtype=np.uint64)
    roots = [up(MW["emb"]), up(MW["gF"]), up(wc.reshape(-1)), up(ws)]
    for LW in MW["layers"]:
        roots += tf_weight_roots(engine, c, LW, R, col)
    return roots


def mdl_prove(engine, tr, w, o, T, art, R, Q, col, strict=True):
    """p3mdl::prove_model (p3_model.cuh:346-448), non-zk: every layer's sub-proofs and the head's on one transcript, ONE
    merged-lookup flush, per-layer seams without public bindings, the embedding gather seams, the head seams and the public
    logits binding, ONE batched opening per size class.  Serialised MdlProof: u32 nlayers vocab seq d batch | per layer
    u32 len + TfProof | rEmb | u32 len + rmsF, qnF, mmH | rRmsFY rCodesF rScalesF rMXH rMWH | u32 count + logits |
    u32 count + seam values | groups | batches."""
    from . import hwl
    from .ig import Ctx
    c = w["cfg"]
    V = w["vocab"]
    lv = V.bit_length() - 1
    ctx = Ctx()
    tr.absorb("mdl-dims", struct.pack("<8I", len(w["lay"]), V, *c.dims()))
    tr.absorb("mdl-ids", np.ascontiguousarray(w["ids"], dtype=np.uint32).tobytes())
    tr.absorb("mdl-emb", o["E"][1])
    lay_subs = [tf_prove_subs(engine, tr, wl, ol, T, art, R, Q, col, ctx, strict) for wl, ol in zip(w["lay"], o["lay"])]
    head = [rms_prove(engine, tr, w["rmsF"], T["rms"], art, o["rmsF"], R, Q, col, ctx, strict),
            qnt_prove(engine, tr, w["qnF"], T["qnt"], o["qnF"], R, Q, col, ctx, strict),
            hwl.prove(engine, tr, w["mmH"], T["hw"], o["mmH"], R, Q, col, w["logits"], ctx, strict)]
    lug = lu_flush(engine, tr, ctx.luq, ctx.ledger, R, strict)
    lay_seams = [tf_prove_seams(engine, tr, wl, ol, ctx, strict, False, False) for wl, ol in zip(w["lay"], o["lay"])]
    S = Seams(engine, tr, ctx.ledger, strict, "mdl")
    bits = lambda v, n: [(int(v) >> i) & 1 for i in range(n)]
    for t in range(c.T):
        z = S.chal_vec(c.ld)
        S.pair(o["X0"], z + bits(t, c.lT), o["E"], z + bits(w["ids"][t], lv), "embedding gather")
    lkH = w["mmH"]["d"].Kpad.bit_length() - 1
    S.codes(o["qnF"]["CODES"], o["mmH"]["X"], c.ld, lkH, c.lT, "head codes")
    S.cl(o["YH"], S.chal_vec(lv + c.lT))
    batches = [engine.prove_class(tr, np.stack(k[1]), k[2], R, Q, "tf-bo%d" % i) for i, k in enumerate(ctx.ledger.cls)]
    out = struct.pack("<5I", len(w["lay"]), V, c.seq, c.d, c.batch)
    for wl, ol, subs, seam in zip(w["lay"], o["lay"], lay_subs, lay_seams):
        out += _blob(tf_serialize(wl, ol, subs, [], seam, []))
    out += o["E"][1] + b"".join(_blob(h) for h in head)
    out += o["rmsF"]["Y"][1] + o["qnF"]["CODES"][1] + o["qnF"]["SCALES"][1] + o["mmH"]["X"][1] + o["mmH"]["W"][1]
    out += struct.pack("<I", len(w["logits"])) + np.ascontiguousarray(w["logits"], dtype=np.uint16).tobytes()
    sl, sb = _ser_tail(lug, batches)
    return out + struct.pack("<I", len(S.vals)) + _u64(S.vals) + sl + sb
