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

from .p3 import GL_P, claimc, lu_flush, make_table


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
    """Bind callback of a lookup whose virtual key columns are affine in committed columns: claim those columns at the
    lookup point (absorbed like any claim); the values ride in the proof as the member's extra slots."""
    def bind(pm, _yv):
        claims, extra = [], []
        for c, root in cols:
            y = engine.eval_h_gpu(c, np.ascontiguousarray(pm, dtype=np.uint64))
            tr.absorb("hwl-y", struct.pack("<Q", y))
            claims.append((c, root, np.ascontiguousarray(pm, dtype=np.uint64), y))
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
    C = [(c, engine.commit_gpu_rootonly(c, R)) for c in (col(t) for t in wt["ws"])]
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
