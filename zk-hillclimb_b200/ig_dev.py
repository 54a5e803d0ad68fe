"""Witness chain of the integer decoder layer on the GPU (torch int64 tensors carrying the field's uint64 bit
patterns): the same integer replays as ig.py's numpy functions (p3itf::build_witness and the gadgets'
gen_witness, zkllm-src/p3_int_layer.cuh:182-318, p3_int_gadgets.cuh), so that no witness column crosses PCIe and
the host does no O(N) work.  Matrix products (the seven weight matmuls and the per-head score and attention-output
products) run in the library's exact integer kernel (zkh_ig_matmul, strided views: no gathers, no index arrays);
the element-wise replays are integer tensor arithmetic.  Every function returns the same dictionary / tuple layout
as its numpy twin with device tensors in place of arrays; index arrays are int32 tensors holding uint32 values.
"""
import numpy as np
import torch

from . import ig

P_S = -(1 << 32) + 1          # the field modulus as a signed 64-bit pattern (p - 2^64)
ABND = ig.ABND


def lift(x):
    """signed int64 tensor -> field elements (uint64 bit patterns in int64)."""
    return torch.where(x < 0, x + P_S, x)


def sig(v):
    """field elements -> signed int64 (elements above p/2 have the top bit set)."""
    return torch.where(v < 0, v - P_S, v)


def _u32(x):
    return x.reshape(-1).to(torch.int32)


def dev(a, device):
    """numpy (uint64 field elements or integer tables) -> device tensor with the same bits.  A torch int32 tensor (the
    signed values, see pin_inputs) is copied as it is and lifted on the device: half the bytes over PCIe, and from
    pinned memory the copy needs no staging."""
    if isinstance(a, torch.Tensor):
        t = a.to(device, non_blocking=True)
        return lift(t.to(torch.int64)) if t.dtype == torch.int32 else t
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint64:
        return torch.from_numpy(a.view(np.int64)).to(device)
    return torch.from_numpy(a).to(device)


def pin_inputs(x0, Wt):
    """The layer's inputs (field-lifted numpy columns as ig.random_layer_inputs returns them) as signed int32 tensors in
    pinned host memory, the form a weight loader would keep them in: (x0, weights) for itf_build_witness."""
    def pin(a):
        a = np.ascontiguousarray(a)
        if a.dtype == np.uint64:
            a = np.where(a >> np.uint64(63), a + np.uint64(0xFFFFFFFF), a).view(np.int64)
        t = torch.from_numpy(a.astype(np.int32))
        return t.pin_memory() if torch.cuda.is_available() else t
    return pin(x0), {"w": [pin(x) for x in Wt["w"]], "g1": pin(Wt["g1"]), "g2": pin(Wt["g2"]), "ct": Wt["ct"], "st": Wt["st"]}


def irs_witness(acc, sf, rng):
    a = sig(acc)
    H = 1 << (sf - 1)
    y = (a + H) >> sf
    rem = (a + H) - (y << sf)
    win = (1 << 19) if rng == 1 else (1 << 15)
    if rng and bool(((y < -win) | (y >= win)).any()):
        raise ValueError("irs: y out of range (data too large)")
    L = [rem & 0xFFFF] + ([rem >> 16] if sf > 16 else [])
    return lift(y), L, [_u32(l) for l in L], (_u32(y + win) if rng else None)


def iadd_witness(a, b):
    o = sig(a) + sig(b)
    if bool(((o < -ABND) | (o >= ABND)).any()):
        raise ValueError("iadd: out of range")
    return lift(o), _u32(o + ABND)


def iswg_witness(g, u, silu_col):
    gv, uv = sig(g), sig(u)
    if bool(((gv < -ABND) | (gv >= ABND)).any()):
        raise ValueError("iswg: G out of range")
    sil = silu_col[gv + ABND]                    # the table column is passed already signed
    m64 = sil * uv
    mo = (m64 + (1 << 15)) >> 16
    rem = (m64 + (1 << 15)) - (mo << 16)
    if bool(((mo < -ABND) | (mo >= ABND)).any()):
        raise ValueError("iswg: M out of range")
    return lift(sil), rem, lift(mo), _u32(gv + ABND), _u32(rem), _u32(mo + ABND)


def rope_pub_cols(ct, st, lseq, ldh, ld, le, device):
    u = torch.arange(1 << le, dtype=torch.int64, device=device)
    j, t = u & ((1 << ld) - 1), u >> ld
    s = t & ((1 << lseq) - 1)
    jj = j & ((1 << ldh) - 1)
    hb = (jj >> (ldh - 1)) & 1
    ti = s * (1 << (ldh - 1)) + (jj & ((1 << (ldh - 1)) - 1))
    ct, st = ct.reshape(-1).to(torch.int64), st.reshape(-1).to(torch.int64)
    return ct[ti], torch.where(hb == 1, st[ti], -st[ti])


def irope_witness(q, ct, st, lseq, ldh, lT, ld):
    le, fb = lT + ld, ldh - 1
    C_, S2 = rope_pub_cols(ct, st, lseq, ldh, ld, le, q.device)
    qv = sig(q)
    qf = qv.view(-1, 2, 1 << fb).flip(1).reshape(-1)
    y64 = qv * C_ + qf * S2
    Y = (y64 + (1 << 13)) >> 14
    rem = (y64 + (1 << 13)) - (Y << 14)
    if bool(((Y < -ABND) | (Y >= ABND)).any()):
        raise ValueError("irope: y out of range")
    return lift(Y), rem, _u32(rem & 0x3FFF), _u32(Y + ABND), C_, S2


def irms_witness(x, g, isq_col, lT, ld):
    B, d = 1 << lT, 1 << ld
    xv = sig(x).reshape(B, d)
    gv = sig(g)
    M = ig.CEPS + (xv * xv).sum(dim=1)
    e = torch.zeros(B, dtype=torch.int64, device=x.device)
    while True:
        big = (M >> (2 * e)) >= (1 << 16)
        if not bool(big.any()):
            break
        e = e + big.to(torch.int64)
    m = M >> (2 * e)
    one = torch.ones_like(e)
    p4, p2 = one << (2 * e), one << e
    h2 = torch.where(e > 0, one << torch.clamp(e - 1, min=0), torch.zeros_like(e))
    r4 = M - m * p4
    d4 = p4 - 1 - r4
    RP = isq_col[m]
    Rr = (RP + h2) >> e
    r2 = RP + h2 - (Rr << e)
    d2 = p2 - 1 - r2
    db = [None] * ig.NDB
    db[ig.B_M], db[ig.B_MM], db[ig.B_MS] = M, m, m - (1 << 14)
    db[ig.B_P4], db[ig.B_P2], db[ig.B_H2], db[ig.B_RP] = p4, p2, h2, RP
    db[ig.B_L40], db[ig.B_L41], db[ig.B_L42] = r4 & 0xFFFF, (r4 >> 16) & 0xFFFF, r4 >> 32
    db[ig.B_D40], db[ig.B_D41], db[ig.B_D42] = d4 & 0xFFFF, (d4 >> 16) & 0xFFFF, d4 >> 32
    db[ig.B_R], db[ig.B_L20], db[ig.B_D20] = Rr, r2, d2
    db[ig.B_LR0], db[ig.B_LR1] = Rr & 0xFFFF, Rr >> 16
    w64 = Rr[:, None] * gv[None, :]
    Wv = (w64 + (1 << 15)) >> 16
    remW = (w64 + (1 << 15)) - (Wv << 16)
    if bool(((Wv < -ABND) | (Wv >= ABND)).any()):
        raise ValueError("irms: W out of range")
    y64 = Wv * xv
    Yv = (y64 + (1 << 15)) >> 16
    remY = (y64 + (1 << 15)) - (Yv << 16)
    if bool(((Yv < -ABND) | (Yv >= ABND)).any()):
        raise ValueError("irms: Y out of range")
    idxL = [_u32(db[c] & 0xFFFF) if c in (ig.B_L20, ig.B_D20) else _u32(db[c]) for c in
            (ig.B_L40, ig.B_L41, ig.B_L42, ig.B_D40, ig.B_D41, ig.B_D42, ig.B_L20, ig.B_D20, ig.B_LR0)]
    return {"db": [lift(c) for c in db], "de": [lift(Wv.reshape(-1)), lift(remW.reshape(-1)), lift(remY.reshape(-1))],
            "y": lift(Yv.reshape(-1)), "idxE4": _u32(e), "idxM16": _u32(m), "idxMS": _u32(m - (1 << 14)), "idxISQ": _u32(m),
            "idxL": idxL, "idxLR1": _u32(Rr >> 16), "idxRW": _u32(remW), "idxW": _u32(Wv + ABND), "idxRY": _u32(remY),
            "idxY": _u32(Yv + ABND)}


def ismx_witness(z, expt_col, la, lseq):
    seq, NR = 1 << lseq, 1 << (la + lseq)
    dv = z.device
    zv = sig(z).reshape(NR, seq)
    i = (torch.arange(NR, device=dv) & (seq - 1))[:, None]
    j = torch.arange(seq, device=dv)[None, :]
    causal = j <= i
    mx = torch.where(causal, zv, torch.full_like(zv, torch.iinfo(torch.int64).min)).max(dim=1).values
    dm = torch.where(causal, mx[:, None] - zv, torch.full_like(zv, 1 << 16))
    if bool(((dm < 0) | (dm >= (1 << 17))).any()):
        raise ValueError("ismx: DM range")
    E = expt_col[dm]
    S = E.sum(dim=1)
    hit = causal & (dm == 0)
    first = hit & (torch.cumsum(hit.to(torch.int64), dim=1) == 1)
    P = torch.div((1 << 17) * E + S[:, None], 2 * S[:, None], rounding_mode="floor")
    r1 = (1 << 17) * E + S[:, None] - 2 * P * S[:, None]
    r2 = 2 * S[:, None] - 1 - r1
    flat = lambda a: a.reshape(-1).contiguous()
    xe = [first.to(torch.int64), dm, E, r1 & 0xFFFF, r1 >> 16, r2 & 0xFFFF, r2 >> 16]
    return {"xe": [lift(flat(c)) for c in xe], "xb": [lift(mx), lift(S)], "p": lift(flat(P)), "idxDM": _u32(dm),
            "idxL": [_u32(r1 & 0xFFFF), _u32(r1 >> 16), _u32(r2 & 0xFFFF), _u32(r2 >> 16)], "idxMX": _u32(mx + (1 << 15))}


def rs20_idx(v):
    s = sig(v)
    if bool(((s < -ABND) | (s >= ABND)).any()):
        raise ValueError("itf: value out of RS20")
    return _u32(s + ABND)


def itf_build_witness(c, x0, Wt, T, device="cuda:0", engine=None):
    """p3itf::build_witness on the device.  x0, Wt as for ig.itf_build_witness (host arrays, or the pinned int32 tensors of
    pin_inputs); returns the same dictionary with device tensors, plus "dev_W" = the weights / gains as device columns
    (for itf_commit_all).  engine: the Prover whose ig_matmul runs the matrix products (one is created for the device
    when none is given)."""
    ld, lT, ldff, lseq, ldh, la = c.ld, c.lT, c.ldff, c.lseq, c.ldh, c.la
    le, lef, lez = ld + lT, ldff + lT, la + 2 * lseq
    if engine is None:
        from .p3 import Prover
        dv = torch.device(device)
        engine = Prover(dv.index or 0, torch.cuda.current_stream(dv).cuda_stream)
    d = lambda a: dev(a, device)
    x0 = d(x0)
    Wd = {"w": [d(x) for x in Wt["w"]], "g1": d(Wt["g1"]), "g2": d(Wt["g2"]), "ct": d(Wt["ct"]), "st": d(Wt["st"])}
    silu, isq, expt = (sig(d(T[n]["cols"][1])) for n in ("SILU", "ISQ", "EXPT"))
    w = {"x0": x0, "dev_W": Wd}
    seq, nh, dh, dm, nb = c.seq, c.nh, c.dh, c.d, c.batch

    def mat(X, Wm, K, N):
        """(rows x K) . (K x N), both row-major columns of field-lifted integers."""
        rows = X.numel() // K
        out = torch.empty(rows * N, dtype=torch.int64, device=X.device)
        engine.ig_matmul(X, (0, 0, K, 1), Wm, (0, 0, N, 1), out, (0, 0, N, 1), 1, 1, rows, K, N)
        return out

    # the library's witness kernels (one per gadget) where the engine has them; the tensor-arithmetic functions of this
    # module otherwise (the CPU check of this chain's layouts runs those)
    irs_w, irms_w, irope_w, ismx_w, iswg_w, iadd_w, rs20 = (irs_witness, irms_witness, irope_witness, ismx_witness, iswg_witness,
                                                              iadd_witness, rs20_idx)
    if hasattr(engine, "ig_rms_witness"):
        from ._lib import ZkhError
        tab = {n: d(T[n]["cols"][1]) for n in ("SILU", "ISQ", "EXPT")}      # value columns, field-lifted

        def guarded(fn):
            def run(*a):
                try:
                    return fn(*a)
                except ZkhError as e:
                    if e.code == -4:
                        raise ValueError("itf: a witness value lies outside its gadget's range (data too large)")
                    raise
            return run

        def irms_k(x, g, _isq, lT_, ld_):
            db, de, y, irow, iel = engine.ig_rms_witness(x, g, tab["ISQ"], lT_, ld_)
            return {"db": db, "de": de, "y": y, "idxE4": irow[0], "idxM16": irow[1], "idxMS": irow[2], "idxISQ": irow[3],
                    "idxL": irow[4:13], "idxLR1": irow[13], "idxRW": iel[0], "idxW": iel[1], "idxRY": iel[2], "idxY": iel[3]}

        def ismx_k(z, _expt, la_, lseq_):
            xe, xb, p, idm, il, imx = engine.ig_softmax_witness(z, tab["EXPT"], la_, lseq_)
            return {"xe": xe, "xb": xb, "p": p, "idxDM": idm, "idxL": il, "idxMX": imx}
        irs_w = guarded(engine.irs_witness)
        irms_w, ismx_w = guarded(irms_k), guarded(ismx_k)
        irope_w = guarded(lambda q, ct, st, lseq_, ldh_, lT_, ld_: engine.ig_rope_witness(
            q, ct.reshape(-1).to(torch.int32).contiguous(), st.reshape(-1).to(torch.int32).contiguous(), lseq_, ldh_, lT_, ld_))
        iswg_w = guarded(lambda g, u, _silu: engine.ig_swiglu_witness(g, u, tab["SILU"]))
        iadd_w = guarded(engine.ig_add_witness)
        rs20 = guarded(engine.ig_rs20_index)
    w["idxW"] = [rs20(x) for x in Wd["w"]]
    w["idxG1"], w["idxG2"], w["idxX0"] = rs20(Wd["g1"]), rs20(Wd["g2"]), rs20(x0)

    w["rms1"] = irms_w(x0, Wd["g1"], isq, lT, ld)
    w["h1"] = w["rms1"]["y"]
    w["acc"] = [None] * 7
    for i in (ig.W_Q, ig.W_K, ig.W_V):
        w["acc"][i] = mat(w["h1"], Wd["w"][i], c.d, c.d)
    w["rsq"], w["rsk"], w["rsv"] = (irs_w(w["acc"][i], 16, 1) for i in (ig.W_Q, ig.W_K, ig.W_V))
    w["yq"], w["yk"], w["yv"] = w["rsq"][0], w["rsk"][0], w["rsv"][0]
    w["rpq"] = irope_w(w["yq"], Wd["ct"], Wd["st"], lseq, ldh, lT, ld)
    w["rpk"] = irope_w(w["yk"], Wd["ct"], Wd["st"], lseq, ldh, lT, ld)
    w["rq"], w["rk"] = w["rpq"][0], w["rpk"][0]
    # scores of head h, batch b (xview_qk / wview_qk / yview_qk, p3_int_layer.cuh:96-122): sc[a][i][k] = sum_j RQ[b][i][h][j] *
    # RK[b][k][h][j], a = b * nh + h; the activations are laid out (batch, position, head, lane)
    sc = torch.empty(1 << lez, dtype=torch.int64, device=device)
    engine.ig_matmul(w["rq"], (seq * dm, dh, dm, 1), w["rk"], (seq * dm, dh, 1, dm), sc, (nh * seq * seq, seq * seq, seq, 1),
                     nb, nh, seq, dh, seq)
    w["sc"] = sc
    w["rsz"] = irs_w(w["sc"], c.sfz, 2)
    w["z"] = w["rsz"][0]
    w["smx"] = ismx_w(w["z"], expt, la, lseq)
    w["p"] = w["smx"]["p"]
    # attention output (xview_pv / wview_pv / yview_pv, p3_int_layer.cuh:124-148): PVA[b][i][h][k] = sum_j P[a][i][j] * YV[b][j][h][k]
    pva = torch.empty(1 << le, dtype=torch.int64, device=device)
    engine.ig_matmul(w["p"], (nh * seq * seq, seq * seq, seq, 1), w["yv"], (seq * dm, dh, dm, 1), pva, (seq * dm, dh, dm, 1),
                     nb, nh, seq, seq, dh)
    w["pva"] = pva
    w["rsat"] = irs_w(w["pva"], 16, 1)
    w["at"] = w["rsat"][0]
    w["acc"][ig.W_O] = mat(w["at"], Wd["w"][ig.W_O], c.d, c.d)
    w["rso"] = irs_w(w["acc"][ig.W_O], 16, 1)
    w["yo"] = w["rso"][0]
    w["res1"], w["idxRes1"] = iadd_w(x0, w["yo"])
    w["rms2"] = irms_w(w["res1"], Wd["g2"], isq, lT, ld)
    w["h2"] = w["rms2"]["y"]
    for i in (ig.W_G, ig.W_U):
        w["acc"][i] = mat(w["h2"], Wd["w"][i], c.d, c.dff)
    w["rsg"], w["rsu"] = irs_w(w["acc"][ig.W_G], 16, 1), irs_w(w["acc"][ig.W_U], 16, 1)
    w["gg"], w["uu"] = w["rsg"][0], w["rsu"][0]
    w["swg"] = iswg_w(w["gg"], w["uu"], silu)
    w["mo"] = w["swg"][2]
    w["acc"][ig.W_D] = mat(w["mo"], Wd["w"][ig.W_D], c.dff, c.d)
    w["rsd"] = irs_w(w["acc"][ig.W_D], 16, 1)
    w["yd"] = w["rsd"][0]
    w["out"], w["idxOut"] = iadd_w(w["res1"], w["yd"])
    return w
