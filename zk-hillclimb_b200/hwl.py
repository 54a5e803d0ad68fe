"""The fp8 (Hawkeye) matmul gadget of the reference's p3 stack (zkllm-src/p3_hawkeye.cuh), non-zk, as host logic over
the engine interface of p3.py.

Statement: committed fp8-e4m3 operand codes X (B x K), W (N x K) and committed per-row fp32 scales produce the public
bf16 output Y (B x N) of the exact Hawkeye forward pass (groups of 32 products, 14-bit internal significand).  The proof
is the reference's p3hwl::LayerProof: witness columns over four domains (per product, per group, per output, per scale
row), 38 deferred lookups, five quartic zero-checks, the accumulator chain, the group-sum binding, the final-state slice
binding, the public-Y binding, one merged-lookup flush and one batched opening per size class.

The witness is the reference's replay (gen_witness, p3_hawkeye.cuh:342-637) written as tensor arithmetic: all outputs
advance together through the K/32 groups, so it runs on the GPU (or on the CPU for small cases) and its columns never
visit the host.
"""
import struct

import numpy as np
import torch

from .p3 import (F_HW_CH, F_HW_DG, F_HW_DO, F_HW_DP, F_HW_DS, F_HW_GS, F_PROD3, GL_P, claimc, commit_cols, lu_flush,
                 make_table)

# ---- column ids (p3_hawkeye.cuh:86-112) ----
(P_EB, P_MAG, P_SG, P_PR, P_SH, P_PW, P_Q, P_R, P_AL, P_SEL) = range(10)
NDP = 10
(G_ASIG, G_BEXP, G_ASGN, G_AZ, G_AINV, G_ABASE, G_ALO, G_ASH, G_APW, G_AQ, G_AR, G_MAX, G_ASEL, G_CSUM, G_TSGN, G_TMAG, G_TZ,
 G_TINV, G_WD, G_PLO, G_PHI, G_PDN, G_PUP, G_NR, G_S14, G_U1H, G_U1L, G_U2H, G_U2L) = range(29)
NDG = 29
(O_S14F, O_BEXP, O_SGN, O_FZ, O_FINV, O_C1, O_REM1, O_RB1, O_RT1, O_RTI1, O_ZRT1, O_FH1, O_FL1, O_FLH1, O_L01, O_RUP1, O_C21,
 O_M1, O_E1, O_S1, O_Z1, O_C2, O_RB2, O_TH2, O_TL2, O_RTI2, O_ZRT2, O_FH2, O_FL2, O_FLH2, O_L02, O_RUP2, O_C22, O_M2, O_E2,
 O_S2, O_Z2, O_Q16, O_Q16H, O_L03, O_RB3, O_RT3, O_RTI3, O_ZRT3, O_RUP3, O_YB) = range(46)
NDO = 46
(S_SS, S_SE, S_SEI, S_ZS, S_SMH, S_SML) = range(6)
NDS = 6
(LU_DM, LU_SH, LU_RM, LU_Q15, LU_ASH, LU_ARM, LU_AQ, LU_ABASE, LU_ALO, LU_WD, LU_U1H, LU_U1L, LU_U2H, LU_U2L, LU_NR, LU_S14,
 LU_M1REM, LU_M1RT, LU_M1FH, LU_M1FL, LU_M1FLH, LU_M1E, LU_M2TH, LU_M2TL, LU_M2FH, LU_M2FL, LU_M2FLH, LU_M2E, LU_Q16, LU_Q16H,
 LU_RT3, LU_S14F, LU_XSE, LU_XSMH, LU_XSML, LU_WSE, LU_WSMH, LU_WSML) = range(38)
NLU = 38
N_DO_CONSTR = 49
TAB_ORDER = ("DM", "SH", "RM", "R15", "ASH", "WIDTH", "R10", "R11", "R12", "R16", "FH", "REXP", "SE", "CREM13", "CREM12", "CTH")

# lookup instances: (table, domain 0 Dp / 1 Dg / 2 Do / 3 Db / 4 Dn, columns; -1 / -2 = the virtual product codes a / b)
LU_DEFS = [
    ("DM", 0, (-1, -2, P_EB, P_MAG, P_SG, P_PR)), ("SH", 0, (P_SH, P_PW)), ("RM", 0, (P_PW, P_R)), ("R15", 0, (P_Q,)),
    ("ASH", 1, (G_ASH, G_APW)), ("RM", 1, (G_APW, G_AR)), ("R15", 1, (G_AQ,)), ("R15", 1, (G_ABASE,)), ("R10", 1, (G_ALO,)),
    ("WIDTH", 1, (G_WD, G_PLO, G_PHI, G_PDN, G_PUP)), ("R10", 1, (G_U1H,)), ("R10", 1, (G_U1L,)), ("R10", 1, (G_U2H,)),
    ("R10", 1, (G_U2L,)), ("RM", 1, (G_PDN, G_NR)), ("R15", 1, (G_S14,)),
    ("CREM13", 2, (O_C1, O_REM1)), ("CREM12", 2, (O_C1, O_RT1)), ("FH", 2, (O_FH1,)), ("R12", 2, (O_FL1,)), ("R11", 2, (O_FLH1,)),
    ("REXP", 2, (O_E1,)), ("CTH", 2, (O_C2, O_TH2)), ("R12", 2, (O_TL2,)), ("FH", 2, (O_FH2,)), ("R12", 2, (O_FL2,)),
    ("R11", 2, (O_FLH2,)), ("REXP", 2, (O_E2,)), ("R16", 2, (O_Q16,)), ("R15", 2, (O_Q16H,)), ("R15", 2, (O_RT3,)),
    ("R15", 2, (O_S14F,)),
    ("SE", 3, (S_SE,)), ("R11", 3, (S_SMH,)), ("R12", 3, (S_SML,)), ("SE", 4, (S_SE,)), ("R11", 4, (S_SMH,)), ("R12", 4, (S_SML,)),
]


def decode_e4m3(code):
    """p3hwl::decode_e4m3 (p3_hawkeye.cuh:119-124) on an integer array / tensor: (effective exponent, significand, sign)."""
    sign = (code >> 7) & 1
    eb, mant = (code >> 3) & 15, code & 7
    nz = (eb != 0) * 1
    return eb + (1 - nz), mant + 8 * nz, sign


def build_tables():
    """p3hwl::build_tables (p3_hawkeye.cuh:125-192): the sixteen fixed public tables."""
    u = lambda a: np.asarray(a, dtype=np.uint64)
    T = {}
    j = np.arange(65536, dtype=np.int64)
    ca, cb = j >> 8, j & 255
    ea, siga, sna = decode_e4m3(ca)
    ebx, sigb, snb = decode_e4m3(cb)
    pr = ((siga != 0) & (sigb != 0)).astype(np.int64)
    T["DM"] = make_table([u(ca), u(cb), u(ea + ebx - 2), u((siga * sigb) << 7), u(pr & (sna ^ snb)), u(pr)])
    s = np.arange(64, dtype=np.int64)
    T["SH"] = make_table([u(s), u(1 << np.minimum(s, 15))])
    s = np.arange(256, dtype=np.int64)
    T["ASH"] = make_table([u(s), u(1 << np.minimum(s, 15))])
    p, r = np.ones(65536, dtype=np.int64), np.zeros(65536, dtype=np.int64)
    row = 0
    for t in range(16):
        p[row:row + (1 << t)] = 1 << t
        r[row:row + (1 << t)] = np.arange(1 << t)
        row += 1 << t
    T["RM"] = make_table([u(p), u(r)])
    wd = np.where(np.arange(32) <= 20, np.arange(32), 0).astype(np.int64)
    T["WIDTH"] = make_table([u(wd), u(np.where(wd > 0, 1 << np.maximum(wd - 1, 0), 0)), u(1 << wd), u(1 << np.maximum(wd - 14, 0)),
                             u(1 << np.maximum(14 - wd, 0))])
    for name, n in (("R10", 1024), ("R11", 2048), ("R12", 4096), ("R15", 32768), ("R16", 65536)):
        T[name] = make_table([u(np.arange(n))])
    T["FH"] = make_table([u(2048 + np.arange(2048))])
    j = np.arange(256)
    T["REXP"] = make_table([u(np.where((j >= 1) & (j <= 254), j, 1))])
    T["SE"] = make_table([u(np.where(j <= 254, j, 0))])

    def crem(rows, b):          # (c, x): c = 0 rows x < 2^b, then c = 1 rows x < 2^(b+1), zero padding
        c, x = np.zeros(rows, dtype=np.int64), np.zeros(rows, dtype=np.int64)
        x[:1 << b] = np.arange(1 << b)
        c[(1 << b):(1 << b) + (2 << b)] = 1
        x[(1 << b):(1 << b) + (2 << b)] = np.arange(2 << b)
        return make_table([u(c), u(x)])
    T["CREM13"], T["CREM12"], T["CTH"] = crem(32768, 13), crem(16384, 12), crem(4096, 10)
    return T


class Dims:
    """p3hwl::make_dims (p3_hawkeye.cuh:195-216): padded grids; one phantom group after the last real one."""

    def __init__(self, B, K, N):
        p2 = lambda x: 1 << max(x - 1, 0).bit_length()
        self.B, self.K, self.N = B, K, N
        self.NG = (K + 31) // 32
        self.Bpad, self.Npad, self.Gpad = p2(max(B, 2)), p2(max(N, 2)), p2(self.NG + 1)
        self.Kpad, self.Opad = 32 * self.Gpad, self.Bpad * self.Npad
        self.lb, self.ln, self.lg = self.Bpad.bit_length() - 1, self.Npad.bit_length() - 1, self.Gpad.bit_length() - 1
        self.lo = self.lb + self.ln
        self.G, self.P = self.Gpad * self.Opad, 32 * self.Gpad * self.Opad
        self.lgi, self.lp = self.lo + self.lg, self.lo + self.lg + 5


NEG_OFF = 1 - (1 << 32)        # field encoding of a negative int64 x is x + p; as a 64-bit pattern that is x + 1 - 2^32


def enc(t):
    """p3hwl::enc (p3_hawkeye.cuh:65): signed int64 tensor -> canonical field elements (as int64 bit patterns)."""
    return torch.where(t < 0, t + NEG_OFF, t)


def host_inverse(t):
    """Inverse of every (non-zero, canonical) element on the host: for CPU-sized witnesses."""
    vals = [pow((int(v) & 0xFFFFFFFFFFFFFFFF) % GL_P, GL_P - 2, GL_P) for v in t.reshape(-1).tolist()]
    return torch.tensor([v - (1 << 64) if v >= (1 << 63) else v for v in vals], dtype=torch.int64).reshape(t.shape)


class WitnessError(ValueError):
    """The layer is outside the gadget's supported domain (the reference's gen_witness throws the same message)."""


def gen_witness(B, K, N, x, w, xs, ws, device="cpu", inverse=host_inverse):
    """p3hwl::gen_witness (p3_hawkeye.cuh:342-637).  x: B*K and w: N*K fp8-e4m3 codes (uint8), xs: B and ws: N fp32 bit
    patterns (uint32).  ``inverse`` maps a tensor of non-zero field elements to their inverses (the engine's batched
    inversion on the GPU).  Returns a dict: d (Dims), xcodes / wcodes / xsb / wsb (padded operand columns), dp / dg / dob /
    db / dn (lists of columns), va / vb (the virtual product-code columns), lidx (38 int32 index columns), Y (B*N uint16,
    host).  All columns are int64 tensors on ``device`` holding canonical field elements."""
    d = Dims(B, K, N)
    I = torch.int64
    dev = torch.device(device)
    z = lambda *shape: torch.zeros(*shape, dtype=I, device=dev)
    one = lambda t: torch.ones_like(t)
    shl = lambda a, s: torch.bitwise_left_shift(a, s)
    shr = lambda a, s: torch.bitwise_right_shift(a, s)
    b2i = lambda t: t.to(I)
    xc, wc = z(d.Bpad, d.Kpad), z(d.Npad, d.Kpad)
    xc[:B, :K] = torch.as_tensor(np.asarray(x, dtype=np.uint8).reshape(B, K).astype(np.int64), device=dev)
    wc[:N, :K] = torch.as_tensor(np.asarray(w, dtype=np.uint8).reshape(N, K).astype(np.int64), device=dev)
    xsb, wsb = z(d.Bpad), z(d.Npad)
    xsb[:B] = torch.as_tensor(np.asarray(xs, dtype=np.uint32).astype(np.int64), device=dev)
    wsb[:N] = torch.as_tensor(np.asarray(ws, dtype=np.uint32).astype(np.int64), device=dev)
    errs = []

    def check(bad, msg):
        errs.append((bad.any(), msg))

    def inv_or0(t):
        nz = t != 0
        return torch.where(nz, inverse(torch.where(nz, t, one(t))), torch.zeros_like(t))

    dp = [z(d.Gpad, d.Opad, 32) for _ in range(NDP)]
    dg = [z(d.Gpad, d.Opad) for _ in range(NDG)]
    lidx = [None] * NLU
    for i in range(LU_DM, LU_Q15 + 1):
        lidx[i] = torch.zeros(d.Gpad, d.Opad, 32, dtype=torch.int32, device=dev)
    for i in range(LU_ASH, LU_S14 + 1):
        lidx[i] = torch.zeros(d.Gpad, d.Opad, dtype=torch.int32, device=dev)
    va, vb = z(d.Gpad, d.Opad, 32), z(d.Gpad, d.Opad, 32)

    # ---- scale decomposition (Db / Dn) ----
    def fill_scale(bits, which, lu0):
        ss, se, sm = shr(bits, 31), shr(bits, 23) & 255, bits & 0x7FFFFF
        check(se == 255, "hwl: inf/nan %s-scale unsupported" % which)
        check((se == 0) & (sm != 0), "hwl: subnormal %s-scale unsupported" % which)
        lidx[lu0], lidx[lu0 + 1], lidx[lu0 + 2] = se.to(torch.int32), shr(sm, 12).to(torch.int32), (sm & 4095).to(torch.int32)
        return [ss, se, inv_or0(se), b2i(se == 0), shr(sm, 12), sm & 4095]
    db, dn = fill_scale(xsb, "x", LU_XSE), fill_scale(wsb, "w", LU_WSE)

    # ---- replay over the groups, all outputs together ----
    ea_x, sig_x, sn_x = decode_e4m3(xc)                                   # [Bpad, Kpad]
    ea_w, sig_w, sn_w = decode_e4m3(wc)                                   # [Npad, Kpad]
    sgn, bexp, sig = z(d.Opad), z(d.Opad), z(d.Opad)
    O3 = (d.Opad, 32)
    for g in range(d.Gpad):
        ks = slice(g * 32, g * 32 + 32)
        bx = lambda t: t[:, None, ks].expand(d.Bpad, d.Npad, 32).reshape(O3)   # per-b value over the (b, n) grid
        bw = lambda t: t[None, :, ks].expand(d.Bpad, d.Npad, 32).reshape(O3)
        ca, cb = bx(xc), bw(wc)
        siga, sigb = bx(sig_x), bw(sig_w)
        pr = (siga != 0) & (sigb != 0)
        eb = bx(ea_x) + bw(ea_w) - 2
        bpe = eb + 127
        mag = shl(siga * sigb, 7)
        sg = pr & ((bx(sn_x) ^ bw(sn_w)) != 0)
        az = sig == 0
        baee = torch.where(az, torch.zeros_like(bexp), bexp)
        bgmax = torch.maximum(baee, torch.where(pr, bpe, torch.full_like(bpe, -1)).amax(dim=1))
        asel = baee == bgmax
        att = pr & (bpe == bgmax[:, None])
        sel = att & (att.cumsum(dim=1) == 1) & ~asel[:, None]
        sh = torch.where(pr, bgmax[:, None] - bpe, torch.zeros_like(bpe))
        check(sh > 63, "hwl: product shift > 63")
        shc = sh.clamp(max=15)
        pw = shl(one(shc), shc)
        q = shr(mag, shc)
        r = mag - shl(q, shc)
        al = torch.where(pr, torch.where(sg, -q, q), torch.zeros_like(q))
        csum = al.sum(dim=1)
        for c, t in ((P_EB, eb), (P_MAG, mag), (P_SG, b2i(sg)), (P_PR, b2i(pr)), (P_SH, sh), (P_PW, pw), (P_Q, q), (P_R, r),
                     (P_AL, enc(al)), (P_SEL, b2i(sel))):
            dp[c][g] = t
        va[g], vb[g] = ca, cb
        lidx[LU_DM][g] = (ca * 256 + cb).to(torch.int32)
        lidx[LU_SH][g] = sh.to(torch.int32)
        lidx[LU_RM][g] = (pw - 1 + r).to(torch.int32)
        lidx[LU_Q15][g] = q.to(torch.int32)
        # accumulator realign
        abase, alo = shr(sig, 10), sig & 1023
        ash = bgmax - baee
        check((ash < 0) | (ash > 255), "hwl: acc shift out of [0,255]")
        ashc = ash.clamp(min=0, max=15)
        apw = shl(one(ashc), ashc)
        aq = shr(abase, ashc)
        ar = abase - shl(aq, ashc)
        total = csum + torch.where(sgn != 0, -aq, aq)
        tsgn, tmag = b2i(total < 0), total.abs()
        tz = tmag == 0
        wd = z(d.Opad)
        for j in range(40):
            wd += b2i(tmag >= (1 << j))
        check(wd > 20, "hwl: total width > 20")
        wdc = wd.clamp(max=20)
        plo = torch.where(wdc > 0, shl(one(wdc), (wdc - 1).clamp(min=0)), torch.zeros_like(wdc))
        phi = shl(one(wdc), wdc)
        dn_s, up_s = (wdc - 14).clamp(min=0), (14 - wdc).clamp(min=0)
        pdn, pup = shl(one(wdc), dn_s), shl(one(wdc), up_s)
        u1, u2 = tmag - plo, phi - 1 - tmag
        nr = torch.where(wdc > 14, tmag & (pdn - 1), torch.zeros_like(tmag))
        s14 = torch.where(wdc > 14, shr(tmag, dn_s), shl(tmag, up_s))
        check(s14 * pdn + nr != tmag * pup, "hwl: s14 identity")
        for c, t in ((G_ASIG, sig), (G_BEXP, bexp), (G_ASGN, sgn), (G_AZ, b2i(az)), (G_ABASE, abase), (G_ALO, alo), (G_ASH, ash),
                     (G_APW, apw), (G_AQ, aq), (G_AR, enc(ar)), (G_MAX, bgmax), (G_ASEL, b2i(asel)), (G_CSUM, enc(csum)),
                     (G_TSGN, tsgn), (G_TMAG, tmag), (G_TZ, b2i(tz)), (G_WD, wd), (G_PLO, plo), (G_PHI, phi), (G_PDN, pdn),
                     (G_PUP, pup), (G_NR, nr), (G_S14, s14), (G_U1H, shr(u1, 10)), (G_U1L, u1 & 1023), (G_U2H, shr(u2, 10)),
                     (G_U2L, u2 & 1023)):
            dg[c][g] = t
        for i, t in ((LU_ASH, ash), (LU_ARM, apw - 1 + ar), (LU_AQ, aq), (LU_ABASE, abase), (LU_ALO, alo), (LU_WD, wd),
                     (LU_U1H, shr(u1, 10)), (LU_U1L, u1 & 1023), (LU_U2H, shr(u2, 10)), (LU_U2L, u2 & 1023),
                     (LU_NR, pdn - 1 + nr), (LU_S14, s14)):
            lidx[i][g] = t.to(torch.int32)
        zero = torch.zeros_like(sig)
        sgn = torch.where(tz, zero, tsgn)
        bexp = torch.where(tz, zero, bgmax + wd - 14)
        sig = torch.where(tz, zero, shl(s14, 10))
    dg[G_AINV] = inv_or0(dg[G_ASIG])
    dg[G_TINV] = inv_or0(dg[G_TMAG])

    # ---- per-output: gfloat -> fp32, two RNE multiplies by the scales, bf16 RNE downcast ----
    dob, Z, ONE = [None] * NDO, z(d.Opad), z(d.Opad) + 1
    s14f = shr(sig, 10)
    check(shl(s14f, 10) != sig, "hwl: fsig low bits")
    fz = sig == 0
    xb = xsb[:, None].expand(d.Bpad, d.Npad).reshape(-1)
    wb = wsb[None, :].expand(d.Bpad, d.Npad).reshape(-1)
    ssx, sex, smx = shr(xb, 31), shr(xb, 23) & 255, xb & 0x7FFFFF
    ssw, sew, smw = shr(wb, 31), shr(wb, 23) & 255, wb & 0x7FFFFF
    z1 = fz | (sex == 0)
    z2 = z1 | (sew == 0)
    s1o, s2o = sgn ^ ssx, sgn ^ ssx ^ ssw
    pick = lambda zf, dflt, val: torch.where(zf, dflt, val)
    # mul1
    mm1 = s14f * ((1 << 23) | smx)                                       # < 2^38
    c1 = b2i(mm1 >= (1 << 37))
    mfl1 = shr(mm1, 13 + c1)
    rem1 = mm1 & (shl(ONE, 13 + c1) - 1)
    fh1, fl1 = shr(mfl1, 12), mfl1 & 4095
    rb1, rt1 = shr(rem1, 12 + c1), rem1 & (shl(ONE, 12 + c1) - 1)
    rup1 = b2i((rb1 != 0) & ((rt1 != 0) | ((fl1 & 1) != 0)))
    mr1 = mfl1 + rup1
    c21 = b2i(mr1 == (1 << 24))
    m1o = mr1 - shl(c21, 23)
    e1o = (bexp - 12) + sex - 127 + c1 + c21
    check(~z1 & ((e1o < 1) | (e1o > 254)), "hwl: mul1 out of normal fp32 range")
    c1, rem1, rb1, rt1, rup1, c21 = (pick(z1, Z, t) for t in (c1, rem1, rb1, rt1, rup1, c21))
    fh1, fl1, m1o, e1o = pick(z1, Z + 2048, fh1), pick(z1, Z, fl1), pick(z1, Z + (1 << 23), m1o), pick(z1, ONE, e1o)
    for c, t in ((O_S14F, s14f), (O_BEXP, bexp), (O_SGN, sgn), (O_FZ, b2i(fz)), (O_C1, c1), (O_REM1, rem1), (O_RB1, rb1),
                 (O_RT1, rt1), (O_ZRT1, b2i(rt1 == 0)), (O_FH1, fh1), (O_FL1, fl1), (O_FLH1, shr(fl1, 1)), (O_L01, fl1 & 1),
                 (O_RUP1, rup1), (O_C21, c21), (O_M1, m1o), (O_E1, e1o), (O_S1, s1o), (O_Z1, b2i(z1))):
        dob[c] = t
    lidx[LU_S14F] = s14f.to(torch.int32)
    lidx[LU_M1REM], lidx[LU_M1RT] = (c1 * 8192 + rem1).to(torch.int32), (c1 * 4096 + rt1).to(torch.int32)
    lidx[LU_M1FH], lidx[LU_M1FL], lidx[LU_M1FLH] = (fh1 - 2048).to(torch.int32), fl1.to(torch.int32), shr(fl1, 1).to(torch.int32)
    lidx[LU_M1E] = e1o.to(torch.int32)
    # mul2
    mm2 = m1o * ((1 << 23) | smw)                                        # < 2^48
    c2 = b2i(mm2 >= (1 << 47))
    mfl2 = shr(mm2, 23 + c2)
    rem2 = mm2 & (shl(ONE, 23 + c2) - 1)
    fh2, fl2 = shr(mfl2, 12), mfl2 & 4095
    rb2, rt2 = shr(rem2, 22 + c2), rem2 & (shl(ONE, 22 + c2) - 1)
    th2, tl2 = shr(rt2, 12), rt2 & 4095
    rup2 = b2i((rb2 != 0) & ((rt2 != 0) | ((fl2 & 1) != 0)))
    mr2 = mfl2 + rup2
    c22 = b2i(mr2 == (1 << 24))
    m2o = mr2 - shl(c22, 23)
    e2o = e1o + sew - 127 + c2 + c22
    check(~z2 & ((e2o < 1) | (e2o > 254)), "hwl: mul2 out of normal fp32 range")
    c2, rb2, th2, tl2, rup2, c22 = (pick(z2, Z, t) for t in (c2, rb2, th2, tl2, rup2, c22))
    fh2, fl2, m2o, e2o = pick(z2, Z + 2048, fh2), pick(z2, Z, fl2), pick(z2, Z + (1 << 23), m2o), pick(z2, ONE, e2o)
    rt2 = th2 * 4096 + tl2
    for c, t in ((O_C2, c2), (O_RB2, rb2), (O_TH2, th2), (O_TL2, tl2), (O_ZRT2, b2i(rt2 == 0)), (O_FH2, fh2), (O_FL2, fl2),
                 (O_FLH2, shr(fl2, 1)), (O_L02, fl2 & 1), (O_RUP2, rup2), (O_C22, c22), (O_M2, m2o), (O_E2, e2o), (O_S2, s2o),
                 (O_Z2, b2i(z2))):
        dob[c] = t
    lidx[LU_M2TH], lidx[LU_M2TL] = (c2 * 1024 + th2).to(torch.int32), tl2.to(torch.int32)
    lidx[LU_M2FH], lidx[LU_M2FL], lidx[LU_M2FLH] = (fh2 - 2048).to(torch.int32), fl2.to(torch.int32), shr(fl2, 1).to(torch.int32)
    lidx[LU_M2E] = e2o.to(torch.int32)
    # bf16 downcast = integer round-to-nearest-even of the fp32 bits >> 16
    b32 = shl(s2o, 31) | pick(z2, Z, shl(e2o, 23) | (m2o - (1 << 23)))
    q16, rem3 = shr(b32, 16), b32 & 0xFFFF
    rb3, rt3 = shr(rem3, 15), rem3 & 0x7FFF
    rup3 = b2i((rb3 != 0) & ((rt3 != 0) | ((q16 & 1) != 0)))
    yb = q16 + rup3
    for c, t in ((O_Q16, q16), (O_Q16H, shr(q16, 1)), (O_L03, q16 & 1), (O_RB3, rb3), (O_RT3, rt3), (O_ZRT3, b2i(rt3 == 0)),
                 (O_RUP3, rup3), (O_YB, yb)):
        dob[c] = t
    lidx[LU_Q16], lidx[LU_Q16H], lidx[LU_RT3] = q16.to(torch.int32), shr(q16, 1).to(torch.int32), rt3.to(torch.int32)
    dob[O_FINV], dob[O_RTI1], dob[O_RTI2], dob[O_RTI3] = inv_or0(s14f), inv_or0(rt1), inv_or0(rt2), inv_or0(rt3)
    bad = torch.stack([e[0] for e in errs]).tolist()
    for flag, (_, msg) in zip(bad, errs):
        if flag:
            raise WitnessError(msg)
    Y = yb.view(d.Bpad, d.Npad)[:B, :N].to(torch.int32).cpu().numpy().astype(np.uint16).reshape(-1)
    flat = lambda cols: [c.reshape(-1).contiguous() for c in cols]
    return {"d": d, "xcodes": xc.reshape(-1), "wcodes": wc.reshape(-1), "xsb": xsb, "wsb": wsb, "dp": flat(dp), "dg": flat(dg),
            "dob": flat(dob), "db": flat(db), "dn": flat(dn), "va": va.reshape(-1), "vb": vb.reshape(-1),
            "lidx": [t.reshape(-1).contiguous() for t in lidx], "Y": Y}



def gen_witness_dev(engine, B, K, N, x, w, xs, ws):
    """The same witness from the CUDA replay kernel (zkh_hwl_witness: one warp per output, lane = product of the group):
    columns are allocated on the engine's GPU and filled in one pass.  Same result dict as gen_witness."""
    d = Dims(B, K, N)
    dev = torch.device("cuda:%d" % engine.device)
    I = torch.int64
    xc, wc = torch.zeros(d.Bpad, d.Kpad, dtype=I, device=dev), torch.zeros(d.Npad, d.Kpad, dtype=I, device=dev)
    xc[:B, :K] = torch.as_tensor(np.asarray(x, dtype=np.uint8).reshape(B, K).astype(np.int64), device=dev)
    wc[:N, :K] = torch.as_tensor(np.asarray(w, dtype=np.uint8).reshape(N, K).astype(np.int64), device=dev)
    xsb, wsb = torch.zeros(d.Bpad, dtype=I, device=dev), torch.zeros(d.Npad, dtype=I, device=dev)
    xsb[:B] = torch.as_tensor(np.asarray(xs, dtype=np.uint32).astype(np.int64), device=dev)
    wsb[:N] = torch.as_tensor(np.asarray(ws, dtype=np.uint32).astype(np.int64), device=dev)
    new = lambda n, dt=I: torch.empty(n, dtype=dt, device=dev)
    dp, dg, dob = [new(d.P) for _ in range(NDP)], [new(d.G) for _ in range(NDG)], [new(d.Opad) for _ in range(NDO)]
    db, dn = [new(d.Bpad) for _ in range(NDS)], [new(d.Npad) for _ in range(NDS)]
    va, vb = new(d.P), new(d.P)
    sizes = [d.P] * 4 + [d.G] * 12 + [d.Opad] * 16 + [d.Bpad] * 3 + [d.Npad] * 3
    lidx = [new(n, torch.int32) for n in sizes]
    try:
        engine.hwl_witness(d.lb, d.ln, d.lg, xc, wc, xsb, wsb, dp + dg + dob + db + dn + [va, vb], lidx)
    except Exception as e:
        if "hwl:" in str(e):
            raise WitnessError(str(e)[str(e).index("hwl:"):]) from None
        raise
    Y = dob[O_YB].view(d.Bpad, d.Npad)[:B, :N].to(torch.int32).cpu().numpy().astype(np.uint16).reshape(-1)
    return {"d": d, "xcodes": xc.reshape(-1), "wcodes": wc.reshape(-1), "xsb": xsb, "wsb": wsb, "dp": dp, "dg": dg, "dob": dob,
            "db": db, "dn": dn, "va": va, "vb": vb, "lidx": lidx, "Y": Y}


def zx_point(d, rA):
    """p3hwl::zx_point (p3_hawkeye.cuh:1856-1862): product-domain point [kk | n | b | g] -> X's point [kk | g | b]."""
    rA = [int(v) for v in rA]
    return rA[:5] + rA[5 + d.ln + d.lb:5 + d.ln + d.lb + d.lg] + rA[5 + d.ln:5 + d.ln + d.lb]


def zw_point(d, rA):
    """p3hwl::zw_point (p3_hawkeye.cuh:1863-1869): product-domain point -> W's point [kk | g | n]."""
    rA = [int(v) for v in rA]
    return rA[:5] + rA[5 + d.ln + d.lb:5 + d.ln + d.lb + d.lg] + rA[5:5 + d.ln]


def commit_operands(engine, wt, R, col):
    """p3hwl::commit_operands (p3_hawkeye.cuh:1873-1882): (column, root) of the padded X / W code columns and the two
    scale-bit columns.  ``col`` turns a witness tensor into an engine column."""
    out = {}
    for name, key in (("X", "xcodes"), ("W", "wcodes"), ("XS", "xsb"), ("WS", "wsb")):
        c = col(wt[key])
        out[name] = (c, engine.commit_gpu_rootonly(c, R))
    return out


def _powers(x, n):
    out = [1]
    for _ in range(n - 1):
        out.append(out[-1] * x % GL_P)
    return out


def prove(engine, tr, wt, T, ops, R, Q, col, Ypub=None, ctx=None, strict=True):
    """p3hwl::prove (p3_hawkeye.cuh:1938-2466), non-zk.  wt: gen_witness(...); T: build_tables(); ops: commit_operands(...).
    With ``ctx`` (a shared ledger + lookup queue, ig.Ctx) the lookup flush and the batched openings are left to the
    caller.  Returns the serialised p3hwl::LayerProof:
      u32 B K N | roots dp[10] dg[29] do[46] db[6] dn[6] | u32 groups (len, GroupProof)* |
      mDp yDp[10] yDpG | mDg yDg[29] | mCh yCh[8] | yGSc yGSa | mGS yGSal yGSsel | mDo yDo[46] | yDbBC[5] yDnBC[5] |
      mDb yDb[6] yXsb | mDn yDn[6] yWsb | ySlA ySlE ySlS ySlF ySlBE ySlSG | mY yY | u32 batches (len, BatchProof)*
    where every message list is u32 rounds + rounds * 40 bytes."""
    from .ig import Ctx
    d = wt["d"]
    Y = np.ascontiguousarray(wt["Y"] if Ypub is None else Ypub, dtype=np.uint16)
    tr.absorb("hwl-dims", struct.pack("<III", d.B, d.K, d.N))
    for name in TAB_ORDER:
        tr.absorb("hwl-tab", T[name]["id"])
    for label, key in (("hwl-X", "X"), ("hwl-W", "W"), ("hwl-xs", "XS"), ("hwl-ws", "WS")):
        tr.absorb(label, ops[key][1])
    tr.absorb("hwl-Y", Y.tobytes())
    own = ctx is None
    if own:
        ctx = Ctx()
    lg = ctx.ledger
    chal_vec = lambda n: [tr.chal() for _ in range(n)]
    eq = lambda z: engine.build_eq_gpu(np.array(z, dtype=np.uint64))
    claim = lambda c, z: claimc(engine, tr, lg, c[0], c[1], z)
    u64 = lambda vals: np.array(vals, dtype=np.uint64).tobytes()
    msgs_bytes = lambda m: struct.pack("<I", len(m)) + np.ascontiguousarray(m, dtype=np.uint64).tobytes()

    # -- witness commitments --
    def commit_all(cols):
        return commit_cols(engine, [col(t) for t in cols], R)
    CDp, CDg, CDo, CDb, CDn = (commit_all(wt[k]) for k in ("dp", "dg", "dob", "db", "dn"))
    for label, cd in (("hwl-cp", CDp), ("hwl-cg", CDg), ("hwl-co", CDo), ("hwl-cb", CDb), ("hwl-cn", CDn)):
        for _, root in cd:
            tr.absorb(label, root)

    # -- lookups: deferred to the merged flush; the virtual product codes are bound to X / W at the lookup point --
    doms = (CDp, CDg, CDo, CDb, CDn)
    va, vb = col(wt["va"]), col(wt["vb"])
    for i, (tab, dom, cids) in enumerate(LU_DEFS):
        spec = [(va, None) if c == -1 else (vb, None) if c == -2 else doms[dom][c] for c in cids]
        ent = {"W": spec, "idx": col(wt["lidx"][i]), "tab": T[tab]}
        if i == LU_DM:
            ent["bind"] = lambda pm, yv: [(ops["X"][0], ops["X"][1], np.array(zx_point(d, pm), dtype=np.uint64), yv[0]),
                                          (ops["W"][0], ops["W"][1], np.array(zw_point(d, pm), dtype=np.uint64), yv[1])]
        ctx.luq.append(ent)

    # -- Dp zero-check --
    zC = chal_vec(d.lp)
    lamP = _powers(tr.chal(), 6)
    cols = [eq(zC)] + [c for c, _ in CDp] + [engine.bcast_rows(CDg[G_MAX][0], 5)]
    rC, mDp, _ = engine.sc5_run(tr, "hwl-scP", cols, F_HW_DP, lamP)
    rC = [int(v) for v in rC]
    yDp = [claim(c, rC) for c in CDp]
    yDpG = claim(CDg[G_MAX], rC[5:d.lp])
    del cols
    # -- Dg zero-check --
    zG = chal_vec(d.lgi)
    lamG = _powers(tr.chal(), 18)
    rG, mDg, _ = engine.sc5_run(tr, "hwl-scG", [eq(zG)] + [c for c, _ in CDg], F_HW_DG, lamG)
    rG = [int(v) for v in rG]
    yDg = [claim(c, rG) for c in CDg]
    # -- accumulator chain: A(g+1) = out(g), A(0) = 0 --
    zc = chal_vec(d.lo)
    lch = tr.chal()
    lam6 = chal_vec(6)
    lpow = _powers(lch, d.Gpad)
    ug = [0] + lpow[:d.Gpad - 1]
    vg = lpow[:d.Gpad - 1] + [0]
    eqO = engine.bcast_cols(eq(zc), d.lg)                                 # eqO[o] at gi = g*Opad + o
    wcol = lambda vals: engine.bcast_rows(engine.upload(np.array(vals, dtype=np.uint64)), d.lo)
    U, V = engine.mul(eqO, wcol(ug)), engine.mul(eqO, wcol(vg))
    U0 = engine.mul(eqO, wcol([1] + [0] * (d.Gpad - 1)))
    CH = (G_ASIG, G_BEXP, G_ASGN, G_TZ, G_S14, G_MAX, G_WD, G_TSGN)
    rH, mCh, _ = engine.sc5_run(tr, "hwl-scH", [U, V, U0] + [CDg[c][0] for c in CH], F_HW_CH, lam6)
    rH = [int(v) for v in rH]
    yCh = [claim(CDg[c], rH) for c in CH]
    del U, V, U0, eqO
    # -- group-sum + attainment-sum binding (Dp -> Dg) --
    z2 = chal_vec(d.lgi)
    yGSc, yGSa = claim(CDg[G_CSUM], z2), claim(CDg[G_ASEL], z2)
    lam2 = [tr.chal(), tr.chal()]
    rS, mGS, _ = engine.sc5_run(tr, "hwl-scS", [engine.bcast_rows(eq(z2), 5), CDp[P_AL][0], CDp[P_SEL][0]], F_HW_GS, lam2)
    rS = [int(v) for v in rS]
    yGSal, yGSsel = claim(CDp[P_AL], rS), claim(CDp[P_SEL], rS)
    # -- Do zero-check --
    zO = chal_vec(d.lo)
    lamO = _powers(tr.chal(), N_DO_CONSTR)
    BCX = (S_SS, S_SE, S_ZS, S_SMH, S_SML)
    cols = [eq(zO)] + [c for c, _ in CDo] + [engine.bcast_rows(CDb[j][0], d.ln) for j in BCX] + \
        [engine.bcast_cols(CDn[j][0], d.lb) for j in BCX]
    rO, mDo, _ = engine.sc5_run(tr, "hwl-scO", cols, F_HW_DO, lamO)
    rO = [int(v) for v in rO]
    yDo = [claim(c, rO) for c in CDo]
    pB, pN = rO[d.ln:d.lo], rO[:d.ln]
    yDbBC = [claim(CDb[j], pB) for j in BCX]
    yDnBC = [claim(CDn[j], pN) for j in BCX]
    del cols
    # -- Db / Dn scale-decomposition zero-checks --
    SC = (S_SS, S_SE, S_SEI, S_ZS, S_SMH, S_SML)

    def scale_check(tag, lv, opcol, cd):
        zz = chal_vec(lv)
        lam = _powers(tr.chal(), 6)
        r, m, _ = engine.sc5_run(tr, tag, [eq(zz), opcol[0]] + [cd[j][0] for j in SC], F_HW_DS, lam)
        r = [int(v) for v in r]
        return m, [claim(cd[j], r) for j in SC], claim(opcol, r)
    mDb, yDb, yXsb = scale_check("hwl-scB", d.lb, ops["XS"], CDb)
    mDn, yDn, yWsb = scale_check("hwl-scN", d.ln, ops["WS"], CDn)
    # -- final-state slice binding: A(., g = NG) feeds the output stage --
    zc2 = chal_vec(d.lo)
    ptg = zc2 + [(d.NG >> i) & 1 for i in range(d.lg)]
    ySl = [claim(CDg[G_ASIG], ptg), claim(CDg[G_BEXP], ptg), claim(CDg[G_ASGN], ptg),
           claim(CDo[O_S14F], zc2), claim(CDo[O_BEXP], zc2), claim(CDo[O_SGN], zc2)]
    # -- public-Y binding restricted to the real B x N grid --
    zY = chal_vec(d.lo)
    Rw = np.zeros((d.Bpad, d.Npad), dtype=np.uint64)
    Rw[:d.B, :d.N] = 1
    rY, mY, _ = engine.sc_prove_gpu(tr, "hwl-scY", [eq(zY), engine.upload(Rw.reshape(-1)), CDo[O_YB][0]], F_PROD3, 5)
    yY = claim(CDo[O_YB], [int(v) for v in rY])

    lug, batches = [], []
    if own:
        lug = lu_flush(engine, tr, ctx.luq, lg, R, strict)
        batches = [engine.prove_class(tr, np.stack(c[1]), c[2], R, Q, "hwl-bo%d" % i) for i, c in enumerate(lg.cls)]
    out = struct.pack("<III", d.B, d.K, d.N)
    for cd in (CDp, CDg, CDo, CDb, CDn):
        out += b"".join(root for _, root in cd)
    out += struct.pack("<I", len(lug)) + b"".join(struct.pack("<I", len(b)) + b for b in lug)
    out += msgs_bytes(mDp) + u64(yDp) + u64([yDpG]) + msgs_bytes(mDg) + u64(yDg) + msgs_bytes(mCh) + u64(yCh)
    out += u64([yGSc, yGSa]) + msgs_bytes(mGS) + u64([yGSal, yGSsel]) + msgs_bytes(mDo) + u64(yDo) + u64(yDbBC) + u64(yDnBC)
    out += msgs_bytes(mDb) + u64(yDb) + u64([yXsb]) + msgs_bytes(mDn) + u64(yDn) + u64([yWsb]) + u64(ySl)
    out += msgs_bytes(mY) + u64([yY])
    out += struct.pack("<I", len(batches)) + b"".join(struct.pack("<I", len(b)) + b for b in batches)
    return out
