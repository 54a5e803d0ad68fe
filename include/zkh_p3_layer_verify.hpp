// Host verifier of the integer decoder layer (the reference's p3itf::verify and the gadget verifiers under it, non-zk), so
// that a layer proved through this library can be checked without the reference and without a GPU:
//   p3imm::verify with operand views   (zkllm-src/p3_int_gadgets.cuh:608-668)   -> imm_verify_views
//   p3iadd / p3iswg / p3irope / p3irms / p3ismx ::verify  (:739-771, :1834-1880, :1324-1367, :1050-1175, :1629-1740)
//   p3itf::verify                       (zkllm-src/p3_int_layer.cuh:586-760)    -> itf_verify
// Each verifier replays the prover's transcript schedule, checks every sumcheck round, the terminal identity of the gadget's
// constraint polynomial on the claimed evaluations, and records the claims for the merged lookups and the batched openings
// (zkh_p3_verify.hpp).  Public columns (RoPE tables, causal mask, layer input and output) are evaluated on the host.
#pragma once
#include "zkh_p3_layer.hpp"
#include "zkh_p3_verify.hpp"

namespace zkh_p3v {

using zkh_p3::IgTables;
using zkh_p3::ItfConfig;
using zkh_p3::View;
using zkh_p3::Views;

inline const Hash* keep(VCtx& V, const Hash& h) {
    V.keep.push_back(h);
    return &V.keep.back();
}
inline void vdefer(VCtx& V, std::vector<const Hash*> roots, const Table* tab, uint32_t n) { V.luq.push_back({std::move(roots), tab, n}); }
inline bool no_tail(Reader& pf) { return pf.u32() == 0 && pf.u32() == 0; }
inline gl_t lift(int64_t v) { return v >= 0 ? (gl_t)v : P - (gl_t)(-v); }
// multilinear extension of a host column at z (bit i of the index is variable i)
inline gl_t mle_eval(std::vector<gl_t> c, const std::vector<gl_t>& z) {
    size_t n = c.size();
    for (size_t i = 0; i < z.size(); i++) {
        n >>= 1;
        for (size_t b = 0; b < n; b++) c[b] = add(c[2 * b], mul(z[i], sub(c[2 * b + 1], c[2 * b])));
    }
    return c[0];
}
inline std::vector<gl_t> tail_of(const std::vector<gl_t>& r, size_t from) { return std::vector<gl_t>(r.begin() + from, r.end()); }
inline std::vector<gl_t> head_of(const std::vector<gl_t>& r, size_t n) { return std::vector<gl_t>(r.begin(), r.begin() + n); }

// ---- matmul through operand views, composed mode ----
inline Verdict imm_verify_views(Transcript& tr, Reader& pf, const Hash& rX, const Hash& rW, const Hash& rY, uint32_t lj, uint32_t lk,
                                uint32_t li, VCtx& V, const Views* vw = nullptr) {
    if (pf.u32() != lj || pf.u32() != lk || pf.u32() != li) return Verdict::reject("imm dims");
    uint32_t d3[3] = {lj, lk, li};
    tr.absorb("imm-dims", d3, 12);
    tr.absorb("imm-X", rX.data(), 32);
    tr.absorb("imm-W", rW.data(), 32);
    tr.absorb("imm-Y", rY.data(), 32);
    std::vector<gl_t> z(lk + li);
    for (auto& x : z) x = tr.chal();
    const std::vector<gl_t> zk_ = head_of(z, lk), zi_ = tail_of(z, lk);
    const uint32_t lt = lj + lk + li;
    Reader msgs(pf.take((size_t)lt * 40), (size_t)lt * 40);
    const gl_t pyY = pf.gl(), pyX = pf.gl(), pyW = pf.gl();
    const gl_t yY = claimv(tr, V.vlg, rY, vw ? zkh_p3::view_point(vw->y, zk_, zi_, zkh_p3::S_A, zkh_p3::S_I) : z, pyY);
    std::vector<gl_t> r;
    gl_t claim;
    if (!sumcheck_verify(msgs, lt, 5, yY, tr, "imm-sc", r, claim)) return Verdict::reject("imm sumcheck");
    const std::vector<gl_t> rj(r.begin(), r.begin() + lj), rk(r.begin() + lj, r.begin() + lj + lk), ri(r.begin() + lj + lk, r.end());
    std::vector<gl_t> zx, zw, rsel(rk);
    rsel.insert(rsel.end(), ri.begin(), ri.end());
    if (vw) {
        zx = zkh_p3::view_point(vw->x, rj, ri);
        zw = zkh_p3::view_point(vw->w, rj, rk);
    } else {
        zx = rj; zx.insert(zx.end(), ri.begin(), ri.end());
        zw = rk; zw.insert(zw.end(), rj.begin(), rj.end());
    }
    const gl_t yX = claimv(tr, V.vlg, rX, zx, pyX), yW = claimv(tr, V.vlg, rW, zw, pyW);
    if (mul(eq_point(rsel, z), mul(yX, yW)) != claim) return Verdict::reject("imm terminal");
    if (pf.u32() != 0) return Verdict::reject("unexpected tail");
    return Verdict();
}

// ---- residual add: OUT = A + B ----
inline Verdict iadd_verify(Transcript& tr, const IgTables& T, Reader& pf, const Hash& rA, const Hash& rB, const Hash& rO, uint32_t le, VCtx& V) {
    if (pf.u32() != le) return Verdict::reject("iadd dims");
    tr.absorb("iad-dims", &le, 4);
    tr.absorb("iad-A", rA.data(), 32);
    tr.absorb("iad-B", rB.data(), 32);
    tr.absorb("iad-O", rO.data(), 32);
    vdefer(V, {keep(V, rO)}, &T.RS20, le);
    std::vector<gl_t> zE(le);
    for (auto& x : zE) x = tr.chal();
    Reader msgs(pf.take((size_t)le * 40), (size_t)le * 40);
    const gl_t pA = pf.gl(), pB = pf.gl(), pO = pf.gl();
    std::vector<gl_t> rE;
    gl_t claim;
    if (!sumcheck_verify(msgs, le, 5, 0, tr, "iad-sc", rE, claim)) return Verdict::reject("iadd sumcheck");
    const gl_t yA = claimv(tr, V.vlg, rA, rE, pA), yB = claimv(tr, V.vlg, rB, rE, pB), yO = claimv(tr, V.vlg, rO, rE, pO);
    if (mul(eq_point(rE, zE), sub(add(yA, yB), yO)) != claim) return Verdict::reject("iadd terminal");
    if (!no_tail(pf)) return Verdict::reject("unexpected tail");
    return Verdict();
}

// ---- SwiGLU product: MO = round(SILU[G] * U / 2^16) ----
inline Verdict iswg_verify(Transcript& tr, const IgTables& T, Reader& pf, const Hash& rG, const Hash& rU, const Hash& rM, uint32_t le, VCtx& V) {
    if (pf.u32() != le) return Verdict::reject("iswg dims");
    const Hash* rS = keep(V, pf.hash());
    const Hash* rR = keep(V, pf.hash());
    tr.absorb("isw-dims", &le, 4);
    tr.absorb("isw-G", rG.data(), 32);
    tr.absorb("isw-U", rU.data(), 32);
    tr.absorb("isw-M", rM.data(), 32);
    tr.absorb("isw-s", rS->data(), 32);
    tr.absorb("isw-r", rR->data(), 32);
    vdefer(V, {keep(V, rG), rS}, &T.SILU, le);
    vdefer(V, {rR}, &T.R16, le);
    vdefer(V, {keep(V, rM)}, &T.RS20, le);
    std::vector<gl_t> zE(le);
    for (auto& x : zE) x = tr.chal();
    Reader msgs(pf.take((size_t)le * 40), (size_t)le * 40);
    const gl_t pS = pf.gl(), pU = pf.gl(), pM = pf.gl(), pR = pf.gl();
    std::vector<gl_t> rE;
    gl_t claim;
    if (!sumcheck_verify(msgs, le, 5, 0, tr, "isw-sc", rE, claim)) return Verdict::reject("iswg sumcheck");
    const gl_t yS = claimv(tr, V.vlg, *rS, rE, pS), yU = claimv(tr, V.vlg, rU, rE, pU), yM = claimv(tr, V.vlg, rM, rE, pM),
               yR = claimv(tr, V.vlg, *rR, rE, pR);
    const gl_t t = sub(add(mul(yS, yU), 32768), add(mul(yM, 65536), yR));
    if (mul(eq_point(rE, zE), t) != claim) return Verdict::reject("iswg terminal");
    if (!no_tail(pf)) return Verdict::reject("unexpected tail");
    return Verdict();
}

// the public cos / signed-sin broadcasts of RoPE over u = lane | position << ld (p3irope::pub_col, zkllm-src/p3_int_gadgets.cuh:1199-1222)
inline void rope_pub_cols(const ItfConfig& c, const std::vector<int32_t>& ct, const std::vector<int32_t>& st, std::vector<gl_t>& C,
                          std::vector<gl_t>& S2) {
    const uint32_t le = c.lT + c.ld;
    C.resize((size_t)1 << le);
    S2.resize((size_t)1 << le);
    const size_t half = (size_t)c.dh / 2;
    for (size_t u = 0; u < C.size(); u++) {
        const size_t j = u & (c.d - 1), t = u >> c.ld, s = t & (c.seq - 1), jj = j & (c.dh - 1);
        const size_t ti = s * half + (jj & (half - 1));
        C[u] = lift(ct[ti]);
        S2[u] = lift(((jj >> (c.ldh - 1)) & 1) ? (int64_t)st[ti] : -(int64_t)st[ti]);
    }
}
// ---- RoPE: Y = round((Q C + Q' S2) / 2^14) ----
inline Verdict irope_verify(Transcript& tr, const IgTables& T, Reader& pf, const std::vector<gl_t>& Cpub, const std::vector<gl_t>& Spub,
                            const Hash& rQ, const Hash& rY, uint32_t ldh, uint32_t lT, uint32_t ld, VCtx& V) {
    const uint32_t le = lT + ld, fb = ldh - 1;
    if (pf.u32() != lT || pf.u32() != ld || pf.u32() != fb) return Verdict::reject("irope dims");
    const Hash* rR = keep(V, pf.hash());
    uint32_t d3[3] = {lT, ld, fb};
    tr.absorb("irp-dims", d3, 12);
    tr.absorb("irp-Q", rQ.data(), 32);
    tr.absorb("irp-Y", rY.data(), 32);
    tr.absorb("irp-r", rR->data(), 32);
    vdefer(V, {rR}, &T.R14, le);
    vdefer(V, {keep(V, rY)}, &T.RS20, le);
    std::vector<gl_t> zE(le);
    for (auto& x : zE) x = tr.chal();
    Reader msgs(pf.take((size_t)le * 40), (size_t)le * 40);
    const gl_t pQ = pf.gl(), pQx = pf.gl(), pY = pf.gl(), pR = pf.gl();
    std::vector<gl_t> rE;
    gl_t claim;
    if (!sumcheck_verify(msgs, le, 5, 0, tr, "irp-sc", rE, claim)) return Verdict::reject("irope sumcheck");
    std::vector<gl_t> rf = rE;
    rf[fb] = sub(1, rf[fb]);
    const gl_t yQ = claimv(tr, V.vlg, rQ, rE, pQ), yQx = claimv(tr, V.vlg, rQ, rf, pQx), yY = claimv(tr, V.vlg, rY, rE, pY),
               yR = claimv(tr, V.vlg, *rR, rE, pR);
    const gl_t yC = mle_eval(Cpub, rE), yS = mle_eval(Spub, rE);
    const gl_t t = sub(add(add(mul(yQ, yC), mul(yQx, yS)), 8192), add(mul(yY, 16384), yR));
    if (mul(eq_point(rE, zE), t) != claim) return Verdict::reject("irope terminal");
    if (!no_tail(pf)) return Verdict::reject("unexpected tail");
    return Verdict();
}

// ---- RMSNorm ----
inline Verdict irms_verify(Transcript& tr, const IgTables& T, Reader& pf, const Hash& rX, const Hash& rG, const Hash& rY, uint32_t lT,
                           uint32_t ld, VCtx& V) {
    using namespace zkh_p3;          // the B_* column names
    const uint32_t le = lT + ld;
    if (pf.u32() != lT || pf.u32() != ld) return Verdict::reject("irms dims");
    const Hash* rdb[NDB];
    const Hash* rde[3];
    for (int k = 0; k < NDB; k++) rdb[k] = keep(V, pf.hash());
    for (int k = 0; k < 3; k++) rde[k] = keep(V, pf.hash());
    uint32_t d2[2] = {lT, ld};
    tr.absorb("irm-dims", d2, 8);
    tr.absorb("irm-X", rX.data(), 32);
    tr.absorb("irm-G", rG.data(), 32);
    tr.absorb("irm-Y", rY.data(), 32);
    for (int k = 0; k < NDB; k++) tr.absorb("irm-cb", rdb[k]->data(), 32);
    for (int k = 0; k < 3; k++) tr.absorb("irm-ce", rde[k]->data(), 32);
    vdefer(V, {rdb[B_P4], rdb[B_P2], rdb[B_H2]}, &T.EXP4, lT);
    vdefer(V, {rdb[B_MM]}, &T.R16, lT);
    vdefer(V, {rdb[B_MS]}, &T.R16, lT);
    vdefer(V, {rdb[B_MM], rdb[B_RP]}, &T.ISQ, lT);
    const int limb[9] = {B_L40, B_L41, B_L42, B_D40, B_D41, B_D42, B_L20, B_D20, B_LR0};
    for (int l = 0; l < 9; l++) vdefer(V, {rdb[limb[l]]}, &T.R16, lT);
    vdefer(V, {rdb[B_LR1]}, &T.R16, lT);
    vdefer(V, {rde[1]}, &T.R16, le);
    vdefer(V, {rde[0]}, &T.RS20, le);
    vdefer(V, {rde[2]}, &T.R16, le);
    vdefer(V, {keep(V, rY)}, &T.RS20, le);
    const gl_t pyM = pf.gl(), pyMX = pf.gl();
    // M row-sum binding: sum_j X^2 = M - 2^14
    std::vector<gl_t> zb(lT);
    for (auto& x : zb) x = tr.chal();
    const gl_t yM = claimv(tr, V.vlg, *rdb[B_M], zb, pyM);
    std::vector<gl_t> rS;
    gl_t claim;
    if (!sumcheck_verify(pf, le, 5, sub(yM, (gl_t)1 << 14), tr, "irm-scS", rS, claim)) return Verdict::reject("irms M sumcheck");
    const gl_t yMX = claimv(tr, V.vlg, rX, rS, pyMX);
    if (mul(eq_point(tail_of(rS, ld), zb), mul(yMX, yMX)) != claim) return Verdict::reject("irms M terminal");
    // per-row constraints
    std::vector<gl_t> zB(lT);
    for (auto& x : zB) x = tr.chal();
    const gl_t lamB = tr.chal();
    std::vector<gl_t> rB;
    if (!sumcheck_verify(pf, lT, 5, 0, tr, "irm-scB", rB, claim)) return Verdict::reject("irms rows sumcheck");
    gl_t c[NDB];
    for (int k = 0; k < NDB; k++) c[k] = claimv(tr, V.vlg, *rdb[k], rB, pf.gl());
    {
        const gl_t r4 = add(c[B_L40], add(mul(c[B_L41], 65536), mul(c[B_L42], 4294967296ULL)));
        const gl_t d4 = add(c[B_D40], add(mul(c[B_D41], 65536), mul(c[B_D42], 4294967296ULL)));
        gl_t r[6];
        r[0] = sub(c[B_M], add(mul(c[B_MM], c[B_P4]), r4));
        r[1] = sub(sub(sub(c[B_P4], 1), r4), d4);
        r[2] = sub(add(mul(c[B_R], c[B_P2]), c[B_L20]), add(c[B_RP], c[B_H2]));
        r[3] = sub(sub(sub(c[B_P2], 1), c[B_L20]), c[B_D20]);
        r[4] = sub(c[B_R], add(c[B_LR0], mul(c[B_LR1], 65536)));
        r[5] = sub(add(c[B_MS], 16384), c[B_MM]);
        gl_t s = 0, lp = 1;
        for (int j = 0; j < 6; j++) { s = add(s, mul(lp, r[j])); lp = mul(lp, lamB); }
        if (mul(eq_point(rB, zB), s) != claim) return Verdict::reject("irms rows terminal");
    }
    // per-element constraints: W = round(R g / 2^16), Y = round(W x / 2^16)
    std::vector<gl_t> zE(le);
    for (auto& x : zE) x = tr.chal();
    const gl_t lamE = tr.chal();
    std::vector<gl_t> rE;
    if (!sumcheck_verify(pf, le, 5, 0, tr, "irm-scE", rE, claim)) return Verdict::reject("irms elements sumcheck");
    const gl_t pE0 = pf.gl(), pE1 = pf.gl(), pE2 = pf.gl(), pEX = pf.gl(), pEY = pf.gl(), pER = pf.gl(), pEG = pf.gl();
    const gl_t yX = claimv(tr, V.vlg, rX, rE, pEX), yY = claimv(tr, V.vlg, rY, rE, pEY);
    const gl_t yW = claimv(tr, V.vlg, *rde[0], rE, pE0), yRW = claimv(tr, V.vlg, *rde[1], rE, pE1), yRY = claimv(tr, V.vlg, *rde[2], rE, pE2);
    const gl_t yR = claimv(tr, V.vlg, *rdb[B_R], tail_of(rE, ld), pER), yG = claimv(tr, V.vlg, rG, head_of(rE, ld), pEG);
    const gl_t t1 = sub(add(mul(yR, yG), 32768), add(mul(yW, 65536), yRW));
    const gl_t t2 = sub(add(mul(yW, yX), 32768), add(mul(yY, 65536), yRY));
    if (mul(eq_point(rE, zE), add(t1, mul(lamE, t2))) != claim) return Verdict::reject("irms elements terminal");
    if (!no_tail(pf)) return Verdict::reject("unexpected tail");
    return Verdict();
}

// ---- causal softmax ----
inline Verdict ismx_verify(Transcript& tr, const IgTables& T, Reader& pf, const Hash& rZ, const Hash& rP, uint32_t la, uint32_t lseq, VCtx& V) {
    using namespace zkh_p3;          // the X_* column names
    const uint32_t lr = la + lseq, le = la + 2 * lseq;
    if (pf.u32() != la || pf.u32() != lseq) return Verdict::reject("ismx dims");
    const Hash* rce[NXE];
    const Hash* rcb[2];
    for (int k = 0; k < NXE; k++) rce[k] = keep(V, pf.hash());
    for (int k = 0; k < 2; k++) rcb[k] = keep(V, pf.hash());
    uint32_t d2[2] = {la, lseq};
    tr.absorb("ism-dims", d2, 8);
    tr.absorb("ism-Z", rZ.data(), 32);
    tr.absorb("ism-P", rP.data(), 32);
    for (int k = 0; k < NXE; k++) tr.absorb("ism-ce", rce[k]->data(), 32);
    for (int k = 0; k < 2; k++) tr.absorb("ism-cb", rcb[k]->data(), 32);
    vdefer(V, {rce[X_DM], rce[X_EE]}, &T.EXPT, le);
    for (int l = 0; l < 4; l++) vdefer(V, {rce[X_L0 + l]}, &T.R16, le);
    vdefer(V, {rcb[0]}, &T.RS16, lr);
    gl_t claim;
    // SEL row sum: sum_j SEL = 1 in every row
    std::vector<gl_t> zb(lr);
    for (auto& x : zb) x = tr.chal();
    std::vector<gl_t> rS;
    if (!sumcheck_verify(pf, le, 5, 1, tr, "ism-scsel", rS, claim)) return Verdict::reject("ismx sel sumcheck");
    const gl_t ySel = claimv(tr, V.vlg, *rce[X_SEL], rS, pf.gl());
    if (mul(eq_point(tail_of(rS, lseq), zb), ySel) != claim) return Verdict::reject("ismx sel terminal");
    // S row sum: sum_j EE = S
    for (auto& x : zb) x = tr.chal();
    const gl_t ySrow = claimv(tr, V.vlg, *rcb[1], zb, pf.gl());
    std::vector<gl_t> rS2;
    if (!sumcheck_verify(pf, le, 5, ySrow, tr, "ism-scs", rS2, claim)) return Verdict::reject("ismx sum sumcheck");
    const gl_t ySE = claimv(tr, V.vlg, *rce[X_EE], rS2, pf.gl());
    if (mul(eq_point(tail_of(rS2, lseq), zb), ySE) != claim) return Verdict::reject("ismx sum terminal");
    // per-element constraints
    std::vector<gl_t> zE(le);
    for (auto& x : zE) x = tr.chal();
    const gl_t lamE = tr.chal();
    std::vector<gl_t> rE;
    if (!sumcheck_verify(pf, le, 5, 0, tr, "ism-sce", rE, claim)) return Verdict::reject("ismx elements sumcheck");
    const gl_t yZ = claimv(tr, V.vlg, rZ, rE, pf.gl());
    gl_t e[NXE];
    for (int k = 0; k < NXE; k++) e[k] = claimv(tr, V.vlg, *rce[k], rE, pf.gl());
    const gl_t yP = claimv(tr, V.vlg, rP, rE, pf.gl());
    const std::vector<gl_t> rb = tail_of(rE, lseq);
    const gl_t yMX = claimv(tr, V.vlg, *rcb[0], rb, pf.gl()), yS = claimv(tr, V.vlg, *rcb[1], rb, pf.gl());
    // causal mask over u = j | i << lseq | a << 2 lseq: the MLE factors into (mask over (j, i)) x (1 over a)
    gl_t mk;
    {
        const size_t seq = (size_t)1 << lseq;
        std::vector<gl_t> m(seq * seq);
        for (size_t i = 0; i < seq; i++)
            for (size_t j = 0; j < seq; j++) m[j | (i << lseq)] = j <= i ? 1 : 0;
        mk = mle_eval(std::move(m), head_of(rE, 2 * lseq));
    }
    gl_t cst[5];
    cst[0] = sub(mul(e[X_SEL], e[X_SEL]), e[X_SEL]);
    cst[1] = mul(e[X_SEL], e[X_DM]);
    cst[2] = sub(add(add(sub(e[X_DM], mul(mk, yMX)), mul(mk, yZ)), mul(mk, 65536)), 65536);
    cst[3] = sub(sub(sub(add(mul(e[X_EE], 131072), yS), mul(2, mul(yP, yS))), e[X_L0]), mul(e[X_L1], 65536));
    cst[4] = sub(add(add(add(add(e[X_L2], mul(e[X_L3], 65536)), e[X_L0]), mul(e[X_L1], 65536)), 1), mul(2, yS));
    gl_t s = 0, lp = 1;
    for (int k = 0; k < 5; k++) { s = add(s, mul(lp, cst[k])); lp = mul(lp, lamE); }
    if (mul(eq_point(rE, zE), s) != claim) return Verdict::reject("ismx elements terminal");
    if (!no_tail(pf)) return Verdict::reject("unexpected tail");
    return Verdict();
}

// what the verifier of a layer holds besides the proof: the public input and output grids, the RoPE tables, and the
// commitment roots of the input, the seven weights and the two gains (in that order)
struct ItfPublic {
    std::vector<gl_t> x0, out;          // field-lifted, 2^(lT + ld) entries each
    std::vector<int32_t> ct, st;        // [seq][dh / 2] at scale 2^14
    Hash rX0, rW[7], rG1, rG2;
};

// p3itf::verify, non-zk.  Layout of the proof: 6 x u32 dims | 24 + 2A length-prefixed sub-proofs in proving order | 27 roots |
// u32 groups (len, GroupProof)* | ioin ioout | u32 batches (len, BatchProof)*
inline Verdict itf_verify(Transcript& tr, Reader pf, const ItfConfig& c, const IgTables& T, const ItfPublic& pub, uint32_t R, uint32_t Q) {
    using namespace zkh_p3;
    if (Q < Q_MIN || R < 1) return Verdict::reject("insecure params");
    const uint32_t ld = c.ld, lT = c.lT, ldff = c.ldff, lseq = c.lseq, ldh = c.ldh, la = c.la;
    const uint32_t le = ld + lT, lef = ldff + lT, lez = la + 2 * lseq;
    const uint32_t dims[6] = {c.seq, c.d, c.nh, c.dh, c.dff, c.batch};
    for (int k = 0; k < 6; k++)
        if (pf.u32() != dims[k]) return Verdict::reject("itf dims");
    if (pub.x0.size() != ((size_t)1 << le) || pub.out.size() != ((size_t)1 << le)) return Verdict::reject("public grids");
    const size_t nsub = 24 + 2 * (size_t)c.A;
    std::vector<Reader> subs;
    for (size_t k = 0; k < nsub; k++) subs.push_back(pf.blob());
    // the 27 roots: x0, h1, acc[7], yq yk yv rq rk sc z p pva at yo res1 h2 gg uu mo yd out
    enum { r_x0 = 0, r_h1, r_acc, r_yq = r_acc + 7, r_yk, r_yv, r_rq, r_rk, r_sc, r_z, r_p, r_pva, r_at, r_yo, r_res1, r_h2, r_gg, r_uu, r_mo,
           r_yd, r_out, NROOT };
    Hash rt[NROOT];
    for (int k = 0; k < NROOT; k++) rt[k] = pf.hash();
    if (rt[r_x0] != pub.rX0) return Verdict::reject("input root");
    VCtx V;
    tr.absorb("itf-dims", dims, 24);
    for (int i = 0; i < 7; i++) vdefer(V, {keep(V, pub.rW[i])}, &T.RS20, ilog2u(c.wrows(i) * c.wcols(i)));
    vdefer(V, {keep(V, pub.rG1)}, &T.RS20, ld);
    vdefer(V, {keep(V, pub.rG2)}, &T.RS20, ld);
    vdefer(V, {keep(V, rt[r_x0])}, &T.RS20, le);
    std::vector<gl_t> Cpub, Spub;
    rope_pub_cols(c, pub.ct, pub.st, Cpub, Spub);
    size_t si = 0;
    Verdict vd;
#define ZKH_SUB(call) do { Reader& sp = subs[si++]; \
                           try { vd = (call); } catch (const Malformed& e) { vd = Verdict::reject(e.what()); } \
                           if (!vd) return Verdict::reject("sub-proof " + std::to_string(si - 1) + ": " + vd.why); \
                           if (!sp.done()) return Verdict::reject("sub-proof " + std::to_string(si - 1) + ": trailing bytes"); } while (0)
    auto irs = [&](Reader& sp, const Hash& rX, const Hash& rY, uint32_t lev, uint32_t sf, int rng) { return irs_verify(tr, T, sp, rX, rY, lev, sf, rng, Q, R, &V); };
    ZKH_SUB(irms_verify(tr, T, sp, rt[r_x0], pub.rG1, rt[r_h1], lT, ld, V));
    for (int i : {W_Q, W_K, W_V}) ZKH_SUB(imm_verify_views(tr, sp, rt[r_h1], pub.rW[i], rt[r_acc + i], ld, ld, lT, V));
    ZKH_SUB(irs(sp, rt[r_acc + W_Q], rt[r_yq], le, 16, 1));
    ZKH_SUB(irs(sp, rt[r_acc + W_K], rt[r_yk], le, 16, 1));
    ZKH_SUB(irs(sp, rt[r_acc + W_V], rt[r_yv], le, 16, 1));
    ZKH_SUB(irope_verify(tr, T, sp, Cpub, Spub, rt[r_yq], rt[r_rq], ldh, lT, ld, V));
    ZKH_SUB(irope_verify(tr, T, sp, Cpub, Spub, rt[r_yk], rt[r_rk], ldh, lT, ld, V));
    for (uint32_t b = 0; b < c.batch; b++)
        for (uint32_t h = 0; h < c.nh; h++) {
            const Views v = views_qk(c, h, b);
            ZKH_SUB(imm_verify_views(tr, sp, rt[r_rq], rt[r_rk], rt[r_sc], ldh, lseq, lseq, V, &v));
        }
    ZKH_SUB(irs(sp, rt[r_sc], rt[r_z], lez, c.sfz, 2));
    ZKH_SUB(ismx_verify(tr, T, sp, rt[r_z], rt[r_p], la, lseq, V));
    for (uint32_t b = 0; b < c.batch; b++)
        for (uint32_t h = 0; h < c.nh; h++) {
            const Views v = views_pv(c, h, b);
            ZKH_SUB(imm_verify_views(tr, sp, rt[r_p], rt[r_yv], rt[r_pva], lseq, ldh, lseq, V, &v));
        }
    ZKH_SUB(irs(sp, rt[r_pva], rt[r_at], le, 16, 1));
    ZKH_SUB(imm_verify_views(tr, sp, rt[r_at], pub.rW[W_O], rt[r_acc + W_O], ld, ld, lT, V));
    ZKH_SUB(irs(sp, rt[r_acc + W_O], rt[r_yo], le, 16, 1));
    ZKH_SUB(iadd_verify(tr, T, sp, rt[r_x0], rt[r_yo], rt[r_res1], le, V));
    ZKH_SUB(irms_verify(tr, T, sp, rt[r_res1], pub.rG2, rt[r_h2], lT, ld, V));
    for (int i : {W_G, W_U}) ZKH_SUB(imm_verify_views(tr, sp, rt[r_h2], pub.rW[i], rt[r_acc + i], ld, ldff, lT, V));
    ZKH_SUB(irs(sp, rt[r_acc + W_G], rt[r_gg], lef, 16, 1));
    ZKH_SUB(irs(sp, rt[r_acc + W_U], rt[r_uu], lef, 16, 1));
    ZKH_SUB(iswg_verify(tr, T, sp, rt[r_gg], rt[r_uu], rt[r_mo], lef, V));
    ZKH_SUB(imm_verify_views(tr, sp, rt[r_mo], pub.rW[W_D], rt[r_acc + W_D], ldff, ld, lT, V));
    ZKH_SUB(irs(sp, rt[r_acc + W_D], rt[r_yd], le, 16, 1));
    ZKH_SUB(iadd_verify(tr, T, sp, rt[r_res1], rt[r_yd], rt[r_out], le, V));
#undef ZKH_SUB
    vd = lu_verify_flush(tr, V, pf);
    if (!vd) return vd;
    // public input / output bindings: the committed grids open to the public values at fresh points
    const gl_t pin = pf.gl(), pout = pf.gl();
    std::vector<gl_t> z1(le), z2(le);
    for (auto& x : z1) x = tr.chal();
    const gl_t ioin = claimv(tr, V.vlg, rt[r_x0], z1, pin);
    for (auto& x : z2) x = tr.chal();
    const gl_t ioout = claimv(tr, V.vlg, rt[r_out], z2, pout);
    if (ioin != mle_eval(pub.x0, z1)) return Verdict::reject("input binding");
    if (ioout != mle_eval(pub.out, z2)) return Verdict::reject("output binding");
    vd = tail_verify(tr, V, pf, Q, R, "itf-bo", false);
    if (!vd) return vd;
    if (!pf.done()) return Verdict::reject("itf trailing bytes");
    return Verdict();
}

}  // namespace zkh_p3v
