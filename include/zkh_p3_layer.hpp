// The integer decoder layer (the reference's p3itf stack, non-zk) as C++ host logic over the C ABI: witness chain,
// commitments and the layer proof, byte-identical to the reference's prover (and to this package's Python mirror).
//   p3ig::build_tables                      (zkllm-src/p3_int_gadgets.cuh:75-127)      -> IgTables
//   p3imm::prove with operand views         (zkllm-src/p3_int_gadgets.cuh:448-497, :546-605) -> imm_prove_views
//   p3irs::prove on a given witness         (zkllm-src/p3_int_gadgets.cuh:282-340)     -> irs_prove_wit
//   p3iadd / p3iswg / p3irope / p3irms / p3ismx ::prove  (:712-737, :1795-1832, :1279-1322, :922-1047, :1518-1643)
//   p3itf::Config / build_witness / commit_all / prove   (zkllm-src/p3_int_layer.cuh:41-62, :182-318, :343-419, :452-581)
// Everything the gadgets do on the device goes through entry points of zkh.h; this header only orders the calls, keeps
// the transcript, and serialises.  Header-only; include after zkh_p3.hpp's dependencies are available, link libzkh.so.
#pragma once
#include <functional>
#include <map>

#include "zkh_p3.hpp"

namespace zkh_p3 {

inline gl_t gl_neg(gl_t x) { x %= GL_P; return x ? GL_P - x : 0; }
inline gl_t gl_powmod(gl_t b, unsigned e) { gl_t r = 1; while (e--) r = gl_mulmod(r, b); return r; }
inline gl_t gl_lift(int64_t v) { return v >= 0 ? (gl_t)v : GL_P - (gl_t)(-v); }
inline uint32_t ilog2u(size_t n) { uint32_t l = 0; while (((size_t)1 << l) < n) l++; return l; }

using Term = std::pair<gl_t, std::vector<uint8_t>>;

// p3ig::build_tables: the range tables of IrsTables plus the function tables (host routine zkh_ig_table, so that the
// values match the reference's libm results) and EXP4 = (4^e, 2^e, floor(2^e / 2)) with e capped at 17
struct IgTables : IrsTables {
    Table EXPT, SILU, ISQ, EXP4;
    uint32_t btop;
    IgTables(uint32_t d, uint32_t btop_) : IrsTables(btop_), btop(btop_) {
        auto fn = [&](int kind, size_t rows) {
            std::vector<gl_t> c0(rows), c1(rows);
            if (zkh_ig_table(kind, d, c0.data(), c1.data()) != 0) throw std::runtime_error("zkh_ig_table failed");
            return make_table({c0, c1});
        };
        EXPT = fn(0, (size_t)1 << 17);
        SILU = fn(1, (size_t)1 << 20);
        ISQ = fn(2, (size_t)1 << 16);
        std::vector<gl_t> a(32), b(32), c(32);
        for (int e = 0; e < 32; e++) {
            const int er = e < 17 ? e : 17;
            a[e] = (gl_t)1 << (2 * er);
            b[e] = (gl_t)1 << er;
            c[e] = er ? (gl_t)1 << (er - 1) : 0;
        }
        EXP4 = make_table({a, b, c});
    }
};

// ---- small device helpers over the C ABI ----
inline DevCol dev_gather_bits(Prover& P, const DevCol& col, size_t n, uint64_t konst, const std::vector<uint64_t>& masks) {
    DevCol out(P, n);
    P.ck(zkh_gl_gather_bits(P.ctx(), col.data(), col.size(), n, konst, masks.data(), (uint32_t)masks.size(), out.data()));
    return out;
}
// out[e] = col[e >> ld]: a per-row value repeated along the row
inline DevCol bcast_rows(Prover& P, const DevCol& col, uint32_t ld) {
    const uint32_t lr = ilog2u(col.size());
    std::vector<uint64_t> m(ld + lr, 0);
    for (uint32_t b = 0; b < lr; b++) m[ld + b] = (uint64_t)1 << b;
    return dev_gather_bits(P, col, col.size() << ld, 0, m);
}
// out[e] = col[e mod len(col)]: a per-column value repeated over 2^lT rows
inline DevCol bcast_cols(Prover& P, const DevCol& col, uint32_t lT) {
    const uint32_t lc = ilog2u(col.size());
    std::vector<uint64_t> m(lc + lT, 0);
    for (uint32_t b = 0; b < lc; b++) m[b] = (uint64_t)1 << b;
    return dev_gather_bits(P, col, col.size() << lT, 0, m);
}
inline DevCol flip_bit(Prover& P, const DevCol& col, uint32_t b) {
    DevCol out(P, col.size());
    P.ck(zkh_gl_gather_xor(P.ctx(), col.data(), col.size(), (uint64_t)1 << b, out.data()));
    return out;
}
inline DevCol dev_matvec(Prover& P, const DevCol& M, uint64_t rows, uint64_t cols, const DevCol& w, bool along_rows) {
    DevCol out(P, along_rows ? rows : cols);
    P.ck(zkh_gl_matvec(P.ctx(), M.data(), rows, cols, w.data(), along_rows ? 1 : 0, out.data()));
    return out;
}
inline DevCol dev_scaled(Prover& P, const DevCol& in, gl_t sc) {
    DevCol out(P, in.size());
    P.ck(zkh_gl_scale(P.ctx(), in.data(), in.size(), sc, out.data()));
    return out;
}

// ---- operand views (p3imm::OpView): bit t of the element index comes from bit `bit` of the contraction index (S_J), of
// the free index (S_A), of Y's row index (S_I), or is the constant `bit` (S_C) ----
enum { S_J = 0, S_A = 1, S_I = 2, S_C = 3 };
using View = std::vector<std::pair<int, int>>;
inline View view_consts(uint32_t bits, uint32_t val) {
    View v;
    for (uint32_t t = 0; t < bits; t++) v.push_back({S_C, (int)((val >> t) & 1)});
    return v;
}
inline void view_cat(View& a, const View& b) { a.insert(a.end(), b.begin(), b.end()); }
inline View view_run(int src, uint32_t bits) {
    View v;
    for (uint32_t t = 0; t < bits; t++) v.push_back({src, (int)t});
    return v;
}
// p3imm::op_pt / y_pt: the claim point on the committed column
inline std::vector<gl_t> view_point(const View& v, const std::vector<gl_t>& r_first, const std::vector<gl_t>& r_second,
                                    int first = S_J, int second = S_A) {
    std::vector<gl_t> z;
    for (auto& sb : v) z.push_back(sb.first == first ? r_first[sb.second] : sb.first == second ? r_second[sb.second]
                                                                                                : sb.first == S_C ? (gl_t)sb.second : 0);
    return z;
}
// dense operand behind a view: out[u] over u = lo | hi << l_lo, where index group `lo_src` supplies the low bits
inline DevCol view_gather(Prover& P, const DevCol& col, const View& v, int lo_src, uint32_t l_lo, int hi_src, uint32_t l_hi) {
    std::vector<uint64_t> m(l_lo + l_hi, 0);
    uint64_t konst = 0;
    for (size_t t = 0; t < v.size(); t++) {
        if (v[t].first == S_C) konst |= (uint64_t)v[t].second << t;
        else if (v[t].first == lo_src) m[v[t].second] |= (uint64_t)1 << t;
        else if (v[t].first == hi_src) m[l_lo + v[t].second] |= (uint64_t)1 << t;
    }
    return dev_gather_bits(P, col, (size_t)1 << (l_lo + l_hi), konst, m);
}

struct Views { View x, w, y; };

// p3imm::prove, composed mode (shared ledger), optionally through operand views into larger committed grids (the per-head
// attention products).  The factored form of zkh_p3::imm_prove; the claims land on the committed columns at the views' points.
inline std::vector<uint8_t> imm_prove_views(Prover& P, Transcript& tr, const CCol& X, const CCol& W, const CCol& Y, uint32_t lj,
                                            uint32_t lk, uint32_t li, XCtx& xc, const Views* vw = nullptr) {
    zkh_ctx* ctx = P.ctx();
    uint32_t d3[3] = {lj, lk, li};
    tr.absorb("imm-dims", d3, 12);
    tr.absorb("imm-X", X.root.data(), 32);
    tr.absorb("imm-W", W.root.data(), 32);
    tr.absorb("imm-Y", Y.root.data(), 32);
    std::vector<gl_t> z(lk + li);
    for (auto& v : z) v = tr.chal();
    std::vector<gl_t> zk_(z.begin(), z.begin() + lk), zi_(z.begin() + lk, z.end());
    const gl_t yY = claimc(P, tr, xc.lg, Y, vw ? view_point(vw->y, zk_, zi_, S_A, S_I) : z);
    DevCol Xg, Wg;
    const DevCol* Xd = X.col;
    const DevCol* Wd = W.col;
    if (vw) {
        Xg = view_gather(P, *X.col, vw->x, S_J, lj, S_A, li);      // [i][j]
        Wg = view_gather(P, *W.col, vw->w, S_A, lk, S_J, lj);      // [j][k]
        Xd = &Xg;
        Wd = &Wg;
    }
    const uint64_t J = 1ull << lj, K = 1ull << lk, I = 1ull << li;
    DevCol eq_i = P.build_eq_gpu(zi_), eq_k = P.build_eq_gpu(zk_);
    std::vector<gl_t> msgs, rj, rk, ri, fin;
    DevCol Xz = dev_matvec(P, *Xd, I, J, eq_i, false), Wz = dev_matvec(P, *Wd, J, K, eq_k, true);
    if (lj) rj = P.sc_prove_gpu(tr, "imm-sc", {Xz.data(), Wz.data()}, (uint32_t)J, ZKH_F_PROD2, 5, nullptr, 0, msgs);
    DevCol eq_rj = P.build_eq_gpu(rj);
    DevCol X1 = dev_matvec(P, *Xd, I, J, eq_rj, true), W1 = dev_matvec(P, *Wd, J, K, eq_rj, false);
    const gl_t SX = P.eval_h_gpu(X1, zi_);
    gl_t Wrr;
    if (lk) {
        DevCol sk = dev_scaled(P, eq_k, SX);
        rk = P.sc_prove_gpu(tr, "imm-sc", {sk.data(), W1.data()}, (uint32_t)K, ZKH_F_PROD2, 5, nullptr, 0, msgs, &fin);
        Wrr = fin[1];
    } else {
        P.ck(zkh_download(ctx, &Wrr, W1.data(), 8));
    }
    gl_t eqk_r = 1;
    for (uint32_t t = 0; t < lk; t++) {
        const gl_t a = rk[t], b = zk_[t];
        const gl_t one_a = (GL_P + 1 - a) % GL_P, one_b = (GL_P + 1 - b) % GL_P;
        eqk_r = gl_mulmod(eqk_r, gl_addmod(gl_mulmod(a, b), gl_mulmod(one_a, one_b)));
    }
    if (li) {
        DevCol si = dev_scaled(P, eq_i, gl_mulmod(eqk_r, Wrr));
        ri = P.sc_prove_gpu(tr, "imm-sc", {si.data(), X1.data()}, (uint32_t)I, ZKH_F_PROD2, 5, nullptr, 0, msgs);
    }
    std::vector<gl_t> zx, zw;
    if (vw) {
        zx = view_point(vw->x, rj, ri);
        zw = view_point(vw->w, rj, rk);
    } else {
        zx = rj; zx.insert(zx.end(), ri.begin(), ri.end());
        zw = rk; zw.insert(zw.end(), rj.begin(), rj.end());
    }
    const gl_t yX = claimc(P, tr, xc.lg, X, zx), yW = claimc(P, tr, xc.lg, W, zw);
    std::vector<uint8_t> out;
    put_raw(out, d3, 12);
    put_raw(out, msgs.data(), msgs.size() * 8);
    put_raw(out, &yY, 8); put_raw(out, &yX, 8); put_raw(out, &yW, 8);
    put_u32(out, 0);
    return out;
}

// deferred lookup of committed columns
inline void defer(XCtx& xc, std::vector<CCol> W, const DevIdx* idx, Table* tab) {
    std::vector<bool> com(W.size(), true);
    xc.luq.push_back({std::move(W), std::move(com), idx, tab});
}
inline const std::vector<uint8_t>& empty_tail() {
    static const std::vector<uint8_t> t(8, 0);       // u32 groups = 0, u32 batches = 0
    return t;
}
// zE <- le challenges; sumcheck of eq(zE, .) * (konst + terms) over cols (column 0 of the term indices is the eq weight)
inline std::vector<gl_t> zerocheck(Prover& P, Transcript& tr, const char* tag, uint32_t le, std::vector<const gl_t*> cols,
                                   const std::vector<Term>& terms, gl_t konst, std::vector<gl_t>& msgs) {
    std::vector<gl_t> zE(le);
    for (auto& v : zE) v = tr.chal();
    DevCol E = P.build_eq_gpu(zE);
    cols.insert(cols.begin(), E.data());
    return P.sc_prove_zc(tr, tag, cols, (uint32_t)1 << le, terms, konst, msgs);
}

// witness of one rescale: y and the columns / index arrays p3irs::gen_witness produces (zkh_irs_witness)
struct IrsWit {
    DevCol y, L0, L1;
    DevIdx i0, i1, iY;
    uint32_t nl = 1;
};
inline IrsWit irs_witness(Prover& P, const DevCol& acc, uint32_t sf, int rng) {
    IrsWit w;
    const size_t n = acc.size();
    w.nl = sf <= 16 ? 1 : 2;
    w.y = DevCol(P, n);
    w.L0 = DevCol(P, n);
    w.L1 = DevCol(P, w.nl == 2 ? n : 1);
    w.i0 = DevIdx(P, n);
    w.i1 = DevIdx(P, w.nl == 2 ? n : 1);
    w.iY = DevIdx(P, rng ? n : 1);
    P.ck(zkh_irs_witness(P.ctx(), acc.data(), n, sf, rng, w.y.data(), w.L0.data(), w.nl == 2 ? w.L1.data() : nullptr, w.i0.data(),
                         w.nl == 2 ? w.i1.data() : nullptr, rng ? w.iY.data() : nullptr));
    return w;
}
// p3irs::prove in composed mode on a witness made earlier (the layer builds its whole chain before it proves)
inline std::vector<uint8_t> irs_prove_wit(Prover& P, Transcript& tr, IrsTables& T, const CCol& X, const CCol& Y, IrsWit& w, uint32_t le,
                                          uint32_t sf, int rng, uint32_t R, XCtx& xc) {
    const size_t n = (size_t)1 << le;
    const uint32_t nl = w.nl;
    uint32_t d4[4] = {le, sf, nl, (uint32_t)rng};
    tr.absorb("irs-dims", d4, 16);
    tr.absorb("irs-X", X.root.data(), 32);
    tr.absorb("irs-Y", Y.root.data(), 32);
    CCol Lc[2] = {{&w.L0, P.commit_gpu_rootonly(w.L0, R)}, {&w.L1, Hash{}}};
    if (nl == 2) Lc[1].root = P.commit_gpu_rootonly(w.L1, R);
    for (uint32_t l = 0; l < nl; l++) tr.absorb("irs-L", Lc[l].root.data(), 32);
    defer(xc, {Lc[0]}, &w.i0, sf == 14 ? &T.R14 : &T.R16);
    if (nl == 2) defer(xc, {Lc[1]}, &w.i1, sf == 32 ? &T.R16 : &T.RTOP);
    if (rng) defer(xc, {Y}, &w.iY, rng == 1 ? &T.RS20 : &T.RS16);
    std::vector<gl_t> zE(le);
    for (auto& v : zE) v = tr.chal();
    DevCol E = P.build_eq_gpu(zE);
    std::vector<const gl_t*> cols = {E.data(), X.col->data(), Y.col->data(), w.L0.data()};
    if (nl == 2) cols.push_back(w.L1.data());
    const gl_t par[2] = {(gl_t)1 << (sf - 1), (gl_t)1 << sf};
    std::vector<gl_t> msgs;
    std::vector<gl_t> rE = P.sc_prove_gpu(tr, "irs-sc", cols, (uint32_t)n, nl == 1 ? ZKH_F_IRS1 : ZKH_F_IRS2, 5, par, 2, msgs);
    const gl_t yX = claimc(P, tr, xc.lg, X, rE), yY = claimc(P, tr, xc.lg, Y, rE);
    gl_t yL[2] = {0, 0};
    for (uint32_t l = 0; l < nl; l++) yL[l] = claimc(P, tr, xc.lg, Lc[l], rE);
    std::vector<uint8_t> out;
    put_raw(out, d4, 16);
    for (uint32_t l = 0; l < nl; l++) put_raw(out, Lc[l].root.data(), 32);
    put_raw(out, msgs.data(), msgs.size() * 8);
    put_raw(out, &yX, 8); put_raw(out, &yY, 8); put_raw(out, yL, 8 * nl);
    put_raw(out, empty_tail().data(), 8);
    return out;
}

// p3iadd::prove: OUT = A + B with OUT in the RS20 window.  Proof: u32 le | messages le*40 | yA yB yO | tail
inline std::vector<uint8_t> iadd_prove(Prover& P, Transcript& tr, IgTables& T, const CCol& A, const CCol& B, const CCol& OUT,
                                       const DevIdx& idxO, uint32_t le, XCtx& xc) {
    tr.absorb("iad-dims", &le, 4);
    tr.absorb("iad-A", A.root.data(), 32);
    tr.absorb("iad-B", B.root.data(), 32);
    tr.absorb("iad-O", OUT.root.data(), 32);
    defer(xc, {OUT}, &idxO, &T.RS20);
    std::vector<gl_t> msgs;
    std::vector<gl_t> rE = zerocheck(P, tr, "iad-sc", le, {A.col->data(), B.col->data(), OUT.col->data()},
                                     {{1, {1}}, {1, {2}}, {gl_neg(1), {3}}}, 0, msgs);
    gl_t ys[3] = {claimc(P, tr, xc.lg, A, rE), claimc(P, tr, xc.lg, B, rE), claimc(P, tr, xc.lg, OUT, rE)};
    std::vector<uint8_t> out;
    put_u32(out, le);
    put_raw(out, msgs.data(), msgs.size() * 8);
    put_raw(out, ys, 24);
    put_raw(out, empty_tail().data(), 8);
    return out;
}

// p3iswg::prove: MO = round(SILU[G] * U / 2^16).  Proof: u32 le | rSIL rREM | messages | ySIL yU yM yR | tail
struct SwgWit { DevCol sil, rem, mo; DevIdx iG, iR, iM; };
inline std::vector<uint8_t> iswg_prove(Prover& P, Transcript& tr, IgTables& T, const CCol& G, const CCol& U, const CCol& MO, SwgWit& w,
                                       uint32_t le, uint32_t R, XCtx& xc) {
    tr.absorb("isw-dims", &le, 4);
    tr.absorb("isw-G", G.root.data(), 32);
    tr.absorb("isw-U", U.root.data(), 32);
    tr.absorb("isw-M", MO.root.data(), 32);
    const CCol S{&w.sil, P.commit_gpu_rootonly(w.sil, R)}, Rm{&w.rem, P.commit_gpu_rootonly(w.rem, R)};
    tr.absorb("isw-s", S.root.data(), 32);
    tr.absorb("isw-r", Rm.root.data(), 32);
    defer(xc, {G, S}, &w.iG, &T.SILU);
    defer(xc, {Rm}, &w.iR, &T.R16);
    defer(xc, {MO}, &w.iM, &T.RS20);
    std::vector<gl_t> msgs;
    std::vector<gl_t> rE = zerocheck(P, tr, "isw-sc", le, {w.sil.data(), U.col->data(), MO.col->data(), w.rem.data()},
                                     {{1, {1, 2}}, {gl_neg(65536), {3}}, {gl_neg(1), {4}}}, 32768, msgs);
    gl_t ys[4] = {claimc(P, tr, xc.lg, S, rE), claimc(P, tr, xc.lg, U, rE), claimc(P, tr, xc.lg, MO, rE), claimc(P, tr, xc.lg, Rm, rE)};
    std::vector<uint8_t> out;
    put_u32(out, le);
    put_raw(out, S.root.data(), 32);
    put_raw(out, Rm.root.data(), 32);
    put_raw(out, msgs.data(), msgs.size() * 8);
    put_raw(out, ys, 32);
    put_raw(out, empty_tail().data(), 8);
    return out;
}

// p3irope::prove: Y = round((Q C + Q' S2) / 2^14), Q' the rotate-half partner.  Proof: u32 lT ld fb | rREM | messages |
// yQ yQx yY yR | tail.  C, S2: the public broadcasts as field columns.
struct RopeWit { DevCol y, rem, C, S2; DevIdx iR, iY; };
inline std::vector<uint8_t> irope_prove(Prover& P, Transcript& tr, IgTables& T, const CCol& Qc, const CCol& Y, RopeWit& w, uint32_t ldh,
                                        uint32_t lT, uint32_t ld, uint32_t R, XCtx& xc) {
    const uint32_t le = lT + ld, fb = ldh - 1;
    uint32_t d3[3] = {lT, ld, fb};
    tr.absorb("irp-dims", d3, 12);
    tr.absorb("irp-Q", Qc.root.data(), 32);
    tr.absorb("irp-Y", Y.root.data(), 32);
    const CCol Rm{&w.rem, P.commit_gpu_rootonly(w.rem, R)};
    tr.absorb("irp-r", Rm.root.data(), 32);
    defer(xc, {Rm}, &w.iR, &T.R14);
    defer(xc, {Y}, &w.iY, &T.RS20);
    DevCol Qx = flip_bit(P, *Qc.col, fb);
    std::vector<gl_t> msgs;
    std::vector<gl_t> rE = zerocheck(P, tr, "irp-sc", le, {Qc.col->data(), Qx.data(), Y.col->data(), w.rem.data(), w.C.data(), w.S2.data()},
                                     {{1, {1, 5}}, {1, {2, 6}}, {gl_neg(16384), {3}}, {gl_neg(1), {4}}}, 8192, msgs);
    std::vector<gl_t> rf = rE;
    rf[fb] = (GL_P + 1 - rf[fb]) % GL_P;
    gl_t ys[4];
    ys[0] = claimc(P, tr, xc.lg, Qc, rE);
    ys[1] = claimc(P, tr, xc.lg, Qc, rf);
    ys[2] = claimc(P, tr, xc.lg, Y, rE);
    ys[3] = claimc(P, tr, xc.lg, Rm, rE);
    std::vector<uint8_t> out;
    put_raw(out, d3, 12);
    put_raw(out, Rm.root.data(), 32);
    put_raw(out, msgs.data(), msgs.size() * 8);
    put_raw(out, ys, 32);
    put_raw(out, empty_tail().data(), 8);
    return out;
}

// ---- RMSNorm (p3irms) ----
enum { B_M = 0, B_MM, B_MS, B_P4, B_P2, B_H2, B_RP, B_L40, B_L41, B_L42, B_D40, B_D41, B_D42, B_R, B_L20, B_D20, B_LR0, B_LR1, NDB };
// zkh_ig_rms_witness: db = the 18 per-row columns, de = W, remW, remY per element, y; irow = lookup rows of e, m, m - 2^14, m,
// the nine 16-bit limbs, LR1; iel = remW, W + 2^19, remY, Y + 2^19
struct RmsWit { DevCol db[NDB], de[3], y; DevIdx irow[14], iel[4]; };
inline RmsWit irms_witness(Prover& P, IgTables& T, const DevCol& x, const DevCol& g, uint32_t lT, uint32_t ld) {
    RmsWit w;
    const size_t B = (size_t)1 << lT, n = (size_t)1 << (lT + ld);
    uint64_t* db[NDB]; uint64_t* de[3]; uint32_t* ir[14]; uint32_t* ie[4];
    for (int k = 0; k < NDB; k++) { w.db[k] = DevCol(P, B); db[k] = w.db[k].data(); }
    for (int k = 0; k < 3; k++) { w.de[k] = DevCol(P, n); de[k] = w.de[k].data(); }
    for (int k = 0; k < 14; k++) { w.irow[k] = DevIdx(P, B); ir[k] = w.irow[k].data(); }
    for (int k = 0; k < 4; k++) { w.iel[k] = DevIdx(P, n); ie[k] = w.iel[k].data(); }
    w.y = DevCol(P, n);
    P.ck(zkh_ig_rms_witness(P.ctx(), x.data(), g.data(), T.ISQ.on(P)[1].data(), lT, ld, db, de, w.y.data(), ir, ie));
    return w;
}
// the six per-row constraints (zkllm-src/p3_int_gadgets.cuh:984-1003) over [E, 18 row columns], batched with powers of lamB
inline void irms_terms_rows(gl_t lamB, std::vector<Term>& t, gl_t& konst) {
    gl_t lam[6];
    for (int j = 0; j < 6; j++) lam[j] = gl_powmod(lamB, j);
    auto c = [](int k) { return (uint8_t)(1 + k); };
    auto n = [](gl_t x) { return gl_neg(x); };
    auto sh = [](gl_t x, int s) { return gl_mulmod(x, (gl_t)1 << s); };
    t = {
        {lam[0], {c(B_M)}}, {n(lam[0]), {c(B_MM), c(B_P4)}}, {n(lam[0]), {c(B_L40)}}, {n(sh(lam[0], 16)), {c(B_L41)}}, {n(sh(lam[0], 32)), {c(B_L42)}},
        {lam[1], {c(B_P4)}}, {n(lam[1]), {c(B_L40)}}, {n(sh(lam[1], 16)), {c(B_L41)}}, {n(sh(lam[1], 32)), {c(B_L42)}},
        {n(lam[1]), {c(B_D40)}}, {n(sh(lam[1], 16)), {c(B_D41)}}, {n(sh(lam[1], 32)), {c(B_D42)}},
        {lam[2], {c(B_R), c(B_P2)}}, {lam[2], {c(B_L20)}}, {n(lam[2]), {c(B_RP)}}, {n(lam[2]), {c(B_H2)}},
        {lam[3], {c(B_P2)}}, {n(lam[3]), {c(B_L20)}}, {n(lam[3]), {c(B_D20)}},
        {lam[4], {c(B_R)}}, {n(lam[4]), {c(B_LR0)}}, {n(sh(lam[4], 16)), {c(B_LR1)}},
        {lam[5], {c(B_MS)}}, {n(lam[5]), {c(B_MM)}},
    };
    konst = gl_addmod(gl_addmod(n(lam[1]), n(lam[3])), gl_mulmod(lam[5], 16384));
}
// p3irms::prove.  Proof: u32 lT ld | 18 row roots | 3 element roots | yM yMX | mS | mB yB[18] | mE yE[3] yEX yEY yER yEG | tail
inline std::vector<uint8_t> irms_prove(Prover& P, Transcript& tr, IgTables& T, const CCol& X, const CCol& G, const CCol& Y, RmsWit& w,
                                       uint32_t lT, uint32_t ld, uint32_t R, XCtx& xc) {
    const uint32_t le = lT + ld;
    uint32_t d2[2] = {lT, ld};
    tr.absorb("irm-dims", d2, 8);
    tr.absorb("irm-X", X.root.data(), 32);
    tr.absorb("irm-G", G.root.data(), 32);
    tr.absorb("irm-Y", Y.root.data(), 32);
    CCol CB[NDB], CE[3];
    for (int k = 0; k < NDB; k++) { CB[k] = {&w.db[k], P.commit_gpu_rootonly(w.db[k], R)}; tr.absorb("irm-cb", CB[k].root.data(), 32); }
    for (int k = 0; k < 3; k++) { CE[k] = {&w.de[k], P.commit_gpu_rootonly(w.de[k], R)}; tr.absorb("irm-ce", CE[k].root.data(), 32); }
    defer(xc, {CB[B_P4], CB[B_P2], CB[B_H2]}, &w.irow[0], &T.EXP4);
    defer(xc, {CB[B_MM]}, &w.irow[1], &T.R16);
    defer(xc, {CB[B_MS]}, &w.irow[2], &T.R16);
    defer(xc, {CB[B_MM], CB[B_RP]}, &w.irow[3], &T.ISQ);
    const int limb[9] = {B_L40, B_L41, B_L42, B_D40, B_D41, B_D42, B_L20, B_D20, B_LR0};
    for (int l = 0; l < 9; l++) defer(xc, {CB[limb[l]]}, &w.irow[4 + l], &T.R16);
    defer(xc, {CB[B_LR1]}, &w.irow[13], &T.R16);
    defer(xc, {CE[1]}, &w.iel[0], &T.R16);
    defer(xc, {CE[0]}, &w.iel[1], &T.RS20);
    defer(xc, {CE[2]}, &w.iel[2], &T.R16);
    defer(xc, {Y}, &w.iel[3], &T.RS20);
    // M row-sum binding: sum_j X^2 = M - 2^14, weighted by eq(zb, row)
    std::vector<gl_t> zb(lT);
    for (auto& v : zb) v = tr.chal();
    const gl_t yM = claimc(P, tr, xc.lg, CB[B_M], zb);
    std::vector<gl_t> mS, mB, mE;
    std::vector<gl_t> rS;
    {
        DevCol eqb = P.build_eq_gpu(zb);
        DevCol EQb = bcast_rows(P, eqb, ld);
        rS = P.sc_prove_zc(tr, "irm-scS", {EQb.data(), X.col->data()}, (uint32_t)1 << le, {{1, {1, 1}}}, 0, mS);
    }
    const gl_t yMX = claimc(P, tr, xc.lg, X, rS);
    // per-row zero-check
    std::vector<gl_t> zB(lT);
    for (auto& v : zB) v = tr.chal();
    const gl_t lamB = tr.chal();
    std::vector<Term> terms;
    gl_t konstB;
    irms_terms_rows(lamB, terms, konstB);
    std::vector<gl_t> rB;
    {
        DevCol EB = P.build_eq_gpu(zB);
        std::vector<const gl_t*> cols = {EB.data()};
        for (int k = 0; k < NDB; k++) cols.push_back(w.db[k].data());
        rB = P.sc_prove_zc(tr, "irm-scB", cols, (uint32_t)1 << lT, terms, konstB, mB);
    }
    gl_t yB[NDB];
    for (int k = 0; k < NDB; k++) yB[k] = claimc(P, tr, xc.lg, CB[k], rB);
    // per-element zero-check: W = round(R g / 2^16), Y = round(W x / 2^16)
    std::vector<gl_t> zE(le);
    for (auto& v : zE) v = tr.chal();
    const gl_t lamE = tr.chal();
    std::vector<gl_t> rE;
    {
        DevCol EE = P.build_eq_gpu(zE);
        DevCol Rb = bcast_rows(P, w.db[B_R], ld), Gb = bcast_cols(P, *G.col, lT);
        auto n = [](gl_t x) { return gl_neg(x); };
        std::vector<Term> tE = {{1, {6, 7}}, {n(65536), {3}}, {n(1), {4}}, {lamE, {3, 1}}, {n(gl_mulmod(lamE, 65536)), {2}}, {n(lamE), {5}}};
        const gl_t konstE = gl_addmod(32768, gl_mulmod(lamE, 32768));
        rE = P.sc_prove_zc(tr, "irm-scE", {EE.data(), X.col->data(), Y.col->data(), w.de[0].data(), w.de[1].data(), w.de[2].data(), Rb.data(), Gb.data()},
                           (uint32_t)1 << le, tE, konstE, mE);
    }
    const gl_t yEX = claimc(P, tr, xc.lg, X, rE), yEY = claimc(P, tr, xc.lg, Y, rE);
    gl_t yE[3];
    for (int k = 0; k < 3; k++) yE[k] = claimc(P, tr, xc.lg, CE[k], rE);
    const gl_t yER = claimc(P, tr, xc.lg, CB[B_R], std::vector<gl_t>(rE.begin() + ld, rE.end()));
    const gl_t yEG = claimc(P, tr, xc.lg, G, std::vector<gl_t>(rE.begin(), rE.begin() + ld));
    std::vector<uint8_t> out;
    put_raw(out, d2, 8);
    for (int k = 0; k < NDB; k++) put_raw(out, CB[k].root.data(), 32);
    for (int k = 0; k < 3; k++) put_raw(out, CE[k].root.data(), 32);
    put_raw(out, &yM, 8); put_raw(out, &yMX, 8);
    put_raw(out, mS.data(), mS.size() * 8);
    put_raw(out, mB.data(), mB.size() * 8);
    put_raw(out, yB, 8 * NDB);
    put_raw(out, mE.data(), mE.size() * 8);
    put_raw(out, yE, 24);
    put_raw(out, &yEX, 8); put_raw(out, &yEY, 8); put_raw(out, &yER, 8); put_raw(out, &yEG, 8);
    put_raw(out, empty_tail().data(), 8);
    return out;
}

// ---- causal softmax (p3ismx) ----
enum { X_SEL = 0, X_DM, X_EE, X_L0, X_L1, X_L2, X_L3, NXE };
struct SmxWit { DevCol xe[NXE], xb[2], p; DevIdx idxDM, idxL[4], idxMX; };
inline SmxWit ismx_witness(Prover& P, IgTables& T, const DevCol& z, uint32_t la, uint32_t lseq) {
    SmxWit w;
    const size_t NR = (size_t)1 << (la + lseq), n = (size_t)1 << (la + 2 * lseq);
    uint64_t* xe[NXE]; uint64_t* xb[2]; uint32_t* il[4];
    for (int k = 0; k < NXE; k++) { w.xe[k] = DevCol(P, n); xe[k] = w.xe[k].data(); }
    for (int k = 0; k < 2; k++) { w.xb[k] = DevCol(P, NR); xb[k] = w.xb[k].data(); }
    for (int k = 0; k < 4; k++) { w.idxL[k] = DevIdx(P, n); il[k] = w.idxL[k].data(); }
    w.p = DevCol(P, n);
    w.idxDM = DevIdx(P, n);
    w.idxMX = DevIdx(P, NR);
    P.ck(zkh_ig_softmax_witness(P.ctx(), z.data(), T.EXPT.on(P)[1].data(), la, lseq, xe, xb, w.p.data(), w.idxDM.data(), il, w.idxMX.data()));
    return w;
}
// p3ismx::prove.  Proof: u32 la lseq | 7 element roots | 2 row roots | mSel ySel | ySrow mS ySE | mE yEZ yE[7] yEP yEMX yES | tail
inline std::vector<uint8_t> ismx_prove(Prover& P, Transcript& tr, IgTables& T, const CCol& Z, const CCol& Pc, SmxWit& w, uint32_t la,
                                       uint32_t lseq, uint32_t R, XCtx& xc) {
    const uint32_t lr = la + lseq, le = la + 2 * lseq;
    uint32_t d2[2] = {la, lseq};
    tr.absorb("ism-dims", d2, 8);
    tr.absorb("ism-Z", Z.root.data(), 32);
    tr.absorb("ism-P", Pc.root.data(), 32);
    CCol CE[NXE], CB[2];
    for (int k = 0; k < NXE; k++) { CE[k] = {&w.xe[k], P.commit_gpu_rootonly(w.xe[k], R)}; tr.absorb("ism-ce", CE[k].root.data(), 32); }
    for (int k = 0; k < 2; k++) CB[k] = {&w.xb[k], P.commit_gpu_rootonly(w.xb[k], R)};
    for (int k = 0; k < 2; k++) tr.absorb("ism-cb", CB[k].root.data(), 32);
    defer(xc, {CE[X_DM], CE[X_EE]}, &w.idxDM, &T.EXPT);
    for (int l = 0; l < 4; l++) defer(xc, {CE[X_L0 + l]}, &w.idxL[l], &T.R16);
    defer(xc, {CB[0]}, &w.idxMX, &T.RS16);
    std::vector<gl_t> mSel, mS, mE;
    // SEL row sum: sum_j SEL = 1, weighted by eq(zb, row)
    std::vector<gl_t> zb(lr);
    for (auto& v : zb) v = tr.chal();
    std::vector<gl_t> rS;
    {
        DevCol eqb = P.build_eq_gpu(zb);
        DevCol EQb = bcast_rows(P, eqb, lseq);
        rS = P.sc_prove_zc(tr, "ism-scsel", {EQb.data(), w.xe[X_SEL].data()}, (uint32_t)1 << le, {{1, {1}}}, 0, mSel);
    }
    const gl_t ySel = claimc(P, tr, xc.lg, CE[X_SEL], rS);
    // S row sum: sum_j EE = S
    for (auto& v : zb) v = tr.chal();
    const gl_t ySrow = claimc(P, tr, xc.lg, CB[1], zb);
    std::vector<gl_t> rS2;
    {
        DevCol eqb = P.build_eq_gpu(zb);
        DevCol EQb = bcast_rows(P, eqb, lseq);
        rS2 = P.sc_prove_zc(tr, "ism-scs", {EQb.data(), w.xe[X_EE].data()}, (uint32_t)1 << le, {{1, {1}}}, 0, mS);
    }
    const gl_t ySE = claimc(P, tr, xc.lg, CE[X_EE], rS2);
    // per-element zero-check (zkllm-src/p3_int_gadgets.cuh:1604-1622): columns 0 E, 1 Z, 2.. the seven element columns, P,
    // MX broadcast, S broadcast, causal mask
    std::vector<gl_t> zE(le);
    for (auto& v : zE) v = tr.chal();
    const gl_t lamE = tr.chal();
    gl_t lam[5];
    for (int k = 0; k < 5; k++) lam[k] = gl_powmod(lamE, k);
    auto n = [](gl_t x) { return gl_neg(x); };
    auto ce = [](int k) { return (uint8_t)(2 + k); };
    const uint8_t Zc = 1, Pk = 2 + NXE, MXb = 3 + NXE, Sb = 4 + NXE, MK = 5 + NXE;
    std::vector<Term> terms = {
        {lam[0], {ce(X_SEL), ce(X_SEL)}}, {n(lam[0]), {ce(X_SEL)}},
        {lam[1], {ce(X_SEL), ce(X_DM)}},
        {lam[2], {ce(X_DM)}}, {n(lam[2]), {MK, MXb}}, {lam[2], {MK, Zc}}, {gl_mulmod(lam[2], 65536), {MK}},
        {gl_mulmod(lam[3], 131072), {ce(X_EE)}}, {lam[3], {Sb}}, {n(gl_mulmod(lam[3], 2)), {Pk, Sb}}, {n(lam[3]), {ce(X_L0)}},
        {n(gl_mulmod(lam[3], 65536)), {ce(X_L1)}},
        {lam[4], {ce(X_L2)}}, {gl_mulmod(lam[4], 65536), {ce(X_L3)}}, {lam[4], {ce(X_L0)}}, {gl_mulmod(lam[4], 65536), {ce(X_L1)}},
        {n(gl_mulmod(lam[4], 2)), {Sb}},
    };
    const gl_t konst = gl_addmod(n(gl_mulmod(lam[2], 65536)), lam[4]);
    std::vector<gl_t> rE;
    {
        DevCol EE = P.build_eq_gpu(zE);
        DevCol MXc = bcast_rows(P, w.xb[0], lseq), Sc = bcast_rows(P, w.xb[1], lseq);
        DevCol mask(P, (size_t)1 << le);
        P.ck(zkh_ig_causal_mask(P.ctx(), la, lseq, mask.data()));
        std::vector<const gl_t*> cols = {EE.data(), Z.col->data()};
        for (int k = 0; k < NXE; k++) cols.push_back(w.xe[k].data());
        cols.push_back(Pc.col->data());
        cols.push_back(MXc.data());
        cols.push_back(Sc.data());
        cols.push_back(mask.data());
        rE = P.sc_prove_zc(tr, "ism-sce", cols, (uint32_t)1 << le, terms, konst, mE);
    }
    const gl_t yEZ = claimc(P, tr, xc.lg, Z, rE);
    gl_t yE[NXE];
    for (int k = 0; k < NXE; k++) yE[k] = claimc(P, tr, xc.lg, CE[k], rE);
    const gl_t yEP = claimc(P, tr, xc.lg, Pc, rE);
    const std::vector<gl_t> rb(rE.begin() + lseq, rE.end());
    const gl_t yEMX = claimc(P, tr, xc.lg, CB[0], rb), yES = claimc(P, tr, xc.lg, CB[1], rb);
    std::vector<uint8_t> out;
    put_raw(out, d2, 8);
    for (int k = 0; k < NXE; k++) put_raw(out, CE[k].root.data(), 32);
    for (int k = 0; k < 2; k++) put_raw(out, CB[k].root.data(), 32);
    put_raw(out, mSel.data(), mSel.size() * 8);
    put_raw(out, &ySel, 8);
    put_raw(out, &ySrow, 8);
    put_raw(out, mS.data(), mS.size() * 8);
    put_raw(out, &ySE, 8);
    put_raw(out, mE.data(), mE.size() * 8);
    put_raw(out, &yEZ, 8);
    put_raw(out, yE, 8 * NXE);
    put_raw(out, &yEP, 8); put_raw(out, &yEMX, 8); put_raw(out, &yES, 8);
    put_raw(out, empty_tail().data(), 8);
    return out;
}

// ---- the decoder layer (p3itf) ----
enum { W_Q = 0, W_K, W_V, W_O, W_G, W_U, W_D };

// p3itf::Config: all dimensions powers of two, nh * dh == d
struct ItfConfig {
    uint32_t seq, d, nh, dh, dff, batch;
    uint32_t lseq, ld, lnh, ldh, ldff, lbb, lT, la, A, tsh, sfz, btop;
    ItfConfig(uint32_t seq_, uint32_t d_, uint32_t nh_, uint32_t dh_, uint32_t dff_, uint32_t batch_ = 1)
        : seq(seq_), d(d_), nh(nh_), dh(dh_), dff(dff_), batch(batch_) {
        auto lg = [](uint32_t x) { uint32_t l = 0; while ((1u << l) < x) l++; return l; };
        lseq = lg(seq); ld = lg(d); lnh = lg(nh); ldh = lg(dh); ldff = lg(dff); lbb = lg(batch);
        if ((1u << lseq) != seq || (1u << ld) != d || (1u << lnh) != nh || (1u << ldh) != dh || (1u << ldff) != dff || (1u << lbb) != batch ||
            nh * dh != d)
            throw std::runtime_error("itf: config must be pow2 with nh*dh == d");
        lT = lseq + lbb; la = lnh + lbb; A = batch * nh;
        tsh = (ldh + 1) / 2;          // power-of-two softmax temperature
        sfz = 24 + tsh;               // scores rescale shift
        btop = sfz - 16;              // width of the top-limb table
    }
    size_t wrows(int i) const { return i == W_D ? dff : d; }
    size_t wcols(int i) const { return (i == W_G || i == W_U) ? dff : d; }
};
// xview_qk / wview_qk / yview_qk (zkllm-src/p3_int_layer.cuh:96-122): scores of head h, batch b, Y = RQ_h . RK_h^T
inline Views views_qk(const ItfConfig& c, uint32_t h, uint32_t b) {
    const uint32_t a = b * c.nh + h;
    Views v;
    v.x = view_run(S_J, c.ldh); view_cat(v.x, view_consts(c.lnh, h)); view_cat(v.x, view_run(S_A, c.lseq)); view_cat(v.x, view_consts(c.lbb, b));
    v.w = v.x;
    v.y = view_run(S_A, c.lseq); view_cat(v.y, view_run(S_I, c.lseq)); view_cat(v.y, view_consts(c.la, a));
    return v;
}
// xview_pv / wview_pv / yview_pv (zkllm-src/p3_int_layer.cuh:124-148): attention output of head h, batch b
inline Views views_pv(const ItfConfig& c, uint32_t h, uint32_t b) {
    const uint32_t a = b * c.nh + h;
    Views v;
    v.x = view_run(S_J, c.lseq); view_cat(v.x, view_run(S_A, c.lseq)); view_cat(v.x, view_consts(c.la, a));
    v.w = view_run(S_A, c.ldh); view_cat(v.w, view_consts(c.lnh, h)); view_cat(v.w, view_run(S_J, c.lseq)); view_cat(v.w, view_consts(c.lbb, b));
    v.y = view_run(S_A, c.ldh); view_cat(v.y, view_consts(c.lnh, h)); view_cat(v.y, view_run(S_I, c.lseq)); view_cat(v.y, view_consts(c.lbb, b));
    return v;
}

// signed 32-bit integers in page-locked host memory (uploads need no staging copy)
class HostI32 {
  public:
    HostI32() = default;
    HostI32(Prover& P, size_t n) : ctx_(P.ctx()), n_(n) {
        void* p = nullptr;
        P.ck(zkh_host_alloc(ctx_, n * 4, &p));
        ptr_ = static_cast<int32_t*>(p);
    }
    HostI32(HostI32&& o) noexcept : ctx_(o.ctx_), ptr_(o.ptr_), n_(o.n_) { o.ptr_ = nullptr; }
    HostI32& operator=(HostI32&& o) noexcept {
        if (this != &o) { if (ptr_) zkh_host_free(ctx_, ptr_); ctx_ = o.ctx_; ptr_ = o.ptr_; n_ = o.n_; o.ptr_ = nullptr; }
        return *this;
    }
    HostI32(const HostI32&) = delete;
    HostI32& operator=(const HostI32&) = delete;
    ~HostI32() { if (ptr_) zkh_host_free(ctx_, ptr_); }
    int32_t* data() const { return ptr_; }
    size_t size() const { return n_; }

  private:
    zkh_ctx* ctx_ = nullptr;
    int32_t* ptr_ = nullptr;
    size_t n_ = 0;
};

// the layer's inputs as a weight loader keeps them: signed 32-bit integers on the host
struct ItfInputs {
    HostI32 x0, w[7], g1, g2, ct, st;                  // ct, st: RoPE tables [seq][dh / 2] at scale 2^14
    ItfInputs(Prover& P, const ItfConfig& c) {
        x0 = HostI32(P, (size_t)c.seq * c.batch * c.d);
        for (int i = 0; i < 7; i++) w[i] = HostI32(P, c.wrows(i) * c.wcols(i));
        g1 = HostI32(P, c.d);
        g2 = HostI32(P, c.d);
        ct = HostI32(P, (size_t)c.seq * c.dh / 2);
        st = HostI32(P, (size_t)c.seq * c.dh / 2);
    }
};

// everything p3itf::build_witness produces, resident on the device
struct ItfWit {
    DevCol x0, W[7], g1, g2;
    DevIdx idxW[7], idxG1, idxG2, idxX0, ct, st;       // ct, st hold int32 values
    RmsWit rms1, rms2;
    DevCol acc[7], sc, pva, res1, out;
    IrsWit rsq, rsk, rsv, rsz, rsat, rso, rsg, rsu, rsd;
    RopeWit rpq, rpk;
    SmxWit smx;
    SwgWit swg;
    DevIdx idxRes1, idxOut;
};

inline DevIdx upload_i32(Prover& P, const HostI32& v) {
    DevIdx raw(P, v.size());
    P.ck(zkh_upload(P.ctx(), raw.data(), v.data(), v.size() * 4));
    return raw;
}
inline DevCol upload_lifted(Prover& P, const HostI32& v) {
    DevIdx raw = upload_i32(P, v);
    DevCol out(P, v.size());
    P.ck(zkh_gl_lift_i32(P.ctx(), reinterpret_cast<const int32_t*>(raw.data()), v.size(), out.data()));
    return out;
}
inline DevIdx rs20_index(Prover& P, const DevCol& c) {
    DevIdx idx(P, c.size());
    P.ck(zkh_ig_rs20_index(P.ctx(), c.data(), c.size(), idx.data()));
    return idx;
}
inline RopeWit irope_witness(Prover& P, const DevCol& q, const DevIdx& ct, const DevIdx& st, uint32_t lseq, uint32_t ldh, uint32_t lT, uint32_t ld) {
    RopeWit w;
    const size_t n = (size_t)1 << (lT + ld);
    w.y = DevCol(P, n); w.rem = DevCol(P, n); w.C = DevCol(P, n); w.S2 = DevCol(P, n);
    w.iR = DevIdx(P, n); w.iY = DevIdx(P, n);
    P.ck(zkh_ig_rope_witness(P.ctx(), q.data(), reinterpret_cast<const int32_t*>(ct.data()), reinterpret_cast<const int32_t*>(st.data()), lseq, ldh,
                             lT, ld, w.y.data(), w.rem.data(), w.iR.data(), w.iY.data(), reinterpret_cast<int64_t*>(w.C.data()),
                             reinterpret_cast<int64_t*>(w.S2.data())));
    // the public columns come back as signed integers: lift them in place
    P.ck(zkh_gl_lift_i64(P.ctx(), reinterpret_cast<const int64_t*>(w.C.data()), n, w.C.data()));
    P.ck(zkh_gl_lift_i64(P.ctx(), reinterpret_cast<const int64_t*>(w.S2.data()), n, w.S2.data()));
    return w;
}
inline DevCol ig_matmul(Prover& P, const DevCol& A, const int64_t sa[4], const DevCol& B, const int64_t sb[4], size_t out_n, const int64_t sc[4],
                        uint32_t nb0, uint32_t nb1, uint32_t I, uint32_t J, uint32_t K) {
    DevCol C(P, out_n);
    P.ck(zkh_ig_matmul(P.ctx(), A.data(), sa, B.data(), sb, C.data(), sc, nb0, nb1, I, J, K));
    return C;
}
// (rows x K) . (K x N), both row-major
inline DevCol ig_mat(Prover& P, const DevCol& X, const DevCol& Wm, uint32_t K, uint32_t N) {
    const uint32_t rows = (uint32_t)(X.size() / K);
    const int64_t sa[4] = {0, 0, (int64_t)K, 1}, sb[4] = {0, 0, (int64_t)N, 1}, sc[4] = {0, 0, (int64_t)N, 1};
    return ig_matmul(P, X, sa, Wm, sb, (size_t)rows * N, sc, 1, 1, rows, K, N);
}

// p3itf::build_witness on the device: the seven weight products and the per-head score / attention-output products in the exact
// integer GEMM (strided views, no gathers), every gadget's replay in its kernel
inline void itf_build_witness(Prover& P, const ItfConfig& c, IgTables& T, const ItfInputs& in, ItfWit& w) {
    const uint32_t ld = c.ld, lT = c.lT, lseq = c.lseq, ldh = c.ldh, la = c.la;
    w.x0 = upload_lifted(P, in.x0);
    for (int i = 0; i < 7; i++) w.W[i] = upload_lifted(P, in.w[i]);
    w.g1 = upload_lifted(P, in.g1);
    w.g2 = upload_lifted(P, in.g2);
    w.ct = upload_i32(P, in.ct);
    w.st = upload_i32(P, in.st);
    for (int i = 0; i < 7; i++) w.idxW[i] = rs20_index(P, w.W[i]);
    w.idxG1 = rs20_index(P, w.g1);
    w.idxG2 = rs20_index(P, w.g2);
    w.idxX0 = rs20_index(P, w.x0);
    const int64_t seq = c.seq, nh = c.nh, dh = c.dh, dm = c.d;
    w.rms1 = irms_witness(P, T, w.x0, w.g1, lT, ld);
    for (int i : {W_Q, W_K, W_V}) w.acc[i] = ig_mat(P, w.rms1.y, w.W[i], c.d, c.d);
    w.rsq = irs_witness(P, w.acc[W_Q], 16, 1);
    w.rsk = irs_witness(P, w.acc[W_K], 16, 1);
    w.rsv = irs_witness(P, w.acc[W_V], 16, 1);
    w.rpq = irope_witness(P, w.rsq.y, w.ct, w.st, lseq, ldh, lT, ld);
    w.rpk = irope_witness(P, w.rsk.y, w.ct, w.st, lseq, ldh, lT, ld);
    {   // sc[a][i][k] = sum_j RQ[b][i][h][j] RK[b][k][h][j], a = b nh + h; activations are laid out (batch, position, head, lane)
        const int64_t sa[4] = {seq * dm, dh, dm, 1}, sb[4] = {seq * dm, dh, 1, dm}, sc[4] = {nh * seq * seq, seq * seq, seq, 1};
        w.sc = ig_matmul(P, w.rpq.y, sa, w.rpk.y, sb, (size_t)1 << (la + 2 * lseq), sc, c.batch, c.nh, c.seq, c.dh, c.seq);
    }
    w.rsz = irs_witness(P, w.sc, c.sfz, 2);
    w.smx = ismx_witness(P, T, w.rsz.y, la, lseq);
    {   // PVA[b][i][h][k] = sum_j P[a][i][j] YV[b][j][h][k]
        const int64_t sa[4] = {nh * seq * seq, seq * seq, seq, 1}, sb[4] = {seq * dm, dh, dm, 1}, sc[4] = {seq * dm, dh, dm, 1};
        w.pva = ig_matmul(P, w.smx.p, sa, w.rsv.y, sb, (size_t)1 << (lT + ld), sc, c.batch, c.nh, c.seq, c.seq, c.dh);
    }
    w.rsat = irs_witness(P, w.pva, 16, 1);
    w.acc[W_O] = ig_mat(P, w.rsat.y, w.W[W_O], c.d, c.d);
    w.rso = irs_witness(P, w.acc[W_O], 16, 1);
    const size_t ne = (size_t)1 << (lT + ld);
    w.res1 = DevCol(P, ne); w.idxRes1 = DevIdx(P, ne);
    P.ck(zkh_ig_add_witness(P.ctx(), w.x0.data(), w.rso.y.data(), ne, w.res1.data(), w.idxRes1.data()));
    w.rms2 = irms_witness(P, T, w.res1, w.g2, lT, ld);
    for (int i : {W_G, W_U}) w.acc[i] = ig_mat(P, w.rms2.y, w.W[i], c.d, c.dff);
    w.rsg = irs_witness(P, w.acc[W_G], 16, 1);
    w.rsu = irs_witness(P, w.acc[W_U], 16, 1);
    {
        const size_t nf = w.rsg.y.size();
        w.swg.sil = DevCol(P, nf); w.swg.rem = DevCol(P, nf); w.swg.mo = DevCol(P, nf);
        w.swg.iG = DevIdx(P, nf); w.swg.iR = DevIdx(P, nf); w.swg.iM = DevIdx(P, nf);
        P.ck(zkh_ig_swiglu_witness(P.ctx(), w.rsg.y.data(), w.rsu.y.data(), T.SILU.on(P)[1].data(), nf, w.swg.sil.data(), w.swg.rem.data(),
                                   w.swg.mo.data(), w.swg.iG.data(), w.swg.iR.data(), w.swg.iM.data()));
    }
    w.acc[W_D] = ig_mat(P, w.swg.mo, w.W[W_D], c.dff, c.d);
    w.rsd = irs_witness(P, w.acc[W_D], 16, 1);
    w.out = DevCol(P, ne); w.idxOut = DevIdx(P, ne);
    P.ck(zkh_ig_add_witness(P.ctx(), w.res1.data(), w.rsd.y.data(), ne, w.out.data(), w.idxOut.data()));
}

// p3itf::commit_all, non-zk: every chain grid, weight, gain and accumulator committed once
struct ItfCom {
    CCol x0, h1, yq, yk, yv, rq, rk, sc, z, p, pva, at, yo, res1, h2, gg, uu, mo, yd, out, g1, g2, w[7], acc[7];
};
inline ItfCom itf_commit_all(Prover& P, ItfWit& w, uint32_t R) {
    auto com = [&](const DevCol& c) { return CCol{&c, P.commit_gpu_rootonly(c, R)}; };
    ItfCom o;
    o.x0 = com(w.x0); o.h1 = com(w.rms1.y); o.yq = com(w.rsq.y); o.yk = com(w.rsk.y); o.yv = com(w.rsv.y);
    o.rq = com(w.rpq.y); o.rk = com(w.rpk.y); o.sc = com(w.sc); o.z = com(w.rsz.y); o.p = com(w.smx.p);
    o.pva = com(w.pva); o.at = com(w.rsat.y); o.yo = com(w.rso.y); o.res1 = com(w.res1); o.h2 = com(w.rms2.y);
    o.gg = com(w.rsg.y); o.uu = com(w.rsu.y); o.mo = com(w.swg.mo); o.yd = com(w.rsd.y); o.out = com(w.out);
    o.g1 = com(w.g1); o.g2 = com(w.g2);
    for (int i = 0; i < 7; i++) o.w[i] = com(w.W[i]);
    for (int i = 0; i < 7; i++) o.acc[i] = com(w.acc[i]);
    return o;
}

// p3itf::prove, non-zk: all sub-proofs in fixed order on one transcript with one ledger and one lookup queue, one merged-lookup
// flush, the public input / output bindings, one batched opening per size class.  Serialised TfProof: 6 x u32 dims | 24 + 2A
// length-prefixed sub-proofs in proving order | 27 roots | u32 groups (len, GroupProof)* | ioin ioout | u32 batches (len, BatchProof)*
inline std::vector<uint8_t> itf_prove(Prover& P, Transcript& tr, const ItfConfig& c, IgTables& T, ItfWit& w, const ItfCom& o, uint32_t R,
                                      uint32_t Q) {
    const uint32_t ld = c.ld, lT = c.lT, ldff = c.ldff, lseq = c.lseq, ldh = c.ldh, la = c.la;
    const uint32_t le = ld + lT, lef = ldff + lT, lez = la + 2 * lseq;
    XCtx xc;
    uint32_t dims[6] = {c.seq, c.d, c.nh, c.dh, c.dff, c.batch};
    tr.absorb("itf-dims", dims, 24);
    for (int i = 0; i < 7; i++) defer(xc, {o.w[i]}, &w.idxW[i], &T.RS20);
    defer(xc, {o.g1}, &w.idxG1, &T.RS20);
    defer(xc, {o.g2}, &w.idxG2, &T.RS20);
    defer(xc, {o.x0}, &w.idxX0, &T.RS20);
    std::vector<std::vector<uint8_t>> subs;
    auto mm = [&](const CCol& X, const CCol& Wc, const CCol& Y, uint32_t lj, uint32_t lk, uint32_t li, const Views* v = nullptr) {
        subs.push_back(imm_prove_views(P, tr, X, Wc, Y, lj, lk, li, xc, v));
    };
    auto irs = [&](IrsWit& iw, const CCol& X, const CCol& Y, uint32_t lev, uint32_t sf, int rng) {
        subs.push_back(irs_prove_wit(P, tr, T, X, Y, iw, lev, sf, rng, R, xc));
    };
    subs.push_back(irms_prove(P, tr, T, o.x0, o.g1, o.h1, w.rms1, lT, ld, R, xc));
    for (int i : {W_Q, W_K, W_V}) mm(o.h1, o.w[i], o.acc[i], ld, ld, lT);
    irs(w.rsq, o.acc[W_Q], o.yq, le, 16, 1);
    irs(w.rsk, o.acc[W_K], o.yk, le, 16, 1);
    irs(w.rsv, o.acc[W_V], o.yv, le, 16, 1);
    subs.push_back(irope_prove(P, tr, T, o.yq, o.rq, w.rpq, ldh, lT, ld, R, xc));
    subs.push_back(irope_prove(P, tr, T, o.yk, o.rk, w.rpk, ldh, lT, ld, R, xc));
    for (uint32_t b = 0; b < c.batch; b++)
        for (uint32_t h = 0; h < c.nh; h++) {
            const Views v = views_qk(c, h, b);
            mm(o.rq, o.rk, o.sc, ldh, lseq, lseq, &v);
        }
    irs(w.rsz, o.sc, o.z, lez, c.sfz, 2);
    subs.push_back(ismx_prove(P, tr, T, o.z, o.p, w.smx, la, lseq, R, xc));
    for (uint32_t b = 0; b < c.batch; b++)
        for (uint32_t h = 0; h < c.nh; h++) {
            const Views v = views_pv(c, h, b);
            mm(o.p, o.yv, o.pva, lseq, ldh, lseq, &v);
        }
    irs(w.rsat, o.pva, o.at, le, 16, 1);
    mm(o.at, o.w[W_O], o.acc[W_O], ld, ld, lT);
    irs(w.rso, o.acc[W_O], o.yo, le, 16, 1);
    subs.push_back(iadd_prove(P, tr, T, o.x0, o.yo, o.res1, w.idxRes1, le, xc));
    subs.push_back(irms_prove(P, tr, T, o.res1, o.g2, o.h2, w.rms2, lT, ld, R, xc));
    for (int i : {W_G, W_U}) mm(o.h2, o.w[i], o.acc[i], ld, ldff, lT);
    irs(w.rsg, o.acc[W_G], o.gg, lef, 16, 1);
    irs(w.rsu, o.acc[W_U], o.uu, lef, 16, 1);
    subs.push_back(iswg_prove(P, tr, T, o.gg, o.uu, o.mo, w.swg, lef, R, xc));
    mm(o.mo, o.w[W_D], o.acc[W_D], ldff, ld, lT);
    irs(w.rsd, o.acc[W_D], o.yd, le, 16, 1);
    subs.push_back(iadd_prove(P, tr, T, o.res1, o.yd, o.out, w.idxOut, le, xc));
    std::vector<std::vector<uint8_t>> lug = lu_flush(P, tr, xc, R);
    std::vector<gl_t> z1(le), z2(le);
    for (auto& v : z1) v = tr.chal();
    const gl_t ioin = claimc(P, tr, xc.lg, o.x0, z1);
    for (auto& v : z2) v = tr.chal();
    const gl_t ioout = claimc(P, tr, xc.lg, o.out, z2);
    std::vector<std::vector<uint8_t>> batches = tail_prove(P, tr, xc.lg, R, Q, "itf-bo");
    std::vector<uint8_t> out;
    put_raw(out, dims, 24);
    for (auto& s : subs) put_blob(out, s);
    const CCol* roots[] = {&o.x0, &o.h1, &o.acc[0], &o.acc[1], &o.acc[2], &o.acc[3], &o.acc[4], &o.acc[5], &o.acc[6], &o.yq, &o.yk, &o.yv,
                           &o.rq, &o.rk, &o.sc, &o.z, &o.p, &o.pva, &o.at, &o.yo, &o.res1, &o.h2, &o.gg, &o.uu, &o.mo, &o.yd, &o.out};
    for (const CCol* r : roots) put_raw(out, r->root.data(), 32);
    put_u32(out, (uint32_t)lug.size());
    for (auto& x : lug) put_blob(out, x);
    put_raw(out, &ioin, 8); put_raw(out, &ioout, 8);
    put_u32(out, (uint32_t)batches.size());
    for (auto& x : batches) put_blob(out, x);
    return out;
}

}  // namespace zkh_p3
