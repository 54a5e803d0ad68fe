// Host-side verifier for the proofs the C++ prover side (zkh_p3.hpp) writes: the quantised matmul proof, the rescale
// proof with its merged lookups, and the batched Basefold openings behind them -- the verifying half of the reference's
// driver pairs (its verifiers are host code too):
//   p3hwl::sc5_verify       zkllm-src/p3_hawkeye.cuh:781-795      -> sumcheck_verify
//   p3gkr::verify           zkllm-src/p3_gkr.cuh:370-421          -> gkr_verify
//   p3lu::verify_super / lu_verify_flush   zkllm-src/p3_logup.cuh:1958-2113  -> verify_super / lu_verify_flush
//   p3bo::verify_class / subset_verify     zkllm-src/p3_batchopen.cuh:108-131, :1149-1302 -> verify_class
//   p3ig::tail_verify       zkllm-src/p3_int_gadgets.cuh:194-205  -> tail_verify
//   p3imm::verify           zkllm-src/p3_int_gadgets.cuh:608-653  -> imm_verify   (direct layouts, non-zk)
//   p3irs::verify           zkllm-src/p3_int_gadgets.cuh:342-389  -> irs_verify   (non-zk)
// It reads the serialised proofs (byte layouts as documented in zkh.h and zkh_p3.hpp), never touches a GPU, and draws
// the same Fiat-Shamir challenges as the prover, so a proof is accepted here exactly when the reference's verifier
// accepts the same bytes.  Every check that fails names itself in Verdict::why; malformed or truncated input is a
// rejection, never an exception that escapes.
// Header-only; needs only the host functions of libzkh.so (transcript, Merkle hashes).
#pragma once
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <deque>
#include <stdexcept>
#include <string>
#include <vector>

#include "zkh_p3.hpp"

namespace zkh_p3v {

using zkh_p3::gl_t;
using zkh_p3::Hash;
using zkh_p3::Table;
using zkh_p3::Transcript;
constexpr gl_t P = zkh_p3::GL_P;
constexpr uint32_t Q_MIN = 20;            // fewer queries than this are refused (the reference's Q_MIN)

inline gl_t add(gl_t a, gl_t b) { return (gl_t)(((unsigned __int128)a + b) % P); }
inline gl_t sub(gl_t a, gl_t b) { return a >= b ? a - b : a + (P - b); }
inline gl_t mul(gl_t a, gl_t b) { return (gl_t)(((unsigned __int128)a * b) % P); }
inline gl_t pw(gl_t a, uint64_t e) {
    gl_t r = 1;
    for (; e; e >>= 1, a = mul(a, a))
        if (e & 1) r = mul(r, a);
    return r;
}
inline gl_t inv(gl_t a) { return pw(a, P - 2); }
inline gl_t root_of_unity(uint32_t logn) { return pw(pw(7, 0xFFFFFFFFULL), 1ULL << (32 - logn)); }

struct Verdict {
    bool ok = true;
    std::string why = "ok";
    explicit operator bool() const { return ok; }
    static Verdict reject(const std::string& w) { Verdict v; v.ok = false; v.why = w; return v; }
};
struct Malformed : std::runtime_error { using std::runtime_error::runtime_error; };

// bounds-checked cursor over a proof
class Reader {
  public:
    Reader(const uint8_t* p, size_t n) : p_(p), n_(n) {}
    explicit Reader(const std::vector<uint8_t>& b) : p_(b.data()), n_(b.size()) {}
    const uint8_t* take(size_t k) {
        if (k > n_ - off_) throw Malformed("proof truncated");
        const uint8_t* q = p_ + off_;
        off_ += k;
        return q;
    }
    uint32_t u32() { uint32_t v; memcpy(&v, take(4), 4); return v; }
    gl_t gl() {
        gl_t v;
        memcpy(&v, take(8), 8);
        if (v >= P) throw Malformed("non-canonical field element");
        return v;
    }
    std::vector<gl_t> gls(size_t k) {
        if (k > (n_ - off_) / 8) throw Malformed("proof truncated");
        std::vector<gl_t> v(k);
        for (auto& x : v) x = gl();
        return v;
    }
    Hash hash() { Hash h; memcpy(h.data(), take(32), 32); return h; }
    Reader blob() { uint32_t k = u32(); return Reader(take(k), k); }
    size_t left() const { return n_ - off_; }
    bool done() const { return off_ == n_; }

  private:
    const uint8_t* p_;
    size_t n_, off_ = 0;
};

// value at t of the polynomial of degree < n through (0, s[0]) .. (n-1, s[n-1])
inline gl_t interpolate(const gl_t* s, int n, gl_t t) {
    gl_t acc = 0;
    for (int i = 0; i < n; i++) {
        gl_t num = 1, den = 1;
        for (int j = 0; j < n; j++) {
            if (j == i) continue;
            num = mul(num, sub(t, (gl_t)j));
            den = mul(den, sub((gl_t)i, (gl_t)j));
        }
        acc = add(acc, mul(s[i], mul(num, inv(den))));
    }
    return acc;
}
inline gl_t eq_point(const std::vector<gl_t>& a, const std::vector<gl_t>& z) {
    gl_t prod = 1;
    for (size_t i = 0; i < a.size(); i++) prod = mul(prod, add(mul(a[i], z[i]), mul(sub(1, a[i]), sub(1, z[i]))));
    return prod;
}
inline std::vector<gl_t> eq_table(const std::vector<gl_t>& z) {
    std::vector<gl_t> e(1, 1);
    for (size_t i = 0; i < z.size(); i++) {          // variable i is bit i of the index
        std::vector<gl_t> nx(e.size() * 2);
        for (size_t b = 0; b < e.size(); b++) { nx[b] = mul(e[b], sub(1, z[i])); nx[b + e.size()] = mul(e[b], z[i]); }
        e.swap(nx);
    }
    return e;
}

// rounds of a sumcheck with nt evaluations per message: claim0 = s(0) + s(1), absorb, challenge, next claim
inline bool sumcheck_verify(Reader& rd, uint32_t v, int nt, gl_t claim0, Transcript& tr, const char* tag, std::vector<gl_t>& r,
                            gl_t& claim) {
    claim = claim0;
    r.clear();
    for (uint32_t k = 0; k < v; k++) {
        const uint8_t* raw = rd.take((size_t)nt * 8);
        gl_t s[5];
        for (int t = 0; t < nt; t++) { memcpy(&s[t], raw + 8 * t, 8); if (s[t] >= P) return false; }
        if (add(s[0], s[1]) != claim) return false;
        tr.absorb(tag, raw, (size_t)nt * 8);
        const gl_t a = tr.chal();
        r.push_back(a);
        claim = interpolate(s, nt, a);
    }
    return true;
}

// ---- verifier's opening ledger (p3bo::VLedger): claims grouped by number of variables ----
struct VLedger {
    struct Ent { Hash root; uint32_t zid; gl_t y; };
    struct Cls { uint32_t v; std::vector<std::vector<gl_t>> pts; std::vector<Ent> ents; };
    std::vector<Cls> cls;
    void add(const Hash& root, const std::vector<gl_t>& z, gl_t y) {
        for (auto& c : cls)
            if (c.v == z.size()) {
                uint32_t zid = 0;
                for (; zid < c.pts.size(); zid++) if (c.pts[zid] == z) break;
                if (zid == c.pts.size()) c.pts.push_back(z);
                c.ents.push_back({root, zid, y});
                return;
            }
        cls.push_back({(uint32_t)z.size(), {z}, {{root, 0, y}}});
    }
};
// a claimed evaluation of a committed column: absorbed, recorded for the batched opening
inline gl_t claimv(Transcript& tr, VLedger& lg, const Hash& root, const std::vector<gl_t>& z, gl_t y) {
    tr.absorb("hwl-y", &y, 8);
    lg.add(root, z, y);
    return y;
}

// ---- Merkle ----
inline Hash leaf_hash(gl_t v) { Hash h; zkh_merkle_leaf_hash(v, h.data()); return h; }
inline Hash node_hash(const Hash& l, const Hash& r) { Hash h; zkh_merkle_node_hash(l.data(), r.data(), h.data()); return h; }
inline bool path_ok(Hash h, size_t idx, const uint8_t* path, uint32_t len, const Hash& root) {
    for (uint32_t l = 0; l < len; l++, idx >>= 1) {
        Hash sib;
        memcpy(sib.data(), path + 32 * l, 32);
        h = (idx & 1) ? node_hash(sib, h) : node_hash(h, sib);
    }
    return h == root;
}
// sorted distinct leaf positions with their hashes, and the siblings the prover had to send, level by level
inline bool subset_ok(uint32_t logM, const std::vector<uint32_t>& pos, std::vector<Hash> cur, Reader& nodes, uint32_t nnodes,
                      const Hash& root) {
    std::vector<uint32_t> idx(pos);
    uint32_t used = 0;
    for (uint32_t l = 0; l < logM; l++) {
        std::vector<uint32_t> nidx;
        std::vector<Hash> nh;
        for (size_t i = 0; i < idx.size();) {
            if (!(idx[i] & 1) && i + 1 < idx.size() && idx[i + 1] == (idx[i] | 1)) {
                nh.push_back(node_hash(cur[i], cur[i + 1]));
                nidx.push_back(idx[i] >> 1);
                i += 2;
            } else {
                if (used == nnodes) return false;
                const Hash sib = nodes.hash();
                used++;
                nh.push_back((idx[i] & 1) ? node_hash(sib, cur[i]) : node_hash(cur[i], sib));
                nidx.push_back(idx[i] >> 1);
                i += 1;
            }
        }
        idx.swap(nidx);
        cur.swap(nh);
    }
    return used == nnodes && cur.size() == 1 && cur[0] == root;
}

// ---- batched opening of one size class ----
inline Verdict verify_class(Transcript& tr, const VLedger::Cls& C, Reader pf, uint32_t Q, uint32_t R, const std::string& label) {
    const uint32_t v = C.v, logM0 = v + R;
    if (v < 1 || logM0 > 31) return Verdict::reject("batch size");
    const uint32_t M0 = 1u << logM0, T = (uint32_t)C.pts.size();
    const size_t k = C.ents.size();
    if (pf.u32() != v || pf.u32() != R || pf.u32() != Q) return Verdict::reject("batch params");
    std::vector<Hash> droots;                        // distinct columns by root, first appearance
    std::vector<uint32_t> colidx(k);
    for (size_t j = 0; j < k; j++) {
        uint32_t c = 0;
        while (c < droots.size() && !(droots[c] == C.ents[j].root)) c++;
        if (c == droots.size()) droots.push_back(C.ents[j].root);
        colidx[j] = c;
    }
    const uint32_t nc = (uint32_t)droots.size();
    if (pf.u32() != nc) return Verdict::reject("batch col count");
    const std::vector<gl_t> ystar = pf.gls(nc);

    const gl_t mu = tr.chal();
    gl_t claim = 0, w = 1;
    for (size_t j = 0; j < k; j++) { claim = add(claim, mul(w, C.ents[j].y)); w = mul(w, mu); }
    std::vector<gl_t> rstar;
    if (!sumcheck_verify(pf, v, 3, claim, tr, "bo-rm", rstar, claim)) return Verdict::reject("batch reduction claim");
    // the proof keeps its sections in struct order: roots and opening messages follow the reduction messages
    std::vector<Hash> roots(v - 1);
    for (auto& h : roots) h = pf.hash();
    tr.absorb("bo-ys", ystar.data(), (size_t)nc * 8);
    {
        std::vector<gl_t> gt(T, 0);
        w = 1;
        for (size_t j = 0; j < k; j++) { gt[C.ents[j].zid] = add(gt[C.ents[j].zid], mul(w, ystar[colidx[j]])); w = mul(w, mu); }
        gl_t end = 0;
        for (uint32_t t = 0; t < T; t++) end = add(end, mul(eq_point(rstar, C.pts[t]), gt[t]));
        if (end != claim) return Verdict::reject("batch reduction terminal");
    }
    const gl_t rho = tr.chal();
    std::vector<gl_t> rhop(nc);
    gl_t yU = 0;
    w = 1;
    for (uint32_t c = 0; c < nc; c++) { rhop[c] = w; yU = add(yU, mul(w, ystar[c])); w = mul(w, rho); }

    // the opening of U = sum_c rho^c col_c at r* on its own transcript; round 0 has no root of its own
    Transcript ot(label);
    ot.absorb("z", rstar.data(), (size_t)v * 8);
    ot.absorb("y", &yU, 8);
    std::vector<gl_t> alphas(v);
    gl_t oclaim = yU;
    for (uint32_t r = 0; r < v; r++) {
        if (r > 0) ot.absorb("root", roots[r - 1].data(), 32);
        const uint8_t* raw = pf.take(24);
        gl_t s[3];
        memcpy(s, raw, 24);
        if (s[0] >= P || s[1] >= P || s[2] >= P || add(s[0], s[1]) != oclaim) return Verdict::reject("batch opening claim");
        ot.absorb("sc", raw, 24);
        alphas[r] = ot.chal();
        oclaim = interpolate(s, 3, alphas[r]);
    }
    const std::vector<gl_t> fin = pf.gls((size_t)1 << R);
    ot.absorb("final", fin.data(), fin.size() * 8);
    for (gl_t x : fin) if (x != fin[0]) return Verdict::reject("batch final not constant");
    if (oclaim != mul(fin[0], eq_point(alphas, rstar))) return Verdict::reject("batch eval tie");

    std::vector<uint32_t> c0q(Q), upos;
    for (uint32_t q = 0; q < Q; q++) {
        c0q[q] = (uint32_t)ot.idx(M0 / 2);
        upos.push_back(c0q[q]);
        upos.push_back(c0q[q] + M0 / 2);
    }
    std::sort(upos.begin(), upos.end());
    upos.erase(std::unique(upos.begin(), upos.end()), upos.end());
    const uint32_t nu = (uint32_t)upos.size();
    auto slot_of = [&](uint32_t p) { return (uint32_t)(std::lower_bound(upos.begin(), upos.end(), p) - upos.begin()); };

    // the per-query section comes first in the bytes, the per-column round-0 openings after it
    size_t per_query = 0;
    for (uint32_t r = 1; r < v; r++) per_query += 16 + (size_t)64 * (logM0 - r);
    Reader qsec(pf.take((size_t)Q * per_query), (size_t)Q * per_query);
    std::vector<std::vector<gl_t>> vals(nc);
    for (uint32_t c = 0; c < nc; c++) {
        if (pf.u32() != nu) return Verdict::reject("batch q0 size");
        vals[c] = pf.gls(nu);
        std::vector<Hash> leaves(nu);
        for (uint32_t i = 0; i < nu; i++) leaves[i] = leaf_hash(vals[c][i]);
        const uint32_t nn = pf.u32();
        if ((size_t)nn * 32 > pf.left()) return Verdict::reject("batch q0 nodes");
        Reader nodes(pf.take((size_t)nn * 32), (size_t)nn * 32);
        if (!subset_ok(logM0, upos, leaves, nodes, nn, droots[c])) return Verdict::reject("batch q0 merkle");
    }
    if (!pf.done()) return Verdict::reject("batch trailing bytes");

    const gl_t inv2 = inv(2);
    for (uint32_t q = 0; q < Q; q++) {
        uint32_t p = c0q[q];
        gl_t carried = 0;            // the folded value the next round must show
        for (uint32_t r = 0; r < v; r++) {
            const uint32_t half = (M0 >> r) / 2, c = p % half;
            gl_t a = 0, b = 0;
            if (r == 0) {
                const uint32_t sa = slot_of(c), sb = slot_of(c + half);
                for (uint32_t cc = 0; cc < nc; cc++) { a = add(a, mul(rhop[cc], vals[cc][sa])); b = add(b, mul(rhop[cc], vals[cc][sb])); }
            } else {
                const uint32_t plen = logM0 - r;
                a = qsec.gl();
                b = qsec.gl();
                const uint8_t* pa = qsec.take((size_t)plen * 32);
                const uint8_t* pb = qsec.take((size_t)plen * 32);
                if (!path_ok(leaf_hash(a), c, pa, plen, roots[r - 1])) return Verdict::reject("batch merkle a");
                if (!path_ok(leaf_hash(b), c + half, pb, plen, roots[r - 1])) return Verdict::reject("batch merkle b");
                // the position this round reads is c or c + half of the value folded in the round before
                if ((p < half ? a : b) != carried) return Verdict::reject("batch fold link");
            }
            const gl_t x = pw(root_of_unity(logM0 - r), c);
            const gl_t even = mul(add(a, b), inv2), odd = mul(mul(sub(a, b), inv2), inv(x));
            carried = add(mul(sub(1, alphas[r]), even), mul(alphas[r], odd));
            if (r + 1 == v && fin[c] != carried) return Verdict::reject("batch fold to final");
            p = c;
        }
    }
    return Verdict();
}

// ---- GKR fractional-sum tree ----
// On success rfin and out4 = {p0, p1, q0, q1} leaf claims (combine_last: out4[0], out4[2] = the combined claims).
struct GkrRoot { gl_t Pn = 0, Qd = 0; };
inline Verdict gkr_verify(Transcript& tr, const char* tag, uint32_t L, Reader& pf, bool combine_last, std::vector<gl_t>& rfin,
                          gl_t out4[4], GkrRoot& root) {
    if (L < 1) return Verdict::reject("gkr layer count");
    root.Pn = pf.gl();
    root.Qd = pf.gl();
    if (root.Qd == 0) return Verdict::reject("gkr zero root Q");
    gl_t rt[2] = {root.Pn, root.Qd};
    tr.absorb(tag, rt, 16);
    std::vector<gl_t> z;
    gl_t cp = 0, cq = 0;
    for (uint32_t h = L; h >= 1; h--) {
        const uint32_t rounds = pf.u32(), want = L - h;
        if (rounds != want) return Verdict::reject(h == L ? "gkr root msgs" : "gkr layer msgs");
        std::vector<gl_t> r;
        gl_t claim = 0, lam = 0;
        if (h < L) {
            lam = tr.chal();
            if (!sumcheck_verify(pf, want, 4, add(cp, mul(lam, cq)), tr, tag, r, claim)) return Verdict::reject("gkr round claim");
        }
        const uint8_t* raw = pf.take(32);
        gl_t t4[4];
        memcpy(t4, raw, 32);
        for (gl_t x : t4) if (x >= P) return Verdict::reject("gkr non-canonical");
        const gl_t p0 = t4[0], p1 = t4[1], q0 = t4[2], q1 = t4[3];
        const gl_t num = add(mul(p0, q1), mul(p1, q0)), den = mul(q0, q1);
        if (h == L) {
            if (num != root.Pn) return Verdict::reject("gkr root P");
            if (den != root.Qd) return Verdict::reject("gkr root Q");
        } else if (claim != mul(eq_point(z, r), add(num, mul(lam, den)))) {
            return Verdict::reject("gkr layer terminal");
        }
        tr.absorb(tag, raw, 32);
        if (h > 1 || combine_last) {
            const gl_t mu = tr.chal();
            cp = add(p0, mul(mu, sub(p1, p0)));
            cq = add(q0, mul(mu, sub(q1, q0)));
            z.assign(1, mu);
            z.insert(z.end(), r.begin(), r.end());
            if (h == 1) { rfin = z; out4[0] = cp; out4[1] = 0; out4[2] = cq; out4[3] = 0; }
        } else {
            rfin = r;
            out4[0] = p0; out4[1] = p1; out4[2] = q0; out4[3] = q1;
        }
    }
    return Verdict();
}

// ---- merged lookups ----
// a deferred lookup as the verifier sees it: the roots of its c witness columns (nullptr: virtual), the table, log rows
struct VLookup { std::vector<const Hash*> roots; const Table* tab; uint32_t n; };
struct VCtx {
    VLedger vlg;
    std::vector<VLookup> luq;
    std::deque<Hash> keep;            // roots read from proofs live here while deferred lookups point at them
};
constexpr uint32_t LU_GCAP = zkh_p3::LU_GCAP;

inline Verdict verify_super(Transcript& tr, VCtx& V, const std::vector<std::pair<uint32_t, std::vector<size_t>>>& subs, Reader pf) {
    const Table& T = *V.luq[subs[0].second[0]].tab;
    const size_t M = T.cols[0].size();
    uint32_t m = 0;
    while (((size_t)1 << m) < M) m++;
    const uint32_t c = (uint32_t)T.cols.size(), ns = (uint32_t)subs.size();
    if (pf.u32() != m || pf.u32() != c || pf.u32() != ns) return Verdict::reject("group dims");
    const Hash root_cnt = pf.hash();
    // the table-side tree sits before the subgroups in the bytes but is checked after them: remember where it starts
    Reader gkT_at = pf;
    {   // skip over it: P Q, then per layer u32 rounds | rounds * 32 | 32
        pf.take(16);
        for (uint32_t h = m; h >= 1; h--) { const uint32_t rounds = pf.u32(); pf.take((size_t)rounds * 32 + 32); }
    }
    tr.absorb("lug-tab", T.id.data(), 32);
    uint32_t sd[3] = {ns, m, c};
    tr.absorb("lug-sdims", sd, 12);
    for (auto& sg : subs) {
        const uint32_t n = sg.first, k = (uint32_t)sg.second.size();
        uint32_t g = 0;
        while ((1u << g) < k) g++;
        uint32_t dm[4] = {n, g, k, c};
        tr.absorb("lug-dims", dm, 16);
        for (size_t j : sg.second) {
            if (V.luq[j].roots.size() != c) return Verdict::reject("group root count");
            for (auto* r : V.luq[j].roots) {
                if (r) tr.absorb("lug-W", r->data(), 32);
                else tr.absorb("lug-Wv", "virt", 4);
            }
        }
    }
    tr.absorb("lug-cnt", root_cnt.data(), 32);
    const gl_t gamma = tr.chal(), beta = tr.chal();
    std::vector<gl_t> gp(c);
    gl_t a0 = 0;
    {
        gl_t w = 1;
        for (uint32_t t = 0; t < c; t++) { gp[t] = w; a0 = add(a0, mul(w, T.cols[t][0])); w = mul(w, gamma); }
    }
    gl_t accP = 0, accQ = 1;
    for (auto& sg : subs) {
        const uint32_t n = sg.first, k = (uint32_t)sg.second.size();
        uint32_t g = 0;
        while ((1u << g) < k) g++;
        if (pf.u32() != n || pf.u32() != k) return Verdict::reject("group dims");
        std::vector<gl_t> rA;
        gl_t o4[4];
        GkrRoot rt;
        Verdict vd = gkr_verify(tr, "lug-gA", n + g, pf, true, rA, o4, rt);
        if (!vd) return vd;
        accP = add(mul(accP, rt.Qd), mul(rt.Pn, accQ));
        accQ = mul(accQ, rt.Qd);
        const std::vector<gl_t> pm(rA.begin(), rA.begin() + n);
        auto eq_bits = [&](uint32_t j) {
            gl_t e = 1;
            for (uint32_t t = 0; t < g; t++) e = mul(e, ((j >> t) & 1) ? rA[n + t] : sub(1, rA[n + t]));
            return e;
        };
        gl_t A_r = 0;
        for (uint32_t j = 0; j < k; j++) {
            const VLookup& L = V.luq[sg.second[j]];
            const std::vector<gl_t> yW = pf.gls(pf.u32());
            const std::vector<gl_t> yv = pf.gls(pf.u32());
            const std::vector<gl_t> extra = pf.gls(pf.u32());
            size_t iw = 0, iv = 0;
            gl_t yj = 0;
            for (uint32_t t = 0; t < c; t++) {
                gl_t y;
                if (L.roots[t]) {
                    if (iw >= yW.size()) return Verdict::reject("group yW count");
                    y = yW[iw++];
                    tr.absorb("lug-yW", &y, 8);
                    V.vlg.add(*L.roots[t], pm, y);
                } else {
                    if (iv >= yv.size()) return Verdict::reject("group y_virt count");
                    y = yv[iv++];
                    tr.absorb("lug-yv", &y, 8);
                }
                yj = add(yj, mul(gp[t], y));
            }
            if (iw != yW.size() || iv != yv.size() || !extra.empty()) return Verdict::reject("group claim count");
            A_r = add(A_r, mul(eq_bits(j), yj));
        }
        for (uint32_t j = k; j < (1u << g); j++) A_r = add(A_r, mul(eq_bits(j), a0));
        if (o4[0] != 1) return Verdict::reject("group A p-claim");
        if (o4[2] != add(A_r, beta)) return Verdict::reject("group A terminal");
    }
    if (!pf.done()) return Verdict::reject("group trailing bytes");
    std::vector<gl_t> rT;
    gl_t t4[4];
    GkrRoot rtT;
    Verdict vd = gkr_verify(tr, "lug-gT", m, gkT_at, true, rT, t4, rtT);
    if (!vd) return vd;
    {   // the public table, gamma-combined, at rT
        const std::vector<gl_t> e = eq_table(rT);
        gl_t Tc = 0;
        for (uint32_t t = 0; t < c; t++) {
            gl_t vsum = 0;
            for (size_t j = 0; j < M; j++) vsum = add(vsum, mul(T.cols[t][j], e[j]));
            Tc = add(Tc, mul(gp[t], vsum));
        }
        if (t4[2] != add(Tc, beta)) return Verdict::reject("group T terminal");
    }
    V.vlg.add(root_cnt, rT, t4[0]);
    if (mul(accP, rtT.Qd) != mul(rtT.Pn, accQ)) return Verdict::reject("group multiset");
    return Verdict();
}

inline Verdict lu_verify_flush(Transcript& tr, VCtx& V, Reader& pf) {
    struct Grp { const Table* tab; uint32_t n; std::vector<size_t> mem; };
    std::vector<Grp> groups;
    for (size_t i = 0; i < V.luq.size(); i++) {
        bool placed = false;
        for (auto& g : groups)
            if (g.tab->id == V.luq[i].tab->id && g.n == V.luq[i].n) { g.mem.push_back(i); placed = true; break; }
        if (!placed) groups.push_back({V.luq[i].tab, V.luq[i].n, {i}});
    }
    std::vector<Grp> split;
    for (auto& g : groups) {
        const size_t cap = g.n >= LU_GCAP ? 1 : (size_t)1 << (LU_GCAP - g.n);
        for (size_t off = 0; off < g.mem.size(); off += cap)
            split.push_back({g.tab, g.n, std::vector<size_t>(g.mem.begin() + off, g.mem.begin() + std::min(off + cap, g.mem.size()))});
    }
    struct Sup { const Table* tab; std::vector<std::pair<uint32_t, std::vector<size_t>>> subs; };
    std::vector<Sup> supers;
    for (auto& g : split) {
        bool placed = false;
        for (auto& sp : supers)
            if (sp.tab->id == g.tab->id) { sp.subs.push_back({g.n, g.mem}); placed = true; break; }
        if (!placed) supers.push_back({g.tab, {{g.n, g.mem}}});
    }
    if (pf.u32() != supers.size()) return Verdict::reject("lookup group count");
    for (auto& sp : supers) {
        Verdict vd = verify_super(tr, V, sp.subs, pf.blob());
        if (!vd) return vd;
    }
    V.luq.clear();
    return Verdict();
}

// u32 groups (len, GroupProof)* | u32 batches (len, BatchProof)*  -- the tail of a standalone gadget proof
inline Verdict tail_verify(Transcript& tr, VCtx& V, Reader& pf, uint32_t Q, uint32_t R, const std::string& tag, bool with_lookups) {
    if (with_lookups) {
        Verdict vd = lu_verify_flush(tr, V, pf);
        if (!vd) return vd;
    }
    if (pf.u32() != V.vlg.cls.size()) return Verdict::reject("batch count");
    for (size_t i = 0; i < V.vlg.cls.size(); i++) {
        Verdict vd = verify_class(tr, V.vlg.cls[i], pf.blob(), Q, R, tag + std::to_string(i));
        if (!vd) return vd;
    }
    return Verdict();
}

// ---- quantised matmul, direct layouts: X = [j | i << lj], W = [k | j << lk], Y = [k | i << lk] ----
// shared: claims and lookups go to the caller's context and the proof carries no tail (composed proofs)
inline Verdict imm_verify(Transcript& tr, Reader& pf, const Hash& rX, const Hash& rW, const Hash& rY, uint32_t lj, uint32_t lk,
                          uint32_t li, uint32_t Q, uint32_t R, VCtx* shared = nullptr) {
    if (Q < Q_MIN || R < 1) return Verdict::reject("insecure params");
    if (pf.u32() != lj || pf.u32() != lk || pf.u32() != li) return Verdict::reject("imm dims");
    VCtx own;
    VCtx& V = shared ? *shared : own;
    uint32_t d3[3] = {lj, lk, li};
    tr.absorb("imm-dims", d3, 12);
    tr.absorb("imm-X", rX.data(), 32);
    tr.absorb("imm-W", rW.data(), 32);
    tr.absorb("imm-Y", rY.data(), 32);
    std::vector<gl_t> z(lk + li);
    for (auto& x : z) x = tr.chal();
    // the claimed values sit behind the messages: read them through a second cursor
    const uint32_t lt = lj + lk + li;
    Reader msgs(pf.take((size_t)lt * 40), (size_t)lt * 40);
    const gl_t pyY = pf.gl(), pyX = pf.gl(), pyW = pf.gl();
    const gl_t yY = claimv(tr, V.vlg, rY, z, pyY);
    std::vector<gl_t> r;
    gl_t claim;
    if (!sumcheck_verify(msgs, lt, 5, yY, tr, "imm-sc", r, claim)) return Verdict::reject("imm sumcheck");
    const std::vector<gl_t> rj(r.begin(), r.begin() + lj), rk(r.begin() + lj, r.begin() + lj + lk), ri(r.begin() + lj + lk, r.end());
    std::vector<gl_t> zx(rj), zw(rk), rsel(rk);
    zx.insert(zx.end(), ri.begin(), ri.end());
    zw.insert(zw.end(), rj.begin(), rj.end());
    rsel.insert(rsel.end(), ri.begin(), ri.end());
    const gl_t yX = claimv(tr, V.vlg, rX, zx, pyX), yW = claimv(tr, V.vlg, rW, zw, pyW);
    if (mul(eq_point(rsel, z), mul(yX, yW)) != claim) return Verdict::reject("imm terminal");
    if (!shared) {
        Verdict vd = tail_verify(tr, V, pf, Q, R, "imm-bo", false);
        if (!vd) return vd;
        if (!pf.done()) return Verdict::reject("imm trailing bytes");
    } else if (pf.u32() != 0) {
        return Verdict::reject("unexpected tail");
    }
    return Verdict();
}

// ---- rescale: X + 2^(sf-1) = Y * 2^sf + L0 (+ 2^16 L1), limbs and Y range-checked by lookups ----
inline Verdict irs_verify(Transcript& tr, const zkh_p3::IrsTables& Tb, Reader& pf, const Hash& rX, const Hash& rY, uint32_t le,
                          uint32_t sf, int rng, uint32_t Q, uint32_t R, VCtx* shared = nullptr) {
    if (Q < Q_MIN || R < 1) return Verdict::reject("insecure params");
    const uint32_t nl = sf <= 16 ? 1u : 2u;
    if (pf.u32() != le || pf.u32() != sf || pf.u32() != nl || pf.u32() != (uint32_t)rng) return Verdict::reject("irs dims");
    if (sf < 1 || sf > 32 || le > 40) return Verdict::reject("irs dims");
    VCtx own;
    VCtx& V = shared ? *shared : own;
    uint32_t d4[4] = {le, sf, nl, (uint32_t)rng};
    tr.absorb("irs-dims", d4, 16);
    tr.absorb("irs-X", rX.data(), 32);
    tr.absorb("irs-Y", rY.data(), 32);
    const Hash* rL[2] = {nullptr, nullptr};
    for (uint32_t l = 0; l < nl; l++) {
        V.keep.push_back(pf.hash());
        rL[l] = &V.keep.back();
        tr.absorb("irs-L", rL[l]->data(), 32);
    }
    V.keep.push_back(rY);
    const Hash* keptY = &V.keep.back();
    V.luq.push_back({{rL[0]}, sf == 14 ? &Tb.R14 : &Tb.R16, le});
    if (nl == 2) V.luq.push_back({{rL[1]}, sf == 32 ? &Tb.R16 : &Tb.RTOP, le});
    if (rng) V.luq.push_back({{keptY}, rng == 1 ? &Tb.RS20 : &Tb.RS16, le});
    std::vector<gl_t> zE(le);
    for (auto& x : zE) x = tr.chal();
    Reader msgs(pf.take((size_t)le * 40), (size_t)le * 40);
    const gl_t pyX = pf.gl(), pyY = pf.gl();
    gl_t pyL[2] = {0, 0};
    for (uint32_t l = 0; l < nl; l++) pyL[l] = pf.gl();
    std::vector<gl_t> rE;
    gl_t claim;
    if (!sumcheck_verify(msgs, le, 5, 0, tr, "irs-sc", rE, claim)) return Verdict::reject("irs sumcheck");
    const gl_t yX = claimv(tr, V.vlg, rX, rE, pyX), yY = claimv(tr, V.vlg, rY, rE, pyY);
    gl_t yL[2] = {0, 0};
    for (uint32_t l = 0; l < nl; l++) yL[l] = claimv(tr, V.vlg, *rL[l], rE, pyL[l]);
    gl_t t = sub(add(yX, (gl_t)1 << (sf - 1)), mul(yY, (gl_t)1 << sf));
    t = sub(t, yL[0]);
    if (nl == 2) t = sub(t, mul(yL[1], 65536));
    if (mul(eq_point(rE, zE), t) != claim) return Verdict::reject("irs terminal");
    if (!shared) {
        Verdict vd = tail_verify(tr, V, pf, Q, R, "irs-bo", true);
        if (!vd) return vd;
        if (!pf.done()) return Verdict::reject("irs trailing bytes");
    } else if (pf.u32() != 0 || pf.u32() != 0) {
        return Verdict::reject("unexpected tail");
    }
    return Verdict();
}

// run a verification, turning malformed input into a rejection
template <class F>
inline Verdict guarded(F&& f) {
    try {
        return f();
    } catch (const Malformed& e) {
        return Verdict::reject(e.what());
    } catch (const std::exception& e) {
        return Verdict::reject(std::string("verifier error: ") + e.what());
    }
}

}  // namespace zkh_p3v
