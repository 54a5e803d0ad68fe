// C++ host side over the C ABI (zkh.h), with the reference's names and calling conventions for the proving
// path, so that gadget code written against the reference's header API keeps its shape:
//   fs::Transcript                      -> zkh_p3::Transcript        (zkllm-src/fs_transcript.hpp:115-166)
//   p3sg::sc_prove_gpu                  -> Prover::sc_prove_gpu      (zkllm-src/p3_scgpu.cuh:91-160)
//   p3bf::build_eq_gpu / eval_h_gpu     -> Prover::build_eq_gpu / eval_h_gpu   (zkllm-src/p3_basefold.cuh:247-283)
//   p3bf::commit_gpu_rootonly           -> Prover::commit_gpu_rootonly          (zkllm-src/p3_basefold.cuh:210-227)
//   p3bf::prove_eval_dev                -> Prover::prove_eval_dev               (zkllm-src/p3_basefold.cuh:355-420)
//   p3gkr::prove_dev                    -> Prover::gkr_prove                    (zkllm-src/p3_gkr.cuh:423-429)
//   p3bo::prove_class                   -> Prover::prove_class                  (zkllm-src/p3_batchopen.cuh:307-1147)
//   p3hwl::sc5_run (fp8 constraint summands), the integer gadgets' zero-checks -> Prover::sc5_run / sc_prove_zc
// Errors surface as std::runtime_error carrying the library's message, as the reference throws.  Device columns
// are DevCol objects (RAII over zkh_dev_alloc).  One Prover per GPU; not thread-safe, like the reference.
// Header-only; link with libzkh.so.
#pragma once
#include <algorithm>
#include <array>
#include <cstdint>
#include <cstring>
#include <deque>
#include <map>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "zkh.h"

namespace zkh_p3 {

using gl_t = uint64_t;
using Hash = std::array<uint8_t, 32>;
constexpr gl_t GL_P = 0xFFFFFFFF00000001ULL;

struct Transcript {
    uint8_t state[32];
    explicit Transcript(const std::string& seed) { zkh_tr_init(state, seed.data(), seed.size()); }
    void absorb(const std::string& label, const void* data, size_t len) { zkh_tr_absorb(state, label.c_str(), data, len); }
    void challenge_bytes(uint8_t out[32]) { zkh_tr_challenge_bytes(state, out); }
    gl_t chal() { return zkh_tr_chal(state); }                        // p3lu::chal
    uint64_t idx(uint64_t mod) { return zkh_tr_idx(state, mod); }      // p3fri::idx_from
};

class Prover;

// device column of n field elements
class DevCol {
  public:
    DevCol() = default;
    DevCol(Prover& p, size_t n);
    DevCol(Prover& p, const std::vector<gl_t>& host);
    DevCol(DevCol&& o) noexcept { *this = std::move(o); }
    DevCol& operator=(DevCol&& o) noexcept {
        if (this != &o) { release(); ctx_ = o.ctx_; ptr_ = o.ptr_; n_ = o.n_; o.ptr_ = nullptr; o.n_ = 0; }
        return *this;
    }
    DevCol(const DevCol&) = delete;
    DevCol& operator=(const DevCol&) = delete;
    ~DevCol() { release(); }
    gl_t* data() const { return ptr_; }
    size_t size() const { return n_; }
    std::vector<gl_t> to_host() const;

  private:
    void release() { if (ptr_) zkh_dev_free(ctx_, ptr_); ptr_ = nullptr; }
    zkh_ctx* ctx_ = nullptr;
    gl_t* ptr_ = nullptr;
    size_t n_ = 0;
};

class Prover {
  public:
    explicit Prover(int device = 0, void* stream = nullptr) {
        if (zkh_ctx_create(device, stream, &ctx_) != ZKH_OK) throw std::runtime_error("zkh: cannot create a context on this device");
    }
    ~Prover() { if (ctx_) { release_kept(); zkh_ctx_destroy(ctx_); } }
    Prover(const Prover&) = delete;
    Prover& operator=(const Prover&) = delete;
    zkh_ctx* ctx() const { return ctx_; }
    void ck(int rc) const { if (rc != ZKH_OK) throw std::runtime_error(std::string("zkh: ") + zkh_last_error(ctx_)); }

    // p3sg::sc_prove_gpu<FF, MsgT, NT, MAXC>: returns the round challenges, appends the messages (NT values per round)
    std::vector<gl_t> sc_prove_gpu(Transcript& tr, const char* tag, const std::vector<const gl_t*>& d_cols, uint32_t N,
                                   int functor, int nt, const gl_t* par, uint32_t npar, std::vector<gl_t>& msgs,
                                   std::vector<gl_t>* finals = nullptr) {
        uint32_t logn = 0;
        while ((1u << logn) < N) logn++;
        std::vector<gl_t> r(logn), m((size_t)logn * nt), fin(d_cols.size());
        ck(zkh_sumcheck(ctx_, functor, nt, d_cols.data(), (int)d_cols.size(), logn, par, (int)npar, tag, tr.state, m.data(),
                        r.data(), fin.data()));
        msgs.insert(msgs.end(), m.begin(), m.end());
        if (finals) *finals = fin;
        return r;
    }
    // p3hwl::sc5_run<FF> for the fp8 gadget's constraint summands (ZKH_F_HW_*), lam = the random coefficients
    std::vector<gl_t> sc5_run(Transcript& tr, const char* tag, const std::vector<const gl_t*>& d_cols, uint32_t N, int functor,
                              const std::vector<gl_t>& lam, std::vector<gl_t>& msgs) {
        uint32_t logn = 0;
        while ((1u << logn) < N) logn++;
        std::vector<gl_t> r(logn), m((size_t)logn * 5);
        ck(zkh_sumcheck_wide(ctx_, functor, d_cols.data(), (int)d_cols.size(), logn, lam.data(), (int)lam.size(), tag, tr.state,
                             m.data(), r.data(), nullptr));
        msgs.insert(msgs.end(), m.begin(), m.end());
        return r;
    }
    // eq-weighted zero-check with a term list: d_cols[0] * (konst + sum coef * prod cols[idx]); terms as (coef, indices)
    std::vector<gl_t> sc_prove_zc(Transcript& tr, const char* tag, const std::vector<const gl_t*>& d_cols, uint32_t N,
                                  const std::vector<std::pair<gl_t, std::vector<uint8_t>>>& terms, gl_t konst,
                                  std::vector<gl_t>& msgs) {
        uint32_t logn = 0;
        while ((1u << logn) < N) logn++;
        std::vector<uint64_t> prog = {terms.size(), konst};
        for (auto& t : terms) {
            uint64_t pk = t.second.size();
            for (size_t k = 0; k < t.second.size(); k++) pk |= (uint64_t)t.second[k] << (8 + 8 * k);
            prog.push_back(t.first);
            prog.push_back(pk);
        }
        std::vector<gl_t> r(logn), m((size_t)logn * 5);
        ck(zkh_sumcheck_zerocheck(ctx_, d_cols.data(), (int)d_cols.size(), logn, prog.data(), (int)prog.size(), tag, tr.state,
                                  m.data(), r.data(), nullptr));
        msgs.insert(msgs.end(), m.begin(), m.end());
        return r;
    }
    DevCol build_eq_gpu(const std::vector<gl_t>& z) {
        DevCol E(*this, (size_t)1 << z.size());
        ck(zkh_gl_eq_build(ctx_, z.data(), (uint32_t)z.size(), E.data()));
        return E;
    }
    gl_t eval_h_gpu(const DevCol& c, const std::vector<gl_t>& z) {
        gl_t y = 0;
        ck(zkh_gl_mle_eval(ctx_, c.data(), z.data(), (uint32_t)z.size(), &y));
        return y;
    }
    // keep_trees: commitments leave their codeword and capped Merkle tree in HBM (zkh_basefold_commit_keep) and prove_class
    // reads authentication paths from them instead of encoding and hashing every opened column again.  The kept buffers are
    // found by the column's device address: call release_kept() before a committed column is freed.
    bool keep_trees = false;
    Hash commit_gpu_rootonly(const DevCol& c, uint32_t R) {
        uint32_t v = 0;
        while (((size_t)1 << v) < c.size()) v++;
        Hash h;
        if (keep_trees && c.size() >= 2) {
            Kept k{R, c.size(), nullptr, nullptr};
            ck(zkh_dev_alloc(ctx_, (c.size() << R) * sizeof(gl_t), &k.cw));
            ck(zkh_dev_alloc(ctx_, zkh_basefold_kept_tree_bytes(v + R), &k.tree));
            ck(zkh_basefold_commit_keep(ctx_, c.data(), v, R, static_cast<uint64_t*>(k.cw), static_cast<uint8_t*>(k.tree), h.data()));
            auto it = kept_.find(c.data());
            if (it != kept_.end()) { zkh_dev_free(ctx_, it->second.cw); zkh_dev_free(ctx_, it->second.tree); }
            kept_[c.data()] = k;
            return h;
        }
        ck(zkh_basefold_commit(ctx_, c.data(), v, R, nullptr, h.data()));
        return h;
    }
    void release_kept() {
        for (auto& kv : kept_) { zkh_dev_free(ctx_, kv.second.cw); zkh_dev_free(ctx_, kv.second.tree); }
        kept_.clear();
    }
    // serialised p3bf::EvalProof (fields in declaration order, see zkh.h)
    std::vector<uint8_t> prove_eval_dev(const DevCol& c, const std::vector<gl_t>& z, gl_t y, uint32_t R, uint32_t Q,
                                        const std::string& seed = "p3-bf") {
        std::vector<uint8_t> out(zkh_basefold_proof_size((uint32_t)z.size(), R, Q));
        size_t wr = 0;
        ck(zkh_basefold_open(ctx_, c.data(), z.data(), (uint32_t)z.size(), y, R, Q, nullptr, seed.c_str(), out.data(), out.size(), &wr));
        out.resize(wr);
        return out;
    }
    // p3gkr::prove_dev: serialised p3gkr::Proof; rfin and (p~, q~)(rfin) come back through the out-parameters
    std::vector<uint8_t> gkr_prove(Transcript& tr, const char* tag, const DevCol& p, const DevCol& q, bool combine_last,
                                   std::vector<gl_t>& rfin, gl_t cpq[2]) {
        uint32_t L = 0;
        while (((size_t)1 << L) < p.size()) L++;
        std::vector<uint8_t> out(zkh_gkr_proof_size(L));
        rfin.assign(combine_last ? L : L - 1, 0);
        size_t wr = 0;
        ck(zkh_gkr_prove(ctx_, p.data(), q.data(), L, combine_last ? 1 : 0, tag, tr.state, rfin.data(), cpq, out.data(), out.size(), &wr));
        out.resize(wr);
        return out;
    }
    // one ledger entry of p3bo::PLedger: column, its root, index of its point
    struct Entry { const DevCol* col; Hash root; uint32_t zid; };
    // p3bo::prove_class: pts = T points of v coordinates; serialised p3bo::BatchProof
    std::vector<uint8_t> prove_class(Transcript& tr, const std::vector<std::vector<gl_t>>& pts, const std::vector<Entry>& ents,
                                     uint32_t R, uint32_t Q, const std::string& label) {
        const uint32_t T = (uint32_t)pts.size(), v = (uint32_t)pts[0].size(), k = (uint32_t)ents.size();
        std::vector<gl_t> flat;
        for (auto& p : pts) flat.insert(flat.end(), p.begin(), p.end());
        std::vector<const gl_t*> cols(k);
        std::vector<uint8_t> roots((size_t)k * 32);
        std::vector<uint32_t> zid(k);
        for (uint32_t j = 0; j < k; j++) {
            cols[j] = ents[j].col->data();
            memcpy(&roots[(size_t)j * 32], ents[j].root.data(), 32);
            zid[j] = ents[j].zid;
        }
        std::vector<uint8_t> out(zkh_batchopen_proof_bound(v, R, Q, k));
        size_t wr = 0;
        std::vector<const uint64_t*> kcw(k, nullptr);
        std::vector<const uint8_t*> ktr(k, nullptr);
        bool any = false;
        for (uint32_t j = 0; j < k; j++) {
            auto it = kept_.find(cols[j]);
            if (it != kept_.end() && it->second.R == R && it->second.n == ents[j].col->size()) {
                kcw[j] = static_cast<const uint64_t*>(it->second.cw);
                ktr[j] = static_cast<const uint8_t*>(it->second.tree);
                any = true;
            }
        }
        if (any)
            ck(zkh_batchopen_prove_class_kept(ctx_, v, flat.data(), T, cols.data(), roots.data(), zid.data(), k, R, Q, label.c_str(), tr.state,
                                              out.data(), out.size(), &wr, kcw.data(), ktr.data()));
        else
            ck(zkh_batchopen_prove_class(ctx_, v, flat.data(), T, cols.data(), roots.data(), zid.data(), k, R, Q, label.c_str(), tr.state,
                                         out.data(), out.size(), &wr));
        out.resize(wr);
        return out;
    }

    // ---- hiding mode (the reference's zk switch): engine calls under p3zkc / sc5z / the zk branches of prove_class ----
    // p3zkc::salted_commit_root_dev (zkllm-src/p3_zkc.cuh:357-397)
    Hash commit_salted(const DevCol& c, uint32_t R, uint64_t sseed) {
        uint32_t v = 0;
        while (((size_t)1 << v) < c.size()) v++;
        Hash h;
        ck(zkh_basefold_commit_salted(ctx_, c.data(), v, R, sseed, nullptr, nullptr, h.data()));
        return h;
    }
    // p3zkc::zprng_fill chain / zprng_at stream on the device (zkllm-src/p3_zkc.cuh:100-117, :464-534)
    DevCol zk_fill_chain(uint64_t s0, size_t n, uint64_t k0 = 0) {
        DevCol out(*this, n);
        ck(zkh_zk_fill_chain(ctx_, s0, k0, n, out.data()));
        return out;
    }
    DevCol zk_fill_at(uint64_t seed, size_t n, uint64_t i0 = 0) {
        DevCol out(*this, n);
        ck(zkh_zk_fill_at(ctx_, seed, i0, n, out.data()));
        return out;
    }
    // [real | mask slices from the chain of mask_seed]: p3zkc::augment over a fresh mask (zkllm-src/p3_zkc.cuh:158-177)
    DevCol zk_augment(const DevCol& c, uint32_t e, uint64_t mask_seed) {
        uint32_t v = 0;
        while (((size_t)1 << v) < c.size()) v++;
        DevCol out(*this, (size_t)1 << (v + e));
        ck(zkh_zk_augment(ctx_, c.data(), v, e, mask_seed, out.data()));
        return out;
    }
    // the blinded chain of p3hwl::sc5z, structured layout (zkllm-src/p3_hawkeye.cuh:1092-1110, :1329-1331): terms may carry a
    // third field "outside the col0 factor"; fix = 7 words per round (g_rd coefficients, A_rd, B_rd); returns r, g(r) in pref
    struct ZTerm { gl_t coef; std::vector<uint8_t> idx; bool outside = false; };
    std::vector<gl_t> sc_prove_zc_blind(Transcript& tr, const char* tag, const std::vector<const gl_t*>& d_cols, uint32_t N,
                                        const std::vector<ZTerm>& terms, gl_t konst, const std::vector<gl_t>& fix,
                                        std::vector<gl_t>& msgs, std::vector<gl_t>& finals, gl_t& pref) {
        uint32_t logn = 0;
        while ((1u << logn) < N) logn++;
        std::vector<uint64_t> prog = {terms.size(), konst};
        for (auto& t : terms) {
            uint64_t pk = t.idx.size() | (t.outside ? 0x80u : 0u);
            for (size_t k = 0; k < t.idx.size(); k++) pk |= (uint64_t)t.idx[k] << (8 + 8 * k);
            prog.push_back(t.coef);
            prog.push_back(pk);
        }
        std::vector<gl_t> r(logn), m((size_t)logn * 5);
        finals.assign(d_cols.size(), 0);
        if (fix.empty())
            ck(zkh_sumcheck_zerocheck(ctx_, d_cols.data(), (int)d_cols.size(), logn, prog.data(), (int)prog.size(), tag, tr.state,
                                      m.data(), r.data(), finals.data()));
        else
            ck(zkh_sumcheck_zerocheck_blind(ctx_, d_cols.data(), (int)d_cols.size(), logn, prog.data(), (int)prog.size(), fix.data(),
                                            tag, tr.state, m.data(), r.data(), finals.data(), &pref));
        msgs.insert(msgs.end(), m.begin(), m.end());
        return r;
    }
    // the first `rounds` rounds of such a chain (factored matmul chain): left = what every column still holds, column after column
    std::vector<gl_t> sc_prove_zc_partial(Transcript& tr, const char* tag, const std::vector<const gl_t*>& d_cols, uint32_t N,
                                          const std::vector<ZTerm>& terms, gl_t konst, uint32_t rounds, const std::vector<gl_t>& fix,
                                          std::vector<gl_t>& msgs, std::vector<gl_t>& left, gl_t& pref) {
        uint32_t logn = 0;
        while ((1u << logn) < N) logn++;
        std::vector<uint64_t> prog = {terms.size(), konst};
        for (auto& t : terms) {
            uint64_t pk = t.idx.size() | (t.outside ? 0x80u : 0u);
            for (size_t k = 0; k < t.idx.size(); k++) pk |= (uint64_t)t.idx[k] << (8 + 8 * k);
            prog.push_back(t.coef);
            prog.push_back(pk);
        }
        std::vector<gl_t> r(rounds), m((size_t)rounds * 5);
        left.assign(d_cols.size() * ((size_t)N >> rounds), 0);
        gl_t pout = pref;
        ck(zkh_sumcheck_zerocheck_partial(ctx_, d_cols.data(), (int)d_cols.size(), logn, rounds, prog.data(), (int)prog.size(),
                                          fix.empty() ? nullptr : fix.data(), pref, tag, tr.state, m.data(), r.data(), left.data(), &pout));
        if (!fix.empty()) pref = pout;
        msgs.insert(msgs.end(), m.begin(), m.end());
        return r;
    }
    // p3bo::prove_class after the class blinder was appended, salted round-0 openings (zkllm-src/p3_batchopen.cuh:969-1131)
    std::vector<uint8_t> prove_class_salted(Transcript& tr, const std::vector<std::vector<gl_t>>& pts, const std::vector<Entry>& ents,
                                            const std::vector<uint64_t>& sseeds, uint32_t R, uint32_t Q, const std::string& label) {
        const uint32_t T = (uint32_t)pts.size(), v = (uint32_t)pts[0].size(), k = (uint32_t)ents.size();
        if (sseeds.size() != k) throw std::runtime_error("zkh: one salt seed per ledger entry");
        std::vector<gl_t> flat;
        for (auto& p : pts) flat.insert(flat.end(), p.begin(), p.end());
        std::vector<const gl_t*> cols(k);
        std::vector<uint8_t> roots((size_t)k * 32);
        std::vector<uint32_t> zid(k);
        for (uint32_t j = 0; j < k; j++) {
            cols[j] = ents[j].col->data();
            memcpy(&roots[(size_t)j * 32], ents[j].root.data(), 32);
            zid[j] = ents[j].zid;
        }
        std::vector<uint8_t> out(zkh_batchopen_proof_bound(v, R, Q, k) + (size_t)k * 2 * Q * 32);
        size_t wr = 0;
        ck(zkh_batchopen_prove_class_salted(ctx_, v, flat.data(), T, cols.data(), roots.data(), zid.data(), sseeds.data(), k, R, Q,
                                            label.c_str(), tr.state, out.data(), out.size(), &wr, nullptr, nullptr));
        out.resize(wr);
        return out;
    }

  private:
    struct Kept { uint32_t R; size_t n; void* cw; void* tree; };
    zkh_ctx* ctx_ = nullptr;
    std::map<const gl_t*, Kept> kept_;
};

inline DevCol::DevCol(Prover& p, size_t n) : ctx_(p.ctx()), n_(n) {
    void* d = nullptr;
    p.ck(zkh_dev_alloc(ctx_, n * sizeof(gl_t), &d));
    ptr_ = static_cast<gl_t*>(d);
}
inline DevCol::DevCol(Prover& p, const std::vector<gl_t>& host) : DevCol(p, host.size()) {
    p.ck(zkh_upload(ctx_, ptr_, host.data(), host.size() * sizeof(gl_t)));
}
inline std::vector<gl_t> DevCol::to_host() const {
    std::vector<gl_t> h(n_);
    if (zkh_download(ctx_, h.data(), ptr_, n_ * sizeof(gl_t)) != ZKH_OK) throw std::runtime_error("zkh: download failed");
    return h;
}


// ======================================================================================================================
// Gadget-level host logic in C++ (the reference's host side is C++ too): opening ledger, merged lookups, the integer
// matmul and rescale gadgets.  Same transcripts and proof bytes as the reference's non-zk provers:
//   p3bo::PLedger (zkllm-src/p3_batchopen.cuh:144-178)          -> Ledger
//   p3hwl::claimc (zkllm-src/p3_hawkeye.cuh:800-838)            -> claimc
//   p3lu::make_table / defer_v / prove_super / lu_flush (zkllm-src/p3_logup.cuh:413-421, :518-543, :1357-1881, :1940-1956)
//   p3ig::tail_prove (zkllm-src/p3_int_gadgets.cuh:186-197)     -> tail_prove
//   p3imm::prove (zkllm-src/p3_int_gadgets.cuh:546-605)         -> imm_prove   (direct layouts)
//   p3irs::prove (zkllm-src/p3_int_gadgets.cuh:291-340)         -> irs_prove
// ======================================================================================================================

inline gl_t gl_mulmod(gl_t a, gl_t b) { return (gl_t)(((unsigned __int128)a * b) % GL_P); }
inline gl_t gl_addmod(gl_t a, gl_t b) { return (gl_t)(((unsigned __int128)a + b) % GL_P); }

// device array of uint32 row indices
class DevIdx {
  public:
    DevIdx() = default;
    DevIdx(Prover& p, const std::vector<uint32_t>& host) : ctx_(p.ctx()), n_(host.size()) {
        void* d = nullptr;
        p.ck(zkh_dev_alloc(ctx_, n_ * 4, &d));
        ptr_ = static_cast<uint32_t*>(d);
        p.ck(zkh_upload(ctx_, ptr_, host.data(), n_ * 4));
    }
    DevIdx(Prover& p, size_t n) : ctx_(p.ctx()), n_(n) {
        void* d = nullptr;
        p.ck(zkh_dev_alloc(ctx_, n * 4, &d));
        ptr_ = static_cast<uint32_t*>(d);
    }
    DevIdx(DevIdx&& o) noexcept : ctx_(o.ctx_), ptr_(o.ptr_), n_(o.n_) { o.ptr_ = nullptr; }
    DevIdx& operator=(DevIdx&& o) noexcept {
        if (this != &o) { if (ptr_) zkh_dev_free(ctx_, ptr_); ctx_ = o.ctx_; ptr_ = o.ptr_; n_ = o.n_; o.ptr_ = nullptr; }
        return *this;
    }
    DevIdx(const DevIdx&) = delete;
    DevIdx& operator=(const DevIdx&) = delete;
    ~DevIdx() { if (ptr_) zkh_dev_free(ctx_, ptr_); }
    uint32_t* data() const { return ptr_; }
    size_t size() const { return n_; }

  private:
    zkh_ctx* ctx_ = nullptr;
    uint32_t* ptr_ = nullptr;
    size_t n_ = 0;
};

// a committed column: the device buffer and its commitment root
struct CCol { const DevCol* col; Hash root; };

struct Ledger {
    struct Cls { uint32_t v; std::vector<std::vector<gl_t>> pts; std::vector<Prover::Entry> ents; std::vector<gl_t> ys; };
    std::vector<Cls> cls;
    void add(const DevCol* col, const Hash& root, const std::vector<gl_t>& z, gl_t y) {
        for (auto& c : cls)
            if (c.v == z.size()) {
                uint32_t zid = 0;
                for (; zid < c.pts.size(); zid++) if (c.pts[zid] == z) break;
                if (zid == c.pts.size()) c.pts.push_back(z);
                c.ents.push_back({col, root, zid});
                c.ys.push_back(y);
                return;
            }
        cls.push_back({(uint32_t)z.size(), {z}, {{col, root, 0}}, {y}});
    }
};

inline gl_t claimc(Prover& P, Transcript& tr, Ledger& lg, const CCol& c, const std::vector<gl_t>& z) {
    gl_t y = P.eval_h_gpu(*c.col, z);
    tr.absorb("hwl-y", &y, 8);
    lg.add(c.col, c.root, z, y);
    return y;
}

inline void put_u32(std::vector<uint8_t>& b, uint32_t v) { const uint8_t* q = (const uint8_t*)&v; b.insert(b.end(), q, q + 4); }
inline void put_raw(std::vector<uint8_t>& b, const void* s, size_t n) { const uint8_t* q = (const uint8_t*)s; b.insert(b.end(), q, q + n); }
inline void put_blob(std::vector<uint8_t>& b, const std::vector<uint8_t>& x) { put_u32(b, (uint32_t)x.size()); put_raw(b, x.data(), x.size()); }

struct Table {
    std::vector<std::vector<gl_t>> cols;
    Hash id;
    std::vector<DevCol> dev;            // uploaded on first use
    const std::vector<DevCol>& on(Prover& P) {
        if (dev.empty()) for (auto& c : cols) dev.emplace_back(P, c);
        return dev;
    }
};
inline Table make_table(std::vector<std::vector<gl_t>> cols) {
    Table t;
    std::vector<uint8_t> b;
    uint64_t nc = cols.size(), nr = cols[0].size();
    put_raw(b, &nc, 8); put_raw(b, &nr, 8);
    for (auto& c : cols) put_raw(b, c.data(), c.size() * 8);
    zkh_tr_init(t.id.data(), b.data(), b.size());          // SHA-256 of the table bytes
    t.cols = std::move(cols);
    return t;
}
inline Table range_table(uint32_t bits, int64_t off) {
    std::vector<gl_t> v((size_t)1 << bits);
    for (size_t j = 0; j < v.size(); j++) { int64_t x = (int64_t)j + off; v[j] = x >= 0 ? (gl_t)x : GL_P - (gl_t)(-x); }
    return make_table({v});
}

// one deferred lookup: c witness columns (committed[t] false: virtual), the row indices, the table
struct Lookup { std::vector<CCol> W; std::vector<bool> committed; const DevIdx* idx; Table* tab; };

// shared proving context of composed gadgets (p3lu::XCtx): the opening ledger, the deferred lookups, and the columns and
// index arrays that must stay alive until the batched openings
struct XCtx {
    Ledger lg;
    std::vector<Lookup> luq;
    std::deque<DevCol> keep;
    std::deque<DevIdx> keepi;
};

inline std::vector<uint8_t> prove_super(Prover& P, Transcript& tr, Table& T, const std::vector<std::pair<uint32_t, std::vector<const Lookup*>>>& subs,
                                        uint32_t R, bool strict, XCtx& xc) {
    zkh_ctx* ctx = P.ctx();
    Ledger& lg = xc.lg;
    const auto& tcols = T.on(P);
    const uint32_t c = (uint32_t)tcols.size();
    const size_t M = tcols[0].size();
    uint32_t m = 0;
    while (((size_t)1 << m) < M) m++;
    tr.absorb("lug-tab", T.id.data(), 32);
    uint32_t sd[3] = {(uint32_t)subs.size(), m, c};
    tr.absorb("lug-sdims", sd, 12);
    DevCol cnt(P, M);
    size_t pad_rows = 0;
    bool first = true;
    DevCol tmp(P, M);
    for (auto& sg : subs) {
        const uint32_t n = sg.first, k = (uint32_t)sg.second.size();
        uint32_t g = 0;
        while ((1u << g) < k) g++;
        uint32_t dm[4] = {n, g, k, c};
        tr.absorb("lug-dims", dm, 16);
        for (auto* L : sg.second) {
            if (L->W.size() != c || L->idx->size() != ((size_t)1 << n)) throw std::runtime_error("p3lu: group member size");
            for (size_t t = 0; t < c; t++) {
                if (L->committed[t]) tr.absorb("lug-W", L->W[t].root.data(), 32);
                else tr.absorb("lug-Wv", "virt", 4);
            }
            P.ck(zkh_histogram(ctx, L->idx->data(), L->idx->size(), (uint32_t)M, first ? cnt.data() : tmp.data()));
            if (!first) {
                const gl_t* two[2] = {cnt.data(), tmp.data()};
                P.ck(zkh_gl_affine(ctx, two, 2, M, 1, 0, cnt.data()));       // cnt += tmp (gamma = 1)
            }
            first = false;
        }
        pad_rows += (((size_t)1 << g) - k) << n;
    }
    if (pad_rows) {
        gl_t c0 = 0;
        P.ck(zkh_download(ctx, &c0, cnt.data(), 8));
        c0 += pad_rows;
        P.ck(zkh_upload(ctx, cnt.data(), &c0, 8));
    }
    Hash root_cnt = P.commit_gpu_rootonly(cnt, R);
    tr.absorb("lug-cnt", root_cnt.data(), 32);
    const gl_t gamma = tr.chal(), beta = tr.chal();
    gl_t a0 = 0, gp = 1;
    for (uint32_t t = 0; t < c; t++) {
        gl_t r0 = 0;
        P.ck(zkh_download(ctx, &r0, tcols[t].data(), 8));
        a0 = gl_addmod(a0, gl_mulmod(gp, r0));
        gp = gl_mulmod(gp, gamma);
    }
    gl_t accP = 0, accQ = 1;
    std::vector<uint8_t> body;
    for (auto& sg : subs) {
        const uint32_t n = sg.first, k = (uint32_t)sg.second.size();
        uint32_t g = 0;
        while ((1u << g) < k) g++;
        const size_t N = (size_t)1 << n, kp = (size_t)1 << g;
        DevCol LQ(P, kp << n), LP(P, kp << n);
        for (size_t j = 0; j < kp; j++) {
            if (j < k) {
                std::vector<const gl_t*> ptrs;
                for (auto& w : sg.second[j]->W) ptrs.push_back(w.col->data());
                P.ck(zkh_gl_affine(ctx, ptrs.data(), (int)c, N, gamma, beta, LQ.data() + j * N));
            } else {
                P.ck(zkh_gl_affine(ctx, nullptr, 0, N, 0, gl_addmod(a0, beta), LQ.data() + j * N));
            }
        }
        P.ck(zkh_gl_affine(ctx, nullptr, 0, kp << n, 0, 1, LP.data()));
        std::vector<gl_t> rA;
        gl_t cpq[2];
        std::vector<uint8_t> gk = P.gkr_prove(tr, "lug-gA", LP, LQ, true, rA, cpq);
        gl_t Pv, Qv;
        memcpy(&Pv, gk.data(), 8); memcpy(&Qv, gk.data() + 8, 8);
        accP = gl_addmod(gl_mulmod(accP, Qv), gl_mulmod(Pv, accQ));
        accQ = gl_mulmod(accQ, Qv);
        std::vector<gl_t> pm(rA.begin(), rA.begin() + n);
        put_u32(body, n); put_u32(body, k); put_raw(body, gk.data(), gk.size());
        for (auto* L : sg.second) {
            std::vector<gl_t> yW, yv;
            for (size_t t = 0; t < c; t++) {
                gl_t y = P.eval_h_gpu(*L->W[t].col, pm);
                if (L->committed[t]) {
                    yW.push_back(y);
                    tr.absorb("lug-yW", &y, 8);
                    lg.add(L->W[t].col, L->W[t].root, pm, y);
                } else {
                    yv.push_back(y);
                    tr.absorb("lug-yv", &y, 8);
                }
            }
            put_u32(body, (uint32_t)yW.size()); put_raw(body, yW.data(), yW.size() * 8);
            put_u32(body, (uint32_t)yv.size()); put_raw(body, yv.data(), yv.size() * 8);
            put_u32(body, 0);
        }
    }
    DevCol LQT(P, M);
    {
        std::vector<const gl_t*> ptrs;
        for (auto& t : tcols) ptrs.push_back(t.data());
        P.ck(zkh_gl_affine(ctx, ptrs.data(), (int)c, M, gamma, beta, LQT.data()));
    }
    std::vector<gl_t> rT;
    gl_t cpq[2];
    std::vector<uint8_t> gkT = P.gkr_prove(tr, "lug-gT", cnt, LQT, true, rT, cpq);
    gl_t PT, QT;
    memcpy(&PT, gkT.data(), 8); memcpy(&QT, gkT.data() + 8, 8);
    if (strict && gl_mulmod(accP, QT) != gl_mulmod(PT, accQ)) throw std::runtime_error("p3lu: witness not in table");
    // the multiplicity column must outlive this call: the ledger refers to it until the batched opening
    xc.keep.push_back(std::move(cnt));
    lg.add(&xc.keep.back(), root_cnt, rT, cpq[0]);
    std::vector<uint8_t> out;
    put_u32(out, m); put_u32(out, c); put_u32(out, (uint32_t)subs.size());
    put_raw(out, root_cnt.data(), 32);
    put_raw(out, gkT.data(), gkT.size());
    put_raw(out, body.data(), body.size());
    return out;
}


constexpr uint32_t LU_GCAP = 25;     // zkllm-src/p3_logup.cuh:1891

// p3lu::lu_flush: group the deferred lookups by (table, log-rows) in first-appearance order, cap groups at 2^LU_GCAP stacked
// rows, bundle the groups by table, prove one merged instance per table.  Returns the GroupProofs.
inline std::vector<std::vector<uint8_t>> lu_flush(Prover& P, Transcript& tr, XCtx& xc, uint32_t R, bool strict = true) {
    struct Grp { Table* tab; uint32_t n; std::vector<const Lookup*> mem; };
    std::vector<Grp> groups;
    for (auto& L : xc.luq) {
        uint32_t n = 0;
        while (((size_t)1 << n) < L.idx->size()) n++;
        bool placed = false;
        for (auto& g : groups)
            if (g.tab->id == L.tab->id && g.n == n) { g.mem.push_back(&L); placed = true; break; }
        if (!placed) groups.push_back({L.tab, n, {&L}});
    }
    std::vector<Grp> split;
    for (auto& g : groups) {
        const size_t cap = g.n >= LU_GCAP ? 1 : (size_t)1 << (LU_GCAP - g.n);
        for (size_t off = 0; off < g.mem.size(); off += cap)
            split.push_back({g.tab, g.n, std::vector<const Lookup*>(g.mem.begin() + off, g.mem.begin() + std::min(off + cap, g.mem.size()))});
    }
    struct Sup { Table* tab; std::vector<std::pair<uint32_t, std::vector<const Lookup*>>> subs; };
    std::vector<Sup> supers;
    for (auto& g : split) {
        bool placed = false;
        for (auto& sp : supers)
            if (sp.tab->id == g.tab->id) { sp.subs.push_back({g.n, g.mem}); placed = true; break; }
        if (!placed) supers.push_back({g.tab, {{g.n, g.mem}}});
    }
    std::vector<std::vector<uint8_t>> out;
    for (auto& sp : supers) out.push_back(prove_super(P, tr, *sp.tab, sp.subs, R, strict, xc));
    xc.luq.clear();
    return out;
}

// p3ig::tail_prove without the lookup flush: one batched opening per size class, labelled tag + index
inline std::vector<std::vector<uint8_t>> tail_prove(Prover& P, Transcript& tr, Ledger& lg, uint32_t R, uint32_t Q, const std::string& tag) {
    std::vector<std::vector<uint8_t>> out;
    for (size_t i = 0; i < lg.cls.size(); i++)
        out.push_back(P.prove_class(tr, lg.cls[i].pts, lg.cls[i].ents, R, Q, tag + std::to_string(i)));
    return out;
}
inline void put_tail(std::vector<uint8_t>& b, const std::vector<std::vector<uint8_t>>& lug, const std::vector<std::vector<uint8_t>>& batches) {
    put_u32(b, (uint32_t)lug.size());
    for (auto& x : lug) put_blob(b, x);
    put_u32(b, (uint32_t)batches.size());
    for (auto& x : batches) put_blob(b, x);
}

// p3imm::prove, direct layouts: Y(i,k) = sum_j X(i,j) W(j,k) for committed X = [j | i<<lj], W = [k | j<<lk], Y = [k | i<<lk].
// The summand eq(z;k,i) X(j,i) W(j,k) factors over the index groups, so the reference's 2^(lj+lk+li)-row cubic sumcheck is
// three short product sumchecks after partial evaluations (matrix-vector products); same messages, same proof bytes.
// Serialised p3imm::Proof: u32 lj lk li | messages (lj+lk+li)*40 | yY yX yW | u32 batches, each u32 length + BatchProof.
inline std::vector<uint8_t> imm_prove(Prover& P, Transcript& tr, const CCol& X, const CCol& W, const CCol& Y, uint32_t lj, uint32_t lk,
                                      uint32_t li, uint32_t R, uint32_t Q, XCtx* shared = nullptr) {
    zkh_ctx* ctx = P.ctx();
    XCtx own;
    XCtx& xc = shared ? *shared : own;
    uint32_t d3[3] = {lj, lk, li};
    tr.absorb("imm-dims", d3, 12);
    tr.absorb("imm-X", X.root.data(), 32);
    tr.absorb("imm-W", W.root.data(), 32);
    tr.absorb("imm-Y", Y.root.data(), 32);
    std::vector<gl_t> z(lk + li);
    for (auto& v : z) v = tr.chal();
    std::vector<gl_t> zk_(z.begin(), z.begin() + lk), zi_(z.begin() + lk, z.end());
    const gl_t yY = claimc(P, tr, xc.lg, Y, z);
    const uint64_t J = 1ull << lj, K = 1ull << lk, I = 1ull << li;
    DevCol eq_i = P.build_eq_gpu(zi_), eq_k = P.build_eq_gpu(zk_);
    auto matvec = [&](const DevCol& Mx, uint64_t rows, uint64_t cols, const DevCol& w, bool along_rows) {
        DevCol out(P, along_rows ? rows : cols);
        P.ck(zkh_gl_matvec(ctx, Mx.data(), rows, cols, w.data(), along_rows ? 1 : 0, out.data()));
        return out;
    };
    auto scaled = [&](const DevCol& in, gl_t sc) {
        DevCol out(P, in.size());
        P.ck(zkh_gl_scale(ctx, in.data(), in.size(), sc, out.data()));
        return out;
    };
    std::vector<gl_t> msgs, rj, rk, ri, fin;
    DevCol Xz = matvec(*X.col, I, J, eq_i, false), Wz = matvec(*W.col, J, K, eq_k, true);
    if (lj) rj = P.sc_prove_gpu(tr, "imm-sc", {Xz.data(), Wz.data()}, (uint32_t)J, ZKH_F_PROD2, 5, nullptr, 0, msgs);
    DevCol eq_rj = P.build_eq_gpu(rj);
    DevCol X1 = matvec(*X.col, I, J, eq_rj, true), W1 = matvec(*W.col, J, K, eq_rj, false);
    const gl_t SX = P.eval_h_gpu(X1, zi_);
    gl_t Wrr;
    if (lk) {
        DevCol sk = scaled(eq_k, SX);
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
        DevCol si = scaled(eq_i, gl_mulmod(eqk_r, Wrr));
        ri = P.sc_prove_gpu(tr, "imm-sc", {si.data(), X1.data()}, (uint32_t)I, ZKH_F_PROD2, 5, nullptr, 0, msgs);
    }
    std::vector<gl_t> zx(rj), zw(rk);
    zx.insert(zx.end(), ri.begin(), ri.end());
    zw.insert(zw.end(), rj.begin(), rj.end());
    const gl_t yX = claimc(P, tr, xc.lg, X, zx), yW = claimc(P, tr, xc.lg, W, zw);
    std::vector<uint8_t> out;
    put_raw(out, d3, 12);
    put_raw(out, msgs.data(), msgs.size() * 8);
    put_raw(out, &yY, 8); put_raw(out, &yX, 8); put_raw(out, &yW, 8);
    std::vector<std::vector<uint8_t>> batches;
    if (!shared) batches = tail_prove(P, tr, xc.lg, R, Q, "imm-bo");
    put_u32(out, (uint32_t)batches.size());
    for (auto& b : batches) put_blob(out, b);
    return out;
}

// the rescale gadget's tables (p3ig::build_tables, zkllm-src/p3_int_gadgets.cuh:75-98): limb ranges and the signed windows
struct IrsTables {
    Table R16 = range_table(16, 0), R14 = range_table(14, 0), RTOP, RS16 = range_table(16, -(1 << 15)), RS20 = range_table(20, -(1 << 19));
    explicit IrsTables(uint32_t btop = 12) : RTOP(range_table(btop, 0)) {}
};

// p3irs::prove: Y = round-half-up(X / 2^sf), remainder limbs and Y range-checked by lookups.
// Serialised p3irs::Proof: u32 le sf nl rng | limb roots nl*32 | messages le*40 | yX yY yL[nl] | u32 groups (len, GroupProof)* |
// u32 batches (len, BatchProof)*.  acc must hold signed values lifted into the field.
inline std::vector<uint8_t> irs_prove(Prover& P, Transcript& tr, IrsTables& T, const CCol& X, DevCol& Yout, Hash& rootY, uint32_t le, uint32_t sf,
                                      int rng, uint32_t R, uint32_t Q, XCtx* shared = nullptr) {
    zkh_ctx* ctx = P.ctx();
    XCtx own;
    XCtx& xc = shared ? *shared : own;
    const size_t n = (size_t)1 << le;
    const uint32_t nl = sf <= 16 ? 1 : 2;
    // witness: y, limbs, lookup rows (the reference's gen_witness, here one kernel)
    xc.keep.emplace_back(P, n); DevCol& L0 = xc.keep.back();
    xc.keep.emplace_back(P, nl == 2 ? n : 1); DevCol& L1 = xc.keep.back();
    xc.keepi.emplace_back(P, n); DevIdx& i0 = xc.keepi.back();
    xc.keepi.emplace_back(P, nl == 2 ? n : 1); DevIdx& i1 = xc.keepi.back();
    xc.keepi.emplace_back(P, rng ? n : 1); DevIdx& iY = xc.keepi.back();
    Yout = DevCol(P, n);
    P.ck(zkh_irs_witness(ctx, X.col->data(), n, sf, rng, Yout.data(), L0.data(), nl == 2 ? L1.data() : nullptr, i0.data(),
                         nl == 2 ? i1.data() : nullptr, rng ? iY.data() : nullptr));
    rootY = P.commit_gpu_rootonly(Yout, R);
    const CCol Y{&Yout, rootY};
    uint32_t d4[4] = {le, sf, nl, (uint32_t)rng};
    tr.absorb("irs-dims", d4, 16);
    tr.absorb("irs-X", X.root.data(), 32);
    tr.absorb("irs-Y", Y.root.data(), 32);
    CCol Lc[2] = {{&L0, P.commit_gpu_rootonly(L0, R)}, {&L1, Hash{}}};
    if (nl == 2) Lc[1].root = P.commit_gpu_rootonly(L1, R);
    for (uint32_t l = 0; l < nl; l++) tr.absorb("irs-L", Lc[l].root.data(), 32);
    xc.luq.push_back({{Lc[0]}, {true}, &i0, sf == 14 ? &T.R14 : &T.R16});
    if (nl == 2) xc.luq.push_back({{Lc[1]}, {true}, &i1, sf == 32 ? &T.R16 : &T.RTOP});
    if (rng) xc.luq.push_back({{Y}, {true}, &iY, rng == 1 ? &T.RS20 : &T.RS16});
    std::vector<gl_t> zE(le);
    for (auto& v : zE) v = tr.chal();
    DevCol E = P.build_eq_gpu(zE);
    std::vector<const gl_t*> cols = {E.data(), X.col->data(), Yout.data(), L0.data()};
    if (nl == 2) cols.push_back(L1.data());
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
    std::vector<std::vector<uint8_t>> lug, batches;
    if (!shared) {
        lug = lu_flush(P, tr, xc, R);
        batches = tail_prove(P, tr, xc.lg, R, Q, "irs-bo");
    }
    put_tail(out, lug, batches);
    return out;
}

}  // namespace zkh_p3
