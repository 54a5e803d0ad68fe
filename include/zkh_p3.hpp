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
#include <array>
#include <cstdint>
#include <cstring>
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
    ~Prover() { if (ctx_) zkh_ctx_destroy(ctx_); }
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
    Hash commit_gpu_rootonly(const DevCol& c, uint32_t R) {
        uint32_t v = 0;
        while (((size_t)1 << v) < c.size()) v++;
        Hash h;
        ck(zkh_basefold_commit(ctx_, c.data(), v, R, nullptr, h.data()));
        return h;
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
        ck(zkh_batchopen_prove_class(ctx_, v, flat.data(), T, cols.data(), roots.data(), zid.data(), k, R, Q, label.c_str(), tr.state,
                                     out.data(), out.size(), &wr));
        out.resize(wr);
        return out;
    }

  private:
    zkh_ctx* ctx_ = nullptr;
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

}  // namespace zkh_p3
