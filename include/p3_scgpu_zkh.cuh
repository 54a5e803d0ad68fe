// p3_scgpu_zkh.cuh -- reference-side binding: the reference's gadget code, unchanged, with its GPU sumcheck engine
// (p3sg::sc_prove_gpu, zkllm-src/p3_scgpu.cuh:91-160) replaced by libzkh's.
//
// Use: force-include this header ahead of the reference's own headers and link the library,
//     nvcc -include p3_scgpu_zkh.cuh -I<this repo>/include -I<reference>/zkllm-src ... -L<this repo>/zk-hillclimb_b200 -lzkh
// It first includes the reference's p3_scgpu.cuh (so that header's include guard is spent and its kernels remain
// available as the fallback), defines p3sg::sc_prove_gpu_zkh with the same template parameters, arguments and effects, and
// then redirects the NAME sc_prove_gpu to it for every call site that follows (p3_logup.cuh, p3_hawkeye.cuh,
// p3_int_gadgets.cuh, ...).  Summands the library has an id for run through zkh_sumcheck; the others, a structured-blind
// fix-up (ScFix) or a replayed challenge tape fall through to the reference's own implementation.
// Proof bytes and transcript are identical either way.
#pragma once
#include <atomic>
#include <stdexcept>          // the reference's header uses std::runtime_error and relies on its includer for this
#include <string>
#include <typeinfo>
#include "p3_scgpu.cuh"
#include "zkh.h"

namespace p3sg {

inline zkh_ctx* zkh_shim_ctx() {
    static zkh_ctx* c = [] {
        zkh_ctx* x = nullptr;
        int dev = 0;
        cudaGetDevice(&dev);
        if (zkh_ctx_create(dev, nullptr, &x) != ZKH_OK) x = nullptr;      // a stream of its own; the call below synchronises on both sides
        return x;
    }();
    return c;
}
// how many sumchecks went through the library (for tests)
inline std::atomic<uint64_t>& zkh_shim_calls() {
    static std::atomic<uint64_t> n{0};
    return n;
}
// the library's id of a reference device functor, by the functor's (mangled) type name; -1: none
inline int zkh_shim_functor(const char* name, int nt, size_t nc) {
    const std::string s(name);
    auto has = [&](const char* k) { return s.find(k) != std::string::npos; };
    if (has("FLuGpuZk") || has("Zk")) return -1;
    if (has("FImmGpu") && nc == 3 && nt >= 4) return ZKH_F_PROD3;
    if (has("FLuGpu") && nc == 4 && nt >= 4) return ZKH_F_LOGUP;
    if (has("FGkrGpu") && nc == 5 && nt >= 4) return ZKH_F_GKR;
    return -1;
}

template <typename FF, typename MsgT, int NT, int MAXC>
static inline std::vector<gl_t> sc_prove_gpu_zkh(fs::Transcript& tr, const char* tag, std::vector<gl_t*>& dcols, uint32_t N,
                                                 const gl_t* par, uint32_t npar, std::vector<MsgT>& msgs,
                                                 const ScFix* fx = nullptr, uint32_t rd0 = 0) {
    static_assert(sizeof(MsgT) == (size_t)NT * sizeof(gl_t), "msg layout");
    const int id = (fx || rd0 || fs::g_tape || N < 2 || (N & (N - 1)) || NT < 3 || NT > 5) ? -1
                                                                                          : zkh_shim_functor(typeid(FF).name(), NT, dcols.size());
    zkh_ctx* ctx = id < 0 ? nullptr : zkh_shim_ctx();
    if (!ctx) return sc_prove_gpu<FF, MsgT, NT, MAXC>(tr, tag, dcols, N, par, npar, msgs, fx, rd0);   // the reference's own
    uint32_t v = 0;
    while ((1u << v) < N) v++;
    const size_t nc = dcols.size();
    std::vector<gl_t> r(v), fin(nc);
    std::vector<MsgT> m(v);
    cudaDeviceSynchronize();                       // the caller's kernels on other streams have filled the columns
    const int rc = zkh_sumcheck(ctx, id, NT, (const uint64_t* const*)dcols.data(), (int)nc, v, par, (int)npar, tag, tr.state,
                                (uint64_t*)m.data(), r.data(), fin.data());
    if (rc != ZKH_OK) throw std::runtime_error(std::string("p3: sc_prove_gpu (libzkh): ") + zkh_last_error(ctx));
    msgs.insert(msgs.end(), m.begin(), m.end());
    // the reference consumes its input columns and leaves the fully bound one-element columns in their place
    for (size_t k = 0; k < nc; k++) {
        gl_t* one = nullptr;
        if (cudaMallocAsync(&one, 8, 0) != cudaSuccess) throw std::runtime_error("p3: sc_prove_gpu bind alloc failed (8 bytes)");
        cudaMemcpy(one, &fin[k], 8, cudaMemcpyHostToDevice);
        cudaFreeAsync(dcols[k], 0);
        dcols[k] = one;
    }
    zkh_shim_calls()++;
    return r;
}

}  // namespace p3sg

#define sc_prove_gpu sc_prove_gpu_zkh
