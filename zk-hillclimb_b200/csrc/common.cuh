// Shared host-side plumbing of the library: the context object, the device
// workspace, error reporting, and small device helpers used by several kernels.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <atomic>
#include <mutex>
#include <string>
#include "gl.cuh"
#include "sha256.cuh"
#include "../../include/zkh.h"

#define ZKH_SM_COUNT_FALLBACK 148

// Device-resident control block of one proving job.  Kernels of consecutive
// rounds communicate through it (transcript state, round challenges), so a whole
// sumcheck / opening runs without the host reading anything back in between.
struct ZkhCtl {
    uint32_t st[8];          // Fiat-Shamir state (digest words)
    unsigned int counter;    // CTA completion counter of the running reduction
    unsigned int err;        // sticky device-side error flag
    gl_t par[8];             // summand parameters (lambda, beta, ...)
    gl_t local[8];           // this GPU's round sums when the reduction is finished elsewhere
    gl_t finals[16];         // column values after the last bind
    gl_t chals[80];          // round challenges
    gl_t msgs[80 * 5];       // round messages
    gl_t aux[64];            // scratch for composite protocols
    void* xchg;              // ZkhXchg* of this GPU when the peer-to-peer round exchange is connected
};

// Peer-to-peer exchange of the per-round sums of a sharded sumcheck (one process per GPU, mailboxes
// mapped into every peer through CUDA IPC).  Each GPU owns one mailbox; rank g writes its values and
// then its flag into slot [seq & 1][g] of EVERY mailbox with plain peer stores over NVLink and waits,
// with a bounded number of polls, until its own mailbox holds the flags of all ranks for this seq.
#define ZKH_XCHG_MAXG 16
struct ZkhMailbox {
    unsigned long long flag[2][ZKH_XCHG_MAXG];
    gl_t data[2][ZKH_XCHG_MAXG][8];
};
struct ZkhXchg {
    ZkhMailbox* mbox[ZKH_XCHG_MAXG];  // mbox[rank] is this GPU's own
    uint32_t rank, G;
    unsigned long long seq;           // exchanges completed so far (same on every rank)
};

struct ZkhTag { char s[ZKH_TR_MAX_LABEL]; uint32_t len; };

struct zkh_ctx {
    int device = 0;
    int sm_count = ZKH_SM_COUNT_FALLBACK;
    cudaStream_t stream = nullptr;
    bool own_stream = false;
    // workspace: one growable device allocation carved up by the running call
    void* ws = nullptr;
    size_t ws_bytes = 0;
    ZkhCtl* d_ctl = nullptr;     // device control block
    ZkhCtl* h_ctl = nullptr;     // pinned host mirror (downloaded once per call)
    gl_t* d_partials = nullptr;  // per-CTA round partial sums
    size_t partials_cap = 0;
    // cached twiddle tables, one set per log-size
    struct Tw { gl_t* lo = nullptr; gl_t* hi = nullptr; gl_t* lo_inv = nullptr; gl_t* hi_inv = nullptr; uint32_t lb = 0; };
    Tw tw[33];
    // CUDA events around the largest launch of the dominant kernel of the last call
    cudaEvent_t prof_ev[2] = {nullptr, nullptr};
    bool prof_valid = false;
    uint64_t prof_bytes = 0;     // algorithmic bytes of that launch
    const char* prof_kernel = "";
    // running sharded sumcheck (zkh_shard_*)
    struct Shard {
        bool active = false;
        int functor = 0, nt = 0, nc = 0;
        uint32_t logn = 0, next_round = 0;
        ZkhTag tag;
        const gl_t* cur_in[8];
        gl_t* bufA = nullptr;
        gl_t* bufB = nullptr;
        gl_t* dst = nullptr;
        gl_t* res = nullptr;  // transposed residual columns
    } shard;
    // peer-to-peer round exchange (zkh_p2p_*)
    struct P2P {
        ZkhMailbox* mine = nullptr;
        ZkhXchg* d_xchg = nullptr;
        void* opened[ZKH_XCHG_MAXG] = {};
        int rank = 0, G = 0;
    } p2p;
    std::string err;
};

static inline int zkh_fail(zkh_ctx* c, int code, const std::string& msg) {
    if (c) c->err = msg;
    return code;
}
#define ZKH_CUDA(c, expr)                                                                     \
    do {                                                                                      \
        cudaError_t e__ = (expr);                                                             \
        if (e__ != cudaSuccess)                                                               \
            return zkh_fail((c), ZKH_ERR_CUDA,                                                \
                            std::string(#expr) + ": " + cudaGetErrorString(e__));             \
    } while (0)
#define ZKH_TRY(expr)                  \
    do {                               \
        int r__ = (expr);              \
        if (r__ != ZKH_OK) return r__; \
    } while (0)

// Function attributes (the dynamic shared-memory limit) belong to a device, not to the process: one bit per device
// ordinal records where a kernel's one-time set-up has run.  The set-up runs exactly once per (guard, device), and a
// thread that arrives while another is still inside it waits: several library contexts of one process (one per host
// thread) may make their first launch of a kernel at the same moment, and a launch that overtook the attribute
// call was refused as "invalid argument".
struct ZkhOncePerDevice {
    std::mutex m;
    uint64_t done = 0;
};
template <class F>
static inline void zkh_once_on_device(ZkhOncePerDevice& g, int device, F&& setup) {
    std::lock_guard<std::mutex> lk(g.m);
    const uint64_t bit = 1ull << (device & 63);
    if (!(g.done & bit)) {
        setup();
        g.done |= bit;
    }
}

// make the workspace at least `bytes` large (contents are not preserved)
int zkh_ws_reserve(zkh_ctx* c, size_t bytes);
extern "C" int zkh_p2p_disconnect(zkh_ctx* c);
static inline ZkhTag zkh_make_tag(const char* s) {
    ZkhTag t;
    memset(&t, 0, sizeof t);
    size_t n = strlen(s);
    if (n > ZKH_TR_MAX_LABEL) n = ZKH_TR_MAX_LABEL;
    memcpy(t.s, s, n);
    t.len = (uint32_t)n;
    return t;
}
static inline size_t zkh_align(size_t x, size_t a = 256) { return (x + a - 1) / a * a; }
namespace zkh {
// eq(b,z) table for all b < 2^v into out_dev (queued on the context's stream; z is host memory)
size_t eq_scratch_bytes(uint32_t v);
int eq_enqueue(zkh_ctx* c, const uint64_t* z, uint32_t v, gl_t* out_dev, void* scratch, bool z_on_device = false);
}  // namespace zkh

#ifdef __CUDACC__
// ---- device helpers ----
__device__ __forceinline__ gl_t shfl_down_gl(gl_t v, int d) {
    uint32_t lo = __shfl_down_sync(0xffffffffu, (uint32_t)v, d);
    uint32_t hi = __shfl_down_sync(0xffffffffu, (uint32_t)(v >> 32), d);
    return ((uint64_t)hi << 32) | lo;
}
// Sum NT per-thread values over the CTA.  Result valid in thread 0.
// sh must hold NT*32 gl_t.  All threads must call.
template <int NT>
__device__ __forceinline__ void block_sum(gl_t (&v)[NT], gl_t* sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int t = 0; t < NT; t++) {
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) v[t] = gl_add(v[t], shfl_down_gl(v[t], d));
    }
    if (lane == 0) {
#pragma unroll
        for (int t = 0; t < NT; t++) sh[t * 32 + warp] = v[t];
    }
    __syncthreads();
    if (warp == 0) {
#pragma unroll
        for (int t = 0; t < NT; t++) {
            gl_t x = lane < nwarp ? sh[t * 32 + lane] : 0;
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) x = gl_add(x, shfl_down_gl(x, d));
            v[t] = x;
        }
    }
    __syncthreads();
}
__device__ __forceinline__ ulonglong2 ld2(const gl_t* p) {
    return __ldg(reinterpret_cast<const ulonglong2*>(p));
}
__device__ __forceinline__ void st2(gl_t* p, gl_t a, gl_t b) {
    *reinterpret_cast<ulonglong2*>(p) = make_ulonglong2(a, b);
}
#endif
