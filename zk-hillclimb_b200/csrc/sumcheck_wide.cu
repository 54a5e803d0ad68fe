// Quartic zero-check sumchecks over many columns (up to 64) for sm_100a: the round engine behind the
// fp8 gadget's constraint summands (hawkeye_fn.cuh).
//
// The reference runs these through sc_prove_gpu<FF, Msg5, 5, 40> when the domain is large
// (zkllm-src/p3_hawkeye.cuh:1016-1033: every column uploaded per call, two launches, a copy back and
// nc allocations per round) and through a host loop (sc5_prove, :641-700) otherwise, which is also the
// only path for the 57-column output constraint.  Here every size and every summand takes the same
// device path: one kernel per round that binds with the previous challenge, stores the halved columns,
// evaluates the summand at t = 0..4 on the pair it just produced, reduces across the grid through the
// last CTA to finish, and advances the Fiat-Shamir transcript on the device.
//
// A thread keeps one pair of every column (value and difference) in registers; at 57 columns the
// compiler spills part of that to local memory, which stays in L1.  These kernels are bound by the
// integer pipe (tens of field multiplications per row and evaluation point), not by HBM.
#include <algorithm>
#include <vector>
#include "sumcheck.cuh"
#include "hawkeye_fn.cuh"

namespace zkh {

constexpr int SCW_MAXC = 64;
constexpr int SCW_NT = 5;
constexpr int SCW_THREADS = 128;

struct WidePtrs {
    const gl_t* in[SCW_MAXC];
    gl_t* out[SCW_MAXC];
};

// first != 0: message over the caller's columns (items = pairs).
// first == 0: bind with *chal_prev, store, message over the bound columns (items = quads).
template <int F>
__global__ void __launch_bounds__(SCW_THREADS)
scw_round_kernel(WidePtrs P, size_t items, int first, ZkhCtl* ctl, gl_t* partials, const gl_t* chal_prev,
                 gl_t* msg_out, gl_t* chal_out, ZkhTag tag) {
    constexpr int NC = WFn<F>::NC, NLAM = WFn<F>::NLAM;
    __shared__ gl_t lam[NLAM];
    __shared__ gl_t sh[SCW_NT * 32];
    for (int j = threadIdx.x; j < NLAM; j += blockDim.x) lam[j] = ctl->aux[j];
    __syncthreads();
    const gl_t a = first ? 0 : *chal_prev;
    gl_t s[SCW_NT];
#pragma unroll
    for (int t = 0; t < SCW_NT; t++) s[t] = 0;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < items; i += stride) {
        gl_t cur[NC], dif[NC];
        if (first) {
#pragma unroll
            for (int k = 0; k < NC; k++) {
                ulonglong2 v = ld2(P.in[k] + 2 * i);
                cur[k] = v.x;
                dif[k] = gl_sub(v.y, v.x);
            }
        } else {
#pragma unroll
            for (int k = 0; k < NC; k++) {
                ulonglong2 u = ld2(P.in[k] + 4 * i), w = ld2(P.in[k] + 4 * i + 2);
                gl_t lo = gl_lerp(u.x, u.y, a), hi = gl_lerp(w.x, w.y, a);
                st2(P.out[k] + 2 * i, lo, hi);
                cur[k] = lo;
                dif[k] = gl_sub(hi, lo);
            }
        }
        s[0] = gl_add(s[0], WFn<F>::eval(cur, lam));
#pragma unroll
        for (int t = 1; t < SCW_NT; t++) {
#pragma unroll
            for (int k = 0; k < NC; k++) cur[k] = gl_add(cur[k], dif[k]);
            s[t] = gl_add(s[t], WFn<F>::eval(cur, lam));
        }
    }
    grid_finish<SCW_NT>(s, sh, ctl, partials, msg_out, chal_out, tag, 0);
}

// The two widest summands (30 and 57 columns, 18 and 49 constraints) with a row shared by the NP warps of a block: the
// block stages value and difference of every column for 32 rows in shared memory (warp w loads, binds and stores the
// columns k = w mod NP; lane = row, so every global access is one 512-byte segment), and warp w evaluates the
// constraints j = w (mod NP) of those 32 rows, reading only the columns they touch.  A thread of the one-row-per-thread
// kernel needs 172 (30 columns) or 255 registers with spills (57 columns), which leaves 8 warps per SM.
template <int F>
struct SmemRow {
    const gl_t (*c)[32];
    uint32_t lane;
    __device__ __forceinline__ gl_t operator[](int k) const { return c[k][lane]; }
};
template <int F, int NP>
__global__ void __launch_bounds__(32 * NP)
scw_split_kernel(WidePtrs P, size_t items, int first, ZkhCtl* ctl, gl_t* partials, const gl_t* chal_prev, gl_t* msg_out,
                 gl_t* chal_out, ZkhTag tag) {
    constexpr int NC = WFn<F>::NC, NLAM = WFn<F>::NLAM;
    static_assert(NP == 4, "the part dispatch below is written for four warps");
    __shared__ gl_t lam[NLAM];
    __shared__ gl_t sh[SCW_NT * 32];
    __shared__ gl_t cur[NC][32];
    __shared__ gl_t dif[NC][32];
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int j = threadIdx.x; j < NLAM; j += blockDim.x) lam[j] = ctl->aux[j];
    const gl_t a = first ? 0 : *chal_prev;
    gl_t s[SCW_NT];
#pragma unroll
    for (int t = 0; t < SCW_NT; t++) s[t] = 0;
    const SmemRow<F> row{cur, lane};
    for (size_t base = (size_t)blockIdx.x * 32; base < items; base += (size_t)gridDim.x * 32) {
        const size_t i = base + lane;
        const bool live = i < items;
        __syncthreads();                                 // the previous rows (and lam on the first pass) are done with
        for (int k = warp; k < NC; k += NP) {
            gl_t lo = 0, hi = 0;
            if (live) {
                if (first) {
                    ulonglong2 v = ld2(P.in[k] + 2 * i);
                    lo = v.x;
                    hi = v.y;
                } else {
                    ulonglong2 u = ld2(P.in[k] + 4 * i), w = ld2(P.in[k] + 4 * i + 2);
                    lo = gl_lerp(u.x, u.y, a);
                    hi = gl_lerp(w.x, w.y, a);
                    st2(P.out[k] + 2 * i, lo, hi);
                }
            }
            cur[k][lane] = lo;
            dif[k][lane] = gl_sub(hi, lo);
        }
        __syncthreads();
#pragma unroll 1
        for (int t = 0; t < SCW_NT; t++) {
            gl_t val;
            if (warp == 0) val = WFn<F>::template eval<0, NP>(row, lam);
            else if (warp == 1) val = WFn<F>::template eval<1, NP>(row, lam);
            else if (warp == 2) val = WFn<F>::template eval<2, NP>(row, lam);
            else val = WFn<F>::template eval<3, NP>(row, lam);
            if (live) s[t] = gl_add(s[t], val);
            if (t + 1 < SCW_NT) {
                __syncthreads();                         // every warp has read this point's values
                for (int k = warp; k < NC; k += NP) cur[k][lane] = gl_add(cur[k][lane], dif[k][lane]);
                __syncthreads();
            }
        }
    }
    __syncthreads();
    grid_finish<SCW_NT>(s, sh, ctl, partials, msg_out, chal_out, tag, 0);
}

// out[k] = in[k][0] + a*(in[k][1] - in[k][0]) after the last round
__global__ void scw_finals_kernel(WidePtrs P, int nc, const gl_t* chal, gl_t* out) {
    int k = threadIdx.x;
    if (k < nc) out[k] = gl_lerp(P.in[k][0], P.in[k][1], *chal);
}

// after a chain stopped early: out[k][p] = lerp(in[k][2p], in[k][2p+1], a) for the nleft pairs every column still holds
__global__ void zc_left_kernel(WidePtrs P, int nc, size_t nleft, const gl_t* chal, gl_t* out) {
    const gl_t a = *chal;
    for (size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x; t < (size_t)nc * nleft; t += (size_t)gridDim.x * blockDim.x) {
        const size_t k = t / nleft, p = t - k * nleft;
        out[t] = gl_lerp(P.in[k][2 * p], P.in[k][2 * p + 1], a);
    }
}

static size_t scw_workspace_bytes(int nc, uint32_t logn) {
    const size_t n = (size_t)1 << logn;
    return zkh_align((size_t)nc * (n / 2 + 1) * 8) + zkh_align((size_t)nc * (n / 4 + 1) * 8) + zkh_align((size_t)nc * 8);
}

template <int F>
static int scw_enqueue_t(zkh_ctx* ctx, const gl_t* const* in, uint32_t logn, const ZkhTag& tag, gl_t* finals_dev) {
    constexpr int NC = WFn<F>::NC;
    constexpr bool SPLIT = NC >= 30;                 // the 30- and 57-column summands: a row shared by four warps
    constexpr int SPLIT_NP = 4;
    cudaStream_t s = ctx->stream;
    ZkhCtl* ctl = ctx->d_ctl;
    const size_t n = (size_t)1 << logn;
    static const int occ = [] {
        int o = 0;
        if constexpr (SPLIT) cudaOccupancyMaxActiveBlocksPerMultiprocessor(&o, scw_split_kernel<F, SPLIT_NP>, 32 * SPLIT_NP, 0);
        else cudaOccupancyMaxActiveBlocksPerMultiprocessor(&o, scw_round_kernel<F>, SCW_THREADS, 0);
        return o < 1 ? 1 : o;
    }();
    const bool split = SPLIT && !getenv("ZKH_SCW_NOSPLIT");      // measurement knob: the one-row-per-thread kernel
    const size_t rows_per_block = split ? 32 : SCW_THREADS;
    auto grid_for = [&](size_t items) {
        size_t want = (items + rows_per_block - 1) / rows_per_block, cap = (size_t)ctx->sm_count * occ;
        if (cap > ctx->partials_cap / SCW_NT) cap = ctx->partials_cap / SCW_NT;
        return (unsigned)(want < cap ? want : cap);
    };
    auto launch = [&](const WidePtrs& P, size_t items, int first, const gl_t* chal_prev, gl_t* msg_out, gl_t* chal_out) {
        if constexpr (SPLIT) {
            if (split) {
                scw_split_kernel<F, SPLIT_NP><<<grid_for(items), 32 * SPLIT_NP, 0, s>>>(P, items, first, ctl, ctx->d_partials, chal_prev,
                                                                                        msg_out, chal_out, tag);
                return;
            }
        }
        scw_round_kernel<F><<<grid_for(items), SCW_THREADS, 0, s>>>(P, items, first, ctl, ctx->d_partials, chal_prev, msg_out, chal_out, tag);
    };
    WidePtrs P;
    memset(&P, 0, sizeof P);
    for (int k = 0; k < NC; k++) P.in[k] = in[k];
    launch(P, n / 2, 1, nullptr, ctl->msgs, ctl->chals);
    gl_t* bufA = (gl_t*)ctx->ws;
    gl_t* bufB = (gl_t*)((char*)ctx->ws + zkh_align((size_t)NC * (n / 2 + 1) * 8));
    gl_t* dst = bufA;
    size_t cur_n = n;
    for (uint32_t r = 1; r < logn; r++) {
        const size_t out_n = cur_n / 2;
        for (int k = 0; k < NC; k++) P.out[k] = dst + (size_t)k * out_n;
        launch(P, cur_n / 4, 0, ctl->chals + (r - 1), ctl->msgs + (size_t)r * SCW_NT, ctl->chals + r);
        for (int k = 0; k < NC; k++) P.in[k] = P.out[k];
        dst = (dst == bufA) ? bufB : bufA;
        cur_n = out_n;
    }
    scw_finals_kernel<<<1, SCW_MAXC, 0, s>>>(P, NC, ctl->chals + (logn - 1), finals_dev);
    return cudaGetLastError() == cudaSuccess ? ZKH_OK : zkh_fail(ctx, ZKH_ERR_CUDA, "wide sumcheck launch");
}


// ------------------------------------------------------------------ programmable zero-check
// Summand  col0 * (konst + sum_j coef_j * prod_{k < deg_j} col[idx_jk]) + sum_f coef_f * prod col[idx_fk],  degrees 1..3
// (the second sum: terms flagged "free", the Libra blind of the hiding mode, zkllm-src/p3_hawkeye.cuh:1035-1053): the shape of every
// eq-weighted constraint of the integer-layer gadgets (residual add, rescale, SwiGLU, RoPE, RMSNorm,
// softmax: zkllm-src/p3_int_gadgets.cuh:326, :726, :977-1035, :1307, :1563-1640, :1818).  The reference runs
// each of them through its host loop sc5_prove with a std::function per row; here the term list is data
// (ZkhZcProg, read from device memory into shared memory), so one kernel serves all gadgets.
// A thread stages the current value of every column in its own shared-memory column (no bank conflicts,
// no synchronisation) so that terms can index columns at run time.
constexpr int ZC_MAXTERMS = 120;
struct ZkhZcProg {
    uint32_t nterms, nc;
    gl_t konst;
    gl_t coef[ZC_MAXTERMS];
    uint32_t packed[ZC_MAXTERMS];   // deg | idx0 << 8 | idx1 << 16 | idx2 << 24
};

template <int NCMAX>
__global__ void __launch_bounds__(SCW_THREADS)
zc_round_kernel(WidePtrs P, size_t items, int first, const ZkhZcProg* prog_g, ZkhCtl* ctl, gl_t* partials,
                const gl_t* chal_prev, gl_t* msg_out, gl_t* chal_out, ZkhTag tag) {
    __shared__ ZkhZcProg prog;
    __shared__ gl_t vals[NCMAX][SCW_THREADS];
    __shared__ gl_t sh[SCW_NT * 32];
    for (uint32_t j = threadIdx.x; j < sizeof(ZkhZcProg) / 4; j += blockDim.x)
        reinterpret_cast<uint32_t*>(&prog)[j] = reinterpret_cast<const uint32_t*>(prog_g)[j];
    __syncthreads();
    const int nc = (int)prog.nc;
    const uint32_t nterms = prog.nterms;
    const gl_t konst = prog.konst;
    const gl_t a = first ? 0 : *chal_prev;
    const uint32_t tid = threadIdx.x;
    gl_t s[SCW_NT];
#pragma unroll
    for (int t = 0; t < SCW_NT; t++) s[t] = 0;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < items; i += stride) {
        gl_t cur[NCMAX], dif[NCMAX];
#pragma unroll
        for (int k = 0; k < NCMAX; k++) {
            if (k < nc) {
                if (first) {
                    ulonglong2 v = ld2(P.in[k] + 2 * i);
                    cur[k] = v.x;
                    dif[k] = gl_sub(v.y, v.x);
                } else {
                    ulonglong2 u = ld2(P.in[k] + 4 * i), w = ld2(P.in[k] + 4 * i + 2);
                    gl_t lo = gl_lerp(u.x, u.y, a), hi = gl_lerp(w.x, w.y, a);
                    st2(P.out[k] + 2 * i, lo, hi);
                    cur[k] = lo;
                    dif[k] = gl_sub(hi, lo);
                }
            }
        }
#pragma unroll 1
        for (int t = 0; t < SCW_NT; t++) {
#pragma unroll
            for (int k = 0; k < NCMAX; k++)
                if (k < nc) { vals[k][tid] = cur[k]; cur[k] = gl_add(cur[k], dif[k]); }
            Acc192 acc, accf;
            acc.clear();
            accf.clear();
            for (uint32_t j = 0; j < nterms; j++) {
                const uint32_t pk = prog.packed[j];
                gl_t x = vals[(pk >> 8) & 0xff][tid];
                if ((pk & 0x7f) >= 2) x = gl_mul(x, vals[(pk >> 16) & 0xff][tid]);
                if ((pk & 0x7f) >= 3) x = gl_mul(x, vals[(pk >> 24) & 0xff][tid]);
                if (pk & 0x80) accf.add_prod(prog.coef[j], x);
                else acc.add_prod(prog.coef[j], x);
            }
            s[t] = gl_add(s[t], gl_add(gl_mul(vals[0][tid], gl_add(acc.reduce(), konst)), accf.reduce()));
        }
    }
    grid_finish<SCW_NT>(s, sh, ctl, partials, msg_out, chal_out, tag, ctl->par[6] ? 3 : 0);
}

template <int NCMAX>
static int zc_enqueue_t(zkh_ctx* ctx, const gl_t* const* in, int nc, uint32_t logn, const ZkhZcProg* prog_dev,
                        const ZkhTag& tag, gl_t* finals_dev, uint32_t rounds) {
    cudaStream_t s = ctx->stream;
    ZkhCtl* ctl = ctx->d_ctl;
    const size_t n = (size_t)1 << logn;
    static const int occ = [] {
        int o = 0;
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&o, zc_round_kernel<NCMAX>, SCW_THREADS, 0);
        return o < 1 ? 1 : o;
    }();
    auto grid_for = [&](size_t items) {
        size_t want = (items + SCW_THREADS - 1) / SCW_THREADS, cap = (size_t)ctx->sm_count * occ;
        if (cap > ctx->partials_cap / SCW_NT) cap = ctx->partials_cap / SCW_NT;
        return (unsigned)(want < cap ? want : cap);
    };
    WidePtrs P;
    memset(&P, 0, sizeof P);
    for (int k = 0; k < nc; k++) P.in[k] = in[k];
    zc_round_kernel<NCMAX><<<grid_for(n / 2), SCW_THREADS, 0, s>>>(P, n / 2, 1, prog_dev, ctl, ctx->d_partials, nullptr,
                                                                  ctl->msgs, ctl->chals, tag);
    gl_t* bufA = (gl_t*)ctx->ws;
    gl_t* bufB = (gl_t*)((char*)ctx->ws + zkh_align((size_t)nc * (n / 2 + 1) * 8));
    gl_t* dst = bufA;
    size_t cur_n = n;
    for (uint32_t r = 1; r < rounds; r++) {
        const size_t out_n = cur_n / 2;
        for (int k = 0; k < nc; k++) P.out[k] = dst + (size_t)k * out_n;
        zc_round_kernel<NCMAX><<<grid_for(cur_n / 4), SCW_THREADS, 0, s>>>(
            P, cur_n / 4, 0, prog_dev, ctl, ctx->d_partials, ctl->chals + (r - 1), ctl->msgs + (size_t)r * SCW_NT,
            ctl->chals + r, tag);
        for (int k = 0; k < nc; k++) P.in[k] = P.out[k];
        dst = (dst == bufA) ? bufB : bufA;
        cur_n = out_n;
    }
    const size_t nleft = n >> rounds;       // 1 after a full chain; more when the caller continues on other columns
    zc_left_kernel<<<(unsigned)std::min<size_t>(((size_t)nc * nleft + 255) / 256, 1024), 256, 0, s>>>(P, nc, nleft, ctl->chals + (rounds - 1),
                                                                                                 finals_dev);
    return cudaGetLastError() == cudaSuccess ? ZKH_OK : zkh_fail(ctx, ZKH_ERR_CUDA, "zero-check sumcheck launch");
}

// Large programs (more than 32 columns or 120 terms: the bf16 gadgets of the fp8 transformer layer, whose constraint
// systems span 60..200 columns and several hundred monomials; the reference runs them through its host loop sc5_prove,
// zkllm-src/p3_bfadd.cuh:214-330 and siblings).  Same summand shape.  The kernel is bound by the field multiplications of
// the monomials, not by memory, so what matters is how many warps an SM holds: a ROW (pair of every column) is shared by
// L adjacent lanes of a warp.  Each lane loads (and binds, and stores) the columns k = sub, sub + L, ... of its row into the
// block's shared memory as value and difference, and evaluates the monomials j = sub, sub + L, ...; the summand is linear
// in the inner sum, so a lane simply adds col0 * (its partial sum) to its own running round sums and the block reduction
// at the end adds the lanes up.  The rows of a warp are produced and consumed by that warp alone: __syncwarp suffices.
// Shared memory per block: 2 * nc * (T / L + 1) words, 16..24 KB, so 9 or more blocks of 128 threads share an SM
// (one block at 204 KB with a column set per thread).
constexpr int ZCX_MAXTERMS = 2048;
constexpr int ZCX_MAXC = 224;
struct ZcxHdr { uint32_t nterms, nc; gl_t konst; };

__global__ void zcx_round_kernel(const uint8_t* prog_g, const gl_t* const* in, gl_t* const* out, size_t items, int first,
                                 uint32_t L, ZkhCtl* ctl, gl_t* partials, const gl_t* chal_prev, gl_t* msg_out, gl_t* chal_out,
                                 ZkhTag tag) {
    extern __shared__ __align__(16) uint8_t smem[];
    const ZcxHdr hdr = *reinterpret_cast<const ZcxHdr*>(prog_g);
    const uint32_t nc = hdr.nc, nterms = hdr.nterms, T = blockDim.x, tid = threadIdx.x;
    const uint32_t R = T / L, RP = R + 1;      // rows per block pass; padded row stride of the value tables
    const uint32_t r = tid / L, sub = tid % L;
    gl_t* coef = reinterpret_cast<gl_t*>(smem);
    gl_t* cur = coef + nterms;                 // [nc][RP]: the columns' values at the current evaluation point
    gl_t* dif = cur + (size_t)nc * RP;         // [nc][RP]: hi - lo
    gl_t* sh = dif + (size_t)nc * RP;          // SCW_NT * 32
    uint32_t* packed = reinterpret_cast<uint32_t*>(sh + SCW_NT * 32);
    const gl_t* coef_g = reinterpret_cast<const gl_t*>(prog_g + sizeof(ZcxHdr));
    const uint32_t* packed_g = reinterpret_cast<const uint32_t*>(coef_g + nterms);
    for (uint32_t j = tid; j < nterms; j += T) { coef[j] = coef_g[j]; packed[j] = packed_g[j]; }
    __syncthreads();
    const gl_t a = first ? 0 : *chal_prev;
    const gl_t konst = sub == 0 ? hdr.konst : 0;
    gl_t s[SCW_NT];
#pragma unroll
    for (int t = 0; t < SCW_NT; t++) s[t] = 0;
    const size_t stride = (size_t)gridDim.x * R;
    for (size_t base = (size_t)blockIdx.x * R; base < items; base += stride) {
        const size_t i = base + r;
        const bool live = i < items;
        for (uint32_t k = sub; k < nc; k += L) {
            gl_t lo = 0, hi = 0;
            if (live) {
                if (first) {
                    ulonglong2 v = ld2(in[k] + 2 * i);
                    lo = v.x;
                    hi = v.y;
                } else {
                    const gl_t* src = in[k];
                    ulonglong2 u = ld2(src + 4 * i), w = ld2(src + 4 * i + 2);
                    lo = gl_lerp(u.x, u.y, a);
                    hi = gl_lerp(w.x, w.y, a);
                    st2(out[k] + 2 * i, lo, hi);
                }
            }
            cur[(size_t)k * RP + r] = lo;
            dif[(size_t)k * RP + r] = gl_sub(hi, lo);
        }
        __syncwarp();
#pragma unroll 1
        for (int t = 0; t < SCW_NT; t++) {
            Acc192 acc, accf;
            acc.clear();
            accf.clear();
            for (uint32_t j = sub; j < nterms; j += L) {
                const uint32_t pk = packed[j];
                gl_t x = cur[(size_t)((pk >> 8) & 0xff) * RP + r];
                if ((pk & 0x7f) >= 2) x = gl_mul(x, cur[(size_t)((pk >> 16) & 0xff) * RP + r]);
                if ((pk & 0x7f) >= 3) x = gl_mul(x, cur[(size_t)((pk >> 24) & 0xff) * RP + r]);
                if (pk & 0x80) accf.add_prod(coef[j], x);
                else acc.add_prod(coef[j], x);
            }
            if (live) s[t] = gl_add(s[t], gl_add(gl_mul(cur[r], gl_add(acc.reduce(), konst)), accf.reduce()));
            __syncwarp();                      // every lane of the row has read the values of this point
            if (t + 1 < SCW_NT)
                for (uint32_t k = sub; k < nc; k += L) cur[(size_t)k * RP + r] = gl_add(cur[(size_t)k * RP + r], dif[(size_t)k * RP + r]);
            __syncwarp();
        }
    }
    grid_finish<SCW_NT>(s, sh, ctl, partials, msg_out, chal_out, tag, ctl->par[6] ? 3 : 0);
}

__global__ void zcx_finals_kernel(const gl_t* const* in, int nc, const gl_t* chal, gl_t* out) {
    for (int k = threadIdx.x; k < nc; k += blockDim.x) out[k] = gl_lerp(in[k][0], in[k][1], *chal);
}

static size_t zcx_smem_bytes(int nc, uint32_t nterms, int T, int L) {
    return (size_t)nterms * 8 + (size_t)2 * nc * (T / L + 1) * 8 + SCW_NT * 32 * 8 + (size_t)nterms * 4 + 16;
}

// prog_dev: ZcxHdr | coef | packed (already uploaded); ptr_dev: room for logn * 2 * nc pointers
static int zcx_enqueue(zkh_ctx* ctx, const gl_t* const* in, int nc, uint32_t nterms, uint32_t logn, const uint8_t* prog_dev,
                       const gl_t** ptr_dev, const ZkhTag& tag, gl_t* finals_dev) {
    cudaStream_t s = ctx->stream;
    ZkhCtl* ctl = ctx->d_ctl;
    const size_t n = (size_t)1 << logn;
    // 128 threads per block; L lanes per row, the smallest power of two that brings the value tables of a block to 24 KB
    const int T = 128;
    int L = 1;
    while (L < 32 && (size_t)2 * nc * (T / L + 1) * 8 > 24 * 1024) L <<= 1;
    if (const char* e = getenv("ZKH_ZCX_LANES")) {            // measurement knob: 1, 2, 4, ... 32
        const int v = atoi(e);
        if (v >= 1 && v <= 32 && !(v & (v - 1))) L = v;
    }
    const size_t smem = zcx_smem_bytes(nc, nterms, T, L);
    if (smem > 220 * 1024) return zkh_fail(ctx, ZKH_ERR_LIMIT, "zero-check: program does not fit shared memory");
    // the limit is raised once per device to the largest program this entry point accepts: a per-call value would let one
    // host thread lower it between another thread's call and its launch
    static ZkhOncePerDevice attr;
    zkh_once_on_device(attr, ctx->device, [] { cudaFuncSetAttribute(zcx_round_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024); });
    int occ = 1;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, zcx_round_kernel, T, smem) != cudaSuccess || occ < 1) occ = 1;
    const size_t R = (size_t)T / L;
    auto grid_for = [&](size_t items) {
        size_t want = (items + R - 1) / R, cap = (size_t)ctx->sm_count * occ;
        if (cap > ctx->partials_cap / SCW_NT) cap = ctx->partials_cap / SCW_NT;
        return (unsigned)(want < cap ? want : cap);
    };
    // pointer tables of every round: round r reads table 2r, writes table 2r+1
    std::vector<const gl_t*> tab((size_t)logn * 2 * nc, nullptr);
    gl_t* bufA = (gl_t*)ctx->ws;
    gl_t* bufB = (gl_t*)((char*)ctx->ws + zkh_align((size_t)nc * (n / 2 + 1) * 8));
    gl_t* dst = bufA;
    size_t cur_n = n;
    for (int k = 0; k < nc; k++) tab[k] = in[k];
    for (uint32_t r = 1; r < logn; r++) {
        const size_t out_n = cur_n / 2;
        for (int k = 0; k < nc; k++) {
            tab[((size_t)2 * r + 1) * nc + k] = dst + (size_t)k * out_n;
            tab[((size_t)2 * r) * nc + k] = r == 1 ? in[k] : tab[((size_t)2 * (r - 1) + 1) * nc + k];
        }
        dst = (dst == bufA) ? bufB : bufA;
        cur_n = out_n;
    }
    ZKH_CUDA(ctx, cudaMemcpyAsync(ptr_dev, tab.data(), tab.size() * sizeof(void*), cudaMemcpyHostToDevice, s));
    ZKH_CUDA(ctx, cudaStreamSynchronize(s));      // tab is a host temporary
    zcx_round_kernel<<<grid_for(n / 2), T, smem, s>>>(prog_dev, ptr_dev, nullptr, n / 2, 1, (uint32_t)L, ctl, ctx->d_partials, nullptr,
                                                     ctl->msgs, ctl->chals, tag);
    cur_n = n;
    for (uint32_t r = 1; r < logn; r++) {
        zcx_round_kernel<<<grid_for(cur_n / 4), T, smem, s>>>(
            prog_dev, ptr_dev + ((size_t)2 * r) * nc, (gl_t* const*)(ptr_dev + ((size_t)2 * r + 1) * nc), cur_n / 4, 0, (uint32_t)L, ctl,
            ctx->d_partials, ctl->chals + (r - 1), ctl->msgs + (size_t)r * SCW_NT, ctl->chals + r, tag);
        cur_n /= 2;
    }
    const gl_t** last = logn == 1 ? ptr_dev : ptr_dev + ((size_t)2 * (logn - 1) + 1) * nc;
    zcx_finals_kernel<<<1, 256, 0, s>>>(last, nc, ctl->chals + (logn - 1), finals_dev);
    return cudaGetLastError() == cudaSuccess ? ZKH_OK : zkh_fail(ctx, ZKH_ERR_CUDA, "zero-check sumcheck launch");
}

static int scw_shape(int functor, int* nc, int* nlam) {
#define CASE(F) if (functor == F) { *nc = WFn<F>::NC; *nlam = WFn<F>::NLAM; return 1; }
    CASE(ZKH_F_HW_DP) CASE(ZKH_F_HW_DG) CASE(ZKH_F_HW_CH) CASE(ZKH_F_HW_GS) CASE(ZKH_F_HW_DS) CASE(ZKH_F_HW_DO)
#undef CASE
    return 0;
}

}  // namespace zkh

using namespace zkh;

extern "C" int zkh_sumcheck_wide_shape(int functor, int* nc, int* nlam) {
    int a = 0, b = 0;
    if (!scw_shape(functor, &a, &b)) return ZKH_ERR_ARG;
    if (nc) *nc = a;
    if (nlam) *nlam = b;
    return ZKH_OK;
}

extern "C" int zkh_sumcheck_wide(zkh_ctx* ctx, int functor, const uint64_t* const* cols_dev, int nc, uint32_t logn,
                                 const uint64_t* lam, int nlam, const char* tag, uint8_t state[32], uint64_t* msgs,
                                 uint64_t* chals, uint64_t* finals) {
    if (!ctx) return ZKH_ERR_ARG;
    if (!cols_dev || !lam || !tag || !state || !msgs || !chals) return zkh_fail(ctx, ZKH_ERR_ARG, "wide sumcheck: null pointer");
    int want_nc = 0, want_nlam = 0;
    if (!scw_shape(functor, &want_nc, &want_nlam)) return zkh_fail(ctx, ZKH_ERR_ARG, "wide sumcheck: unknown summand");
    if (nc != want_nc || nlam != want_nlam)
        return zkh_fail(ctx, ZKH_ERR_ARG, "wide sumcheck: column or coefficient count does not match the summand");
    if (logn < 1 || logn > 34) return zkh_fail(ctx, ZKH_ERR_ARG, "wide sumcheck: logn must be 1..34");
    if (strlen(tag) > ZKH_TR_MAX_LABEL) return zkh_fail(ctx, ZKH_ERR_LIMIT, "wide sumcheck: tag longer than 48 bytes");
    for (int j = 0; j < nlam; j++)
        if (lam[j] >= GL_P) return zkh_fail(ctx, ZKH_ERR_DOMAIN, "wide sumcheck: coefficient not canonical");
    ZKH_CUDA(ctx, cudaSetDevice(ctx->device));
    ZKH_TRY(zkh_ws_reserve(ctx, scw_workspace_bytes(nc, logn)));
    ZkhCtl* h = ctx->h_ctl;
    digest_from_bytes(state, h->st);
    h->counter = 0;
    h->err = 0;
    for (int i = 0; i < 8; i++) h->par[i] = 0;
    for (int j = 0; j < 64; j++) h->aux[j] = j < nlam ? lam[j] : 0;
    ZKH_CUDA(ctx, cudaMemcpyAsync(ctx->d_ctl, h, offsetof(ZkhCtl, local), cudaMemcpyHostToDevice, ctx->stream));
    ZKH_CUDA(ctx, cudaMemcpyAsync(ctx->d_ctl->aux, h->aux, sizeof h->aux, cudaMemcpyHostToDevice, ctx->stream));
    const size_t n = (size_t)1 << logn;
    gl_t* finals_dev = (gl_t*)((char*)ctx->ws + zkh_align((size_t)nc * (n / 2 + 1) * 8) + zkh_align((size_t)nc * (n / 4 + 1) * 8));
    const ZkhTag t = zkh_make_tag(tag);
    int rc = ZKH_ERR_ARG;
#define CASE(F) if (functor == F) rc = scw_enqueue_t<F>(ctx, cols_dev, logn, t, finals_dev);
    CASE(ZKH_F_HW_DP) CASE(ZKH_F_HW_DG) CASE(ZKH_F_HW_CH) CASE(ZKH_F_HW_GS) CASE(ZKH_F_HW_DS) CASE(ZKH_F_HW_DO)
#undef CASE
    ZKH_TRY(rc);
    ZKH_CUDA(ctx, cudaMemcpyAsync(h, ctx->d_ctl, sizeof(ZkhCtl), cudaMemcpyDeviceToHost, ctx->stream));
    if (finals)
        ZKH_CUDA(ctx, cudaMemcpyAsync(finals, finals_dev, (size_t)nc * 8, cudaMemcpyDeviceToHost, ctx->stream));
    ZKH_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (h->err) return zkh_fail(ctx, ZKH_ERR_DEVICE, "wide sumcheck: device error flag set");
    memcpy(msgs, h->msgs, (size_t)logn * SCW_NT * 8);
    memcpy(chals, h->chals, (size_t)logn * 8);
    digest_to_bytes(h->st, state);
    return ZKH_OK;
}

// prog: [0] = number of terms, [1] = constant inside the bracket, then per term (coefficient, packed) with
// packed = degree | idx0 << 8 | idx1 << 16 | idx2 << 24
static int zerocheck_impl(zkh_ctx* ctx, const uint64_t* const* cols_dev, int nc, uint32_t logn,
                          const uint64_t* prog, int nwords, const char* tag, uint8_t state[32], uint64_t* msgs,
                          uint64_t* chals, uint64_t* finals, const uint64_t* fix, uint64_t* pref_out, uint32_t rounds = 0,
                          uint64_t pref_in = 0) {
    if (!ctx) return ZKH_ERR_ARG;
    if (rounds == 0) rounds = logn;
    if (!cols_dev || !prog || !tag || !state || !msgs || !chals) return zkh_fail(ctx, ZKH_ERR_ARG, "zero-check: null pointer");
    if (nc < 1 || nc > ZCX_MAXC) return zkh_fail(ctx, ZKH_ERR_ARG, "zero-check: 1..224 columns");
    if (logn < 1 || logn > 34) return zkh_fail(ctx, ZKH_ERR_ARG, "zero-check: logn must be 1..34");
    if (strlen(tag) > ZKH_TR_MAX_LABEL) return zkh_fail(ctx, ZKH_ERR_LIMIT, "zero-check: tag longer than 48 bytes");
    if (nwords < 2 || prog[0] > ZCX_MAXTERMS || (uint64_t)nwords != 2 + 2 * prog[0])
        return zkh_fail(ctx, ZKH_ERR_ARG, "zero-check: malformed program (at most 2048 terms)");
    const uint32_t nterms = (uint32_t)prog[0];
    const bool large = nc > 32 || nterms > ZC_MAXTERMS;
    if (rounds > logn || pref_in >= GL_P) return zkh_fail(ctx, ZKH_ERR_ARG, "zero-check: rounds beyond the chain or pref not canonical");
    if (rounds < logn && large) return zkh_fail(ctx, ZKH_ERR_LIMIT, "zero-check: partial chains run on the small engine (<= 32 columns, 120 terms)");
    const size_t nleft = ((size_t)1 << logn) >> rounds;
    if (prog[1] >= GL_P) return zkh_fail(ctx, ZKH_ERR_DOMAIN, "zero-check: constant not canonical");
    ZkhZcProg hp;          // staging copies (pageable memory: the asynchronous copies below return after staging them)
    std::vector<uint8_t> hx;
    if (!large) {
        memset(&hp, 0, sizeof hp);
        hp.nterms = nterms;
        hp.nc = (uint32_t)nc;
        hp.konst = prog[1];
    } else {
        hx.assign(sizeof(ZcxHdr) + (size_t)nterms * 12, 0);
        ZcxHdr hd{nterms, (uint32_t)nc, prog[1]};
        memcpy(hx.data(), &hd, sizeof hd);
    }
    for (uint32_t j = 0; j < nterms; j++) {
        const uint64_t coef = prog[2 + 2 * j], pk = prog[3 + 2 * j];
        const uint32_t deg = pk & 0x7f;      // bit 7: the term stands outside the col0 factor
        if (coef >= GL_P) return zkh_fail(ctx, ZKH_ERR_DOMAIN, "zero-check: coefficient not canonical");
        if (deg < 1 || deg > 3 || (pk >> 32)) return zkh_fail(ctx, ZKH_ERR_ARG, "zero-check: term degree must be 1..3");
        for (uint32_t k = 0; k < deg; k++)
            if (((pk >> (8 + 8 * k)) & 0xff) >= (uint64_t)nc) return zkh_fail(ctx, ZKH_ERR_ARG, "zero-check: column index out of range");
        if (!large) {
            hp.coef[j] = coef;
            hp.packed[j] = (uint32_t)pk;
        } else {
            memcpy(hx.data() + sizeof(ZcxHdr) + (size_t)j * 8, &coef, 8);
            const uint32_t pk32 = (uint32_t)pk;
            memcpy(hx.data() + sizeof(ZcxHdr) + (size_t)nterms * 8 + (size_t)j * 4, &pk32, 4);
        }
    }
    ZKH_CUDA(ctx, cudaSetDevice(ctx->device));
    const size_t n = (size_t)1 << logn;
    const size_t szA = zkh_align((size_t)nc * (n / 2 + 1) * 8), szB = zkh_align((size_t)nc * (n / 4 + 1) * 8);
    const size_t szF = zkh_align((size_t)nc * nleft * 8);
    const size_t szP = zkh_align(large ? hx.size() : sizeof(ZkhZcProg)), szT = zkh_align((size_t)logn * 2 * nc * sizeof(void*));
    const size_t szX = zkh_align((8 + 8 * (size_t)logn) * 8);
    ZKH_TRY(zkh_ws_reserve(ctx, szA + szB + szF + szP + szT + szX));
    gl_t* fix_dev = (gl_t*)((char*)ctx->ws + szA + szB + szF + szP + szT);
    std::vector<gl_t> hfix;
    if (fix) {
        hfix.assign(8 + 8 * (size_t)logn, 0);
        hfix[0] = pref_in;
        for (uint32_t r = 0; r < rounds; r++)
            for (int k = 0; k < 7; k++) {
                if (fix[7 * (size_t)r + k] >= GL_P) return zkh_fail(ctx, ZKH_ERR_DOMAIN, "zero-check: blind coefficient not canonical");
                hfix[8 + 8 * (size_t)r + k] = fix[7 * (size_t)r + k];
            }
    }
    gl_t* finals_dev = (gl_t*)((char*)ctx->ws + szA + szB);
    uint8_t* prog_dev = (uint8_t*)ctx->ws + szA + szB + szF;
    const gl_t** ptr_dev = (const gl_t**)((char*)ctx->ws + szA + szB + szF + szP);
    ZkhCtl* h = ctx->h_ctl;
    digest_from_bytes(state, h->st);
    h->counter = 0;
    h->err = 0;
    for (int i = 0; i < 8; i++) h->par[i] = 0;
    if (fix) {
        h->par[6] = (gl_t)(uintptr_t)fix_dev;
        ZKH_CUDA(ctx, cudaMemcpyAsync(fix_dev, hfix.data(), hfix.size() * 8, cudaMemcpyHostToDevice, ctx->stream));
    }
    ZKH_CUDA(ctx, cudaMemcpyAsync(ctx->d_ctl, h, offsetof(ZkhCtl, local), cudaMemcpyHostToDevice, ctx->stream));
    ZKH_CUDA(ctx, cudaMemcpyAsync(prog_dev, large ? (const void*)hx.data() : (const void*)&hp, large ? hx.size() : sizeof hp,
                                  cudaMemcpyHostToDevice, ctx->stream));
    const ZkhTag t = zkh_make_tag(tag);
    int rc = large ? zcx_enqueue(ctx, cols_dev, nc, nterms, logn, prog_dev, ptr_dev, t, finals_dev)
           : nc <= 8 ? zc_enqueue_t<8>(ctx, cols_dev, nc, logn, (const ZkhZcProg*)prog_dev, t, finals_dev, rounds)
           : nc <= 16 ? zc_enqueue_t<16>(ctx, cols_dev, nc, logn, (const ZkhZcProg*)prog_dev, t, finals_dev, rounds)
                      : zc_enqueue_t<32>(ctx, cols_dev, nc, logn, (const ZkhZcProg*)prog_dev, t, finals_dev, rounds);
    ZKH_TRY(rc);
    ZKH_CUDA(ctx, cudaMemcpyAsync(h, ctx->d_ctl, sizeof(ZkhCtl), cudaMemcpyDeviceToHost, ctx->stream));
    if (finals)
        ZKH_CUDA(ctx, cudaMemcpyAsync(finals, finals_dev, (size_t)nc * nleft * 8, cudaMemcpyDeviceToHost, ctx->stream));
    if (fix && pref_out) ZKH_CUDA(ctx, cudaMemcpyAsync(pref_out, fix_dev, 8, cudaMemcpyDeviceToHost, ctx->stream));
    ZKH_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (h->err) return zkh_fail(ctx, ZKH_ERR_DEVICE, "zero-check: device error flag set");
    memcpy(msgs, h->msgs, (size_t)rounds * SCW_NT * 8);
    memcpy(chals, h->chals, (size_t)rounds * 8);
    digest_to_bytes(h->st, state);
    return ZKH_OK;
}

extern "C" int zkh_sumcheck_zerocheck(zkh_ctx* ctx, const uint64_t* const* cols_dev, int nc, uint32_t logn,
                                      const uint64_t* prog, int nwords, const char* tag, uint8_t state[32], uint64_t* msgs,
                                      uint64_t* chals, uint64_t* finals) {
    return zerocheck_impl(ctx, cols_dev, nc, logn, prog, nwords, tag, state, msgs, chals, finals, nullptr, nullptr);
}
// The same chain under a structured Libra blind (zkllm-src/p3_hawkeye.cuh:1065-1110, :1329-1331): fix holds, per round, the five
// coefficients of g_rd, A_rd = rho * 2^(v-1-rd) and B_rd = rho * 2^(v-2-rd) * suf[rd+1]; the message of round rd gains
// A_rd * (pref + g_rd(t)) + B_rd with pref = sum_{i < rd} g_i(a_i), all on the device.  pref_out: g(r) after the last round.
extern "C" int zkh_sumcheck_zerocheck_blind(zkh_ctx* ctx, const uint64_t* const* cols_dev, int nc, uint32_t logn,
                                            const uint64_t* prog, int nwords, const uint64_t* fix, const char* tag,
                                            uint8_t state[32], uint64_t* msgs, uint64_t* chals, uint64_t* finals,
                                            uint64_t* pref_out) {
    if (!ctx) return ZKH_ERR_ARG;
    if (!fix || !pref_out) return zkh_fail(ctx, ZKH_ERR_ARG, "zero-check: the blinded chain needs its table and pref_out");
    return zerocheck_impl(ctx, cols_dev, nc, logn, prog, nwords, tag, state, msgs, chals, finals, fix, pref_out);
}

// The first `rounds` rounds of a chain whose later variables belong to other columns (a factored product domain): messages,
// challenges and transcript advance as in the full chain; `left` receives, per column, the 2^(logn - rounds) values that remain
// after the last bind.  fix (optional): the structured blind's table rows of THESE rounds (7 words each), pref_in / pref_out
// its running prefix, carried from one partial chain to the next.
extern "C" int zkh_sumcheck_zerocheck_partial(zkh_ctx* ctx, const uint64_t* const* cols_dev, int nc, uint32_t logn, uint32_t rounds,
                                              const uint64_t* prog, int nwords, const uint64_t* fix, uint64_t pref_in,
                                              const char* tag, uint8_t state[32], uint64_t* msgs, uint64_t* chals,
                                              uint64_t* left, uint64_t* pref_out) {
    if (!ctx) return ZKH_ERR_ARG;
    if (rounds < 1 || !left) return zkh_fail(ctx, ZKH_ERR_ARG, "zero-check: a partial chain needs 1..logn rounds and the buffer for what is left");
    if (fix && !pref_out) return zkh_fail(ctx, ZKH_ERR_ARG, "zero-check: the blinded chain needs pref_out");
    return zerocheck_impl(ctx, cols_dev, nc, logn, prog, nwords, tag, state, msgs, chals, left, fix, pref_out, rounds, pref_in);
}
