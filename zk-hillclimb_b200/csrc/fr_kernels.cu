// BLS12-381 Fr back-end of the sumcheck engine for sm_100a: multilinear folds, eq tables and the
// round loops of the reference's product sumchecks (inner product, Hadamard, bracket).
//
// Reference paths replaced (all values plain canonical integers mod p, 32 bytes each):
//   * zkip round loop              zkllm-src/zkob_fc.cu:276-332, kernels zkfc.cu:94-127
//   * Hadamard / bracket rounds    zkllm-src/zkob_lookup.cuh:214-315 (k_hp3_step, fs_hadamard), :321-425
//   * k_fr_fold, k_eq_expand, build_eq_tensor   zkob_lookup.cuh:202-212, :247-268
//   * FrTensor::partial_me / operator()(u) / multi_dim_me   fr-tensor.cu:542-652
// The reference spends per round: one kernel writing nt full-size temporaries, nt log-depth tree sums,
// a host transcript step, one fold kernel per column with a fresh allocation, and device-wide syncs in
// between.  Here one kernel per round binds the columns with the previous challenge (MSB-first pairs
// (i, i+h), as the reference folds), stores the halved columns, accumulates the round evaluations from
// the values it just produced, reduces over the grid through the last CTA to finish, and runs the
// Fiat-Shamir step (nt labelled 32-byte absorbs, challenge with the reference's limb mapping) on the
// device.  The host queues all rounds and reads the results back once.
#include "fr_dev.cuh"

namespace zkh {

// Round end on warp 0: make the sums plain, publish them, absorb each under its label, draw the
// challenge (zkllm-src/vrf_common.cuh:233-244: limbs from the challenge bytes, top limb reduced
// modulo the top limb of p, redraw on zero; the redraw is bounded here and flags an error).
template <int NT>
__device__ __noinline__ void fr_finish_round(Fr (&s)[NT], int rpow, ZkhCtl* ctl, Fr* msg_out, Fr* chal_out,
                                             const FrLabels& lab) {
    __shared__ uint32_t trbuf[ZKH_TRBUF_WORDS];
    __shared__ __align__(16) Fr mvals[NT];
    const uint32_t lane = threadIdx.x & 31;
    if (lane == 0) {
#pragma unroll
        for (int t = 0; t < NT; t++) {
            Fr plain = fr_mmul(s[t], FR_RPOW[rpow]);
            msg_out[t] = plain;
            mvals[t] = plain;
        }
    }
    __syncwarp();
    uint32_t st[8];
#pragma unroll
    for (int i = 0; i < 8; i++) st[i] = ctl->st[i];
    for (int t = 0; t < NT; t++)
        tr_warp_absorb(st, lab.t[t].s, lab.t[t].len, reinterpret_cast<const uint64_t*>(&mvals[t]), 4, trbuf);
    Fr x;
    bool ok = false;
    for (int tries = 0; tries < 8 && !ok; tries++) {
        tr_warp_challenge_limbs(st, x.v);
        x.v[7] %= 0x73eda753u;
        ok = !fr_is_zero(x);
    }
    if (lane == 0) {
        if (!ok) atomicOr(&ctl->err, 2u);
#pragma unroll
        for (int i = 0; i < 8; i++) ctl->st[i] = st[i];
        *chal_out = x;
    }
}

template <int NT>
__device__ __forceinline__ void fr_grid_finish(Fr (&s)[NT], int rpow, Fr* sh, ZkhCtl* ctl, Fr* partials, Fr* msg_out,
                                               Fr* chal_out, const FrLabels& lab) {
    __shared__ int is_last;
    fr_block_sum<NT>(s, sh);
    if (threadIdx.x == 0) {
#pragma unroll
        for (int t = 0; t < NT; t++) partials[(size_t)blockIdx.x * NT + t] = s[t];
        __threadfence();
        unsigned prev = atomicAdd(&ctl->counter, 1u);
        is_last = (prev == gridDim.x - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    Fr v[NT];
#pragma unroll
    for (int t = 0; t < NT; t++) v[t] = fr_zero();
    for (unsigned b = threadIdx.x; b < gridDim.x; b += blockDim.x)
#pragma unroll
        for (int t = 0; t < NT; t++) {
            const volatile uint32_t* src = reinterpret_cast<const volatile uint32_t*>(&partials[(size_t)b * NT + t]);
            Fr x;
#pragma unroll
            for (int i = 0; i < 8; i++) x.v[i] = src[i];
            v[t] = fr_add(v[t], x);
        }
    fr_block_sum<NT>(v, sh);
    if (threadIdx.x < 32) {
        if (threadIdx.x == 0) ctl->counter = 0;
        fr_finish_round<NT>(v, rpow, ctl, msg_out, chal_out, lab);
    }
}

// ------------------------------------------------------------------ product sumcheck rounds
// Summand: the product of NC columns; NT = NC + 1 evaluations at t = 0..NC.
// first: message over in[] of length 2*half (pairs (i, i+half)), items = half.
// else : in[] has length 4*items; bind pairs (i, i+2*items) with *chal_prev into out[] (length
//        2*items), message over pairs (i, i+items) of out[].
template <int NC>
__global__ void __launch_bounds__(FR_THREADS)
fr_sc_round_kernel(FrPtrs P, size_t items, int first, ZkhCtl* ctl, Fr* partials, const Fr* chal_prev, Fr* msg_out,
                   Fr* chal_out, FrLabels lab) {
    constexpr int NT = NC + 1;
    __shared__ __align__(16) Fr sh[NT * 32];
    Fr xm = fr_zero();
    if (!first) xm = fr_to_mont(*chal_prev);
    Fr acc[NT];
#pragma unroll
    for (int t = 0; t < NT; t++) acc[t] = fr_zero();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < items; i += stride) {
        Fr cur[NC], dif[NC];
#pragma unroll
        for (int k = 0; k < NC; k++) {
            Fr lo, hi;
            if (first) {
                lo = fr_load(P.in[k] + i);
                hi = fr_load(P.in[k] + i + items);
            } else {
                lo = fr_lerp(fr_load(P.in[k] + i), fr_load(P.in[k] + i + 2 * items), xm);
                hi = fr_lerp(fr_load(P.in[k] + i + items), fr_load(P.in[k] + i + 3 * items), xm);
                fr_store(P.out[k] + i, lo);
                fr_store(P.out[k] + i + items, hi);
            }
            cur[k] = lo;
            dif[k] = fr_sub(hi, lo);
        }
#pragma unroll
        for (int t = 0; t < NT; t++) {
            Fr prod = cur[0];
#pragma unroll
            for (int k = 1; k < NC; k++) prod = fr_mmul(prod, cur[k]);  // carries R^-(NC-1)
            acc[t] = fr_add(acc[t], prod);
            if (t + 1 < NT) {
#pragma unroll
                for (int k = 0; k < NC; k++) cur[k] = fr_add(cur[k], dif[k]);
            }
        }
    }
    fr_grid_finish<NT>(acc, NC - 1, sh, ctl, partials, msg_out, chal_out, lab);
}

// finals[k] = in[k][0] + x*(in[k][1] - in[k][0])
__global__ void fr_sc_finals_kernel(FrPtrs P, int nc, const Fr* chal, Fr* out) {
    int k = threadIdx.x;
    if (k < nc) out[k] = fr_lerp(P.in[k][0], P.in[k][1], fr_to_mont(*chal));
}

// ------------------------------------------------------------------ folds and eq tables
// out[i] = in[i] + w*(in[i+h] - in[i])      (k_fr_fold)
__global__ void fr_fold_kernel(const Fr* in, Fr w, Fr* out, size_t h) {
    const Fr wm = fr_to_mont(w);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < h; i += (size_t)gridDim.x * blockDim.x)
        fr_store(out + i, fr_lerp(fr_load(in + i), fr_load(in + i + h), wm));
}
// one doubling step in place: E[i+n] = c*E[i], E[i] = E[i] - c*E[i]   (k_eq_expand: same values)
__global__ void fr_eq_expand_kernel(Fr* E, Fr c, size_t n) {
    const Fr cm = fr_to_mont(c);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        Fr e = E[i], hi = fr_mmul(cm, e);
        fr_store(E + i + n, hi);
        fr_store(E + i, fr_sub(e, hi));
    }
}
// the first levels (up to 2^10 entries) in one CTA
__global__ void fr_eq_head_kernel(Fr* E, const Fr* u, int levels) {
    if (threadIdx.x == 0) { Fr one = fr_zero(); one.v[0] = 1; E[0] = one; }
    __syncthreads();
    for (int l = 0; l < levels; l++) {
        const uint32_t n = 1u << l;
        const Fr cm = fr_to_mont(u[l]);
        if (threadIdx.x < n) {
            Fr e = E[threadIdx.x], hi = fr_mmul(cm, e);
            E[threadIdx.x + n] = hi;
            E[threadIdx.x] = fr_sub(e, hi);
        }
        __syncthreads();
    }
}

// partials[b] = sum over this CTA of a[i]*b[i] / R
__global__ void __launch_bounds__(FR_THREADS) fr_dot_kernel(const Fr* a, const Fr* b, size_t n, Fr* partials) {
    __shared__ __align__(16) Fr sh[32];
    Fr acc[1] = {fr_zero()};
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        acc[0] = fr_add(acc[0], fr_mmul(fr_load(a + i), fr_load(b + i)));
    fr_block_sum<1>(acc, sh);
    if (threadIdx.x == 0) partials[blockIdx.x] = acc[0];
}
// out = (sum of partials) * R^2 / R : plain value of a sum that carries R^-1
__global__ void __launch_bounds__(FR_THREADS) fr_sum_fix_kernel(const Fr* partials, unsigned n, Fr* out) {
    __shared__ __align__(16) Fr sh[32];
    Fr acc[1] = {fr_zero()};
    for (unsigned i = threadIdx.x; i < n; i += blockDim.x) acc[0] = fr_add(acc[0], partials[i]);
    fr_block_sum<1>(acc, sh);
    if (threadIdx.x == 0) *out = fr_mmul(acc[0], FR_RPOW[1]);
}

// out[o, w] = sum_d eq[d] * t[o, d, w]  for t viewed as [other, D, window]  (FrTensor::partial_me with
// D = 2^|u| a power of two).  One thread per output element; consecutive threads read consecutive w.
__global__ void __launch_bounds__(FR_THREADS)
fr_pme_strided_kernel(const Fr* t, const Fr* eq, size_t other, uint32_t D, size_t window, Fr* out) {
    const size_t total = other * window;
    for (size_t g = (size_t)blockIdx.x * blockDim.x + threadIdx.x; g < total; g += (size_t)gridDim.x * blockDim.x) {
        const size_t o = g / window, w = g % window;
        const Fr* base = t + o * D * window + w;
        Fr acc = fr_zero();
        for (uint32_t d = 0; d < D; d++) acc = fr_add(acc, fr_mmul(fr_load(eq + d), fr_load(base + (size_t)d * window)));
        fr_store(out + g, fr_mmul(acc, FR_RPOW[1]));
    }
}
// window == 1: one warp per output row, lanes stride over d (coalesced), shuffle reduction
__global__ void __launch_bounds__(FR_THREADS)
fr_pme_rows_kernel(const Fr* t, const Fr* eq, size_t other, uint32_t D, Fr* out) {
    const uint32_t lane = threadIdx.x & 31;
    const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = ((size_t)gridDim.x * blockDim.x) >> 5;
    for (size_t o = warp; o < other; o += nwarps) {
        Fr acc = fr_zero();
        for (uint32_t d = lane; d < D; d += 32) acc = fr_add(acc, fr_mmul(fr_load(eq + d), fr_load(t + o * D + d)));
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) acc = fr_add(acc, fr_shfl_down(acc, s));
        if (lane == 0) fr_store(out + o, fr_mmul(acc, FR_RPOW[1]));
    }
}

// integer-pipe probe: four independent chains of Montgomery products per thread
__global__ void __launch_bounds__(256) fr_mul_probe_kernel(Fr seed, uint32_t iters, Fr* out) {
    Fr a = seed, b = seed, c = seed, d = seed;
    a.v[0] ^= threadIdx.x; b.v[1] ^= blockIdx.x; c.v[2] ^= threadIdx.x * 7u; d.v[3] ^= blockIdx.x * 5u;
    for (uint32_t i = 0; i < iters; i++) {
        a = fr_mmul(a, b); b = fr_mmul(b, c); c = fr_mmul(c, d); d = fr_mmul(d, a);
    }
    if (fr_is_zero(fr_add(fr_add(a, b), fr_add(c, d)))) out[0] = a;   // keeps the chains alive
}

// E (2^v entries) from the point u (device, v entries)
int fr_eq_enqueue(zkh_ctx* c, const Fr* u_dev, const Fr* u_host, uint32_t v, Fr* E) {
    const int head = v < 10 ? (int)v : 10;
    fr_eq_head_kernel<<<1, 512, 0, c->stream>>>(E, u_dev, head);
    for (uint32_t l = head; l < v; l++) {
        const size_t n = (size_t)1 << l;
        fr_eq_expand_kernel<<<fr_grid(c, n, 8), FR_THREADS, 0, c->stream>>>(E, u_host[l], n);
    }
    return cudaGetLastError() == cudaSuccess ? ZKH_OK : zkh_fail(c, ZKH_ERR_CUDA, "fr eq launch");
}

// out[i] += c * in[i] (k_bo_axpy, zkllm-src/zkob_claims.cuh:386-391); c plain
__global__ void __launch_bounds__(FR_THREADS) fr_axpy_plain_kernel(Fr* out, const Fr* __restrict__ in, Fr cplain, size_t n) {
    const Fr cm = fr_to_mont(cplain);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        fr_store(out + i, fr_add(fr_load(out + i), fr_mmul(cm, fr_load(in + i))));
}
// out[i] = a[i] * b[i], all plain (Fr_elementwise_mul, zkllm-src/fr-tensor.cu:141-147); out may alias a or b
__global__ void __launch_bounds__(FR_THREADS) fr_mul_plain_kernel(Fr* out, const Fr* a, const Fr* b, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        fr_store(out + i, fr_mmul(fr_to_mont(fr_load(a + i)), fr_load(b + i)));
}
// partials[b][t] = sum over this CTA of (a_i + t da_i)(b_i + t db_i) / R for t = 0, 1, 2, pairs (i, i + h): the round
// evaluations of sum_x M(x) P(x) with the top variable free (k_bo_hp2, zkllm-src/zkob_claims.cuh:365-384)
__global__ void __launch_bounds__(FR_THREADS) fr_round_sums_kernel(const Fr* __restrict__ a, const Fr* __restrict__ b, size_t h, Fr* partials) {
    __shared__ __align__(16) Fr sh[3 * 32];
    Fr acc[3] = {fr_zero(), fr_zero(), fr_zero()};
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < h; i += (size_t)gridDim.x * blockDim.x) {
        Fr m = fr_load(a + i), p = fr_load(b + i);
        const Fr dm = fr_sub(fr_load(a + i + h), m), dp = fr_sub(fr_load(b + i + h), p);
#pragma unroll
        for (int t = 0; t < 3; t++) {
            acc[t] = fr_add(acc[t], fr_mmul(m, p));
            m = fr_add(m, dm);
            p = fr_add(p, dp);
        }
    }
    fr_block_sum<3>(acc, sh);
    if (threadIdx.x == 0)
#pragma unroll
        for (int t = 0; t < 3; t++) partials[(size_t)blockIdx.x * 3 + t] = acc[t];
}
__global__ void __launch_bounds__(FR_THREADS) fr_sum3_fix_kernel(const Fr* partials, unsigned n, Fr* out) {
    __shared__ __align__(16) Fr sh[3 * 32];
    Fr acc[3] = {fr_zero(), fr_zero(), fr_zero()};
    for (unsigned i = threadIdx.x; i < n; i += blockDim.x)
#pragma unroll
        for (int t = 0; t < 3; t++) acc[t] = fr_add(acc[t], partials[(size_t)i * 3 + t]);
    fr_block_sum<3>(acc, sh);
    if (threadIdx.x == 0)
#pragma unroll
        for (int t = 0; t < 3; t++) out[t] = fr_mmul(acc[t], FR_RPOW[1]);
}

}  // namespace zkh

using namespace zkh;

static int fr_point_check(zkh_ctx* c, const void* u, uint32_t v, const char* what) {
    if (v > 0 && !u) return zkh_fail(c, ZKH_ERR_ARG, what);
    for (uint32_t i = 0; i < v; i++)
        if (!fr_canonical((const uint32_t*)u + 8 * i)) return zkh_fail(c, ZKH_ERR_DOMAIN, "fr: point coordinate not below p");
    return ZKH_OK;
}

extern "C" int zkh_fr_eq_build(zkh_ctx* c, const void* u, uint32_t v, void* out_dev) {
    if (!c) return ZKH_ERR_ARG;
    if (!out_dev || v > 30) return zkh_fail(c, ZKH_ERR_ARG, "fr_eq_build: bad arguments");
    ZKH_TRY(fr_point_check(c, u, v, "fr_eq_build: null point"));
    ZKH_CUDA(c, cudaSetDevice(c->device));
    ZKH_TRY(zkh_ws_reserve(c, 32 * 32));
    ZKH_CUDA(c, cudaMemcpyAsync(c->ws, u, (size_t)v * 32, cudaMemcpyHostToDevice, c->stream));
    return fr_eq_enqueue(c, (const Fr*)c->ws, (const Fr*)u, v, (Fr*)out_dev);
}

extern "C" int zkh_fr_fold(zkh_ctx* c, const void* in_dev, uint64_t h, const void* w, void* out_dev) {
    if (!c) return ZKH_ERR_ARG;
    if (!in_dev || !out_dev || !w || h == 0) return zkh_fail(c, ZKH_ERR_ARG, "fr_fold: bad arguments");
    ZKH_TRY(fr_point_check(c, w, 1, "fr_fold: null challenge"));
    ZKH_CUDA(c, cudaSetDevice(c->device));
    Fr wv;
    memcpy(&wv, w, 32);
    fr_fold_kernel<<<fr_grid(c, h, 8), FR_THREADS, 0, c->stream>>>((const Fr*)in_dev, wv, (Fr*)out_dev, h);
    return cudaGetLastError() == cudaSuccess ? ZKH_OK : zkh_fail(c, ZKH_ERR_CUDA, "fr_fold launch");
}

extern "C" int zkh_fr_partial_me(zkh_ctx* c, const void* t_dev, uint64_t other, uint32_t logd, uint64_t window,
                                 const void* u, void* out_dev) {
    if (!c) return ZKH_ERR_ARG;
    if (!t_dev || !out_dev || other == 0 || window == 0 || logd > 30)
        return zkh_fail(c, ZKH_ERR_ARG, "fr_partial_me: bad arguments");
    ZKH_TRY(fr_point_check(c, u, logd, "fr_partial_me: null point"));
    ZKH_CUDA(c, cudaSetDevice(c->device));
    const size_t D = (size_t)1 << logd;
    ZKH_TRY(zkh_ws_reserve(c, 32 * 32 + D * 32));
    Fr* u_dev = (Fr*)c->ws;
    Fr* eq = (Fr*)((char*)c->ws + 32 * 32);
    ZKH_CUDA(c, cudaMemcpyAsync(u_dev, u, (size_t)logd * 32, cudaMemcpyHostToDevice, c->stream));
    ZKH_TRY(fr_eq_enqueue(c, u_dev, (const Fr*)u, logd, eq));
    if (window == 1)
        fr_pme_rows_kernel<<<fr_grid(c, other * 32, 8), FR_THREADS, 0, c->stream>>>((const Fr*)t_dev, eq, other, (uint32_t)D,
                                                                                   (Fr*)out_dev);
    else
        fr_pme_strided_kernel<<<fr_grid(c, other * window, 8), FR_THREADS, 0, c->stream>>>(
            (const Fr*)t_dev, eq, other, (uint32_t)D, window, (Fr*)out_dev);
    return cudaGetLastError() == cudaSuccess ? ZKH_OK : zkh_fail(c, ZKH_ERR_CUDA, "fr_partial_me launch");
}

extern "C" int zkh_fr_mle_eval(zkh_ctx* c, const void* t_dev, const void* u, uint32_t v, void* out32) {
    if (!c) return ZKH_ERR_ARG;
    if (!t_dev || !out32 || v > 30) return zkh_fail(c, ZKH_ERR_ARG, "fr_mle_eval: bad arguments");
    ZKH_TRY(fr_point_check(c, u, v, "fr_mle_eval: null point"));
    ZKH_CUDA(c, cudaSetDevice(c->device));
    const size_t n = (size_t)1 << v;
    const unsigned g = fr_grid(c, n, 8);
    ZKH_TRY(zkh_ws_reserve(c, 32 * 32 + n * 32 + (size_t)g * 32 + 32));
    Fr* u_dev = (Fr*)c->ws;
    Fr* eq = u_dev + 32;
    Fr* part = eq + n;
    Fr* res = part + g;
    ZKH_CUDA(c, cudaMemcpyAsync(u_dev, u, (size_t)v * 32, cudaMemcpyHostToDevice, c->stream));
    ZKH_TRY(fr_eq_enqueue(c, u_dev, (const Fr*)u, v, eq));
    fr_dot_kernel<<<g, FR_THREADS, 0, c->stream>>>((const Fr*)t_dev, eq, n, part);
    fr_sum_fix_kernel<<<1, FR_THREADS, 0, c->stream>>>(part, g, res);
    ZKH_CUDA(c, cudaMemcpyAsync(out32, res, 32, cudaMemcpyDeviceToHost, c->stream));
    ZKH_CUDA(c, cudaStreamSynchronize(c->stream));
    return ZKH_OK;
}

extern "C" int zkh_fr_dot(zkh_ctx* c, const void* a_dev, const void* b_dev, uint64_t n, void* out32) {
    if (!c) return ZKH_ERR_ARG;
    if (!a_dev || !b_dev || !out32 || !n) return zkh_fail(c, ZKH_ERR_ARG, "fr_dot: bad arguments");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    const unsigned g = fr_grid(c, n, 8);
    ZKH_TRY(zkh_ws_reserve(c, (size_t)g * 32 + 32));
    Fr* part = (Fr*)c->ws;
    Fr* res = part + g;
    fr_dot_kernel<<<g, FR_THREADS, 0, c->stream>>>((const Fr*)a_dev, (const Fr*)b_dev, (size_t)n, part);
    fr_sum_fix_kernel<<<1, FR_THREADS, 0, c->stream>>>(part, g, res);
    ZKH_CUDA(c, cudaMemcpyAsync(out32, res, 32, cudaMemcpyDeviceToHost, c->stream));
    ZKH_CUDA(c, cudaStreamSynchronize(c->stream));
    return ZKH_OK;
}

template <int NC>
static int fr_sc_enqueue(zkh_ctx* c, const Fr* const* in, uint32_t logn, const FrLabels& lab, Fr* bufA, Fr* bufB,
                         Fr* partials, unsigned pcap, Fr* msgs, Fr* chals, Fr* finals) {
    constexpr int NT = NC + 1;
    const size_t n = (size_t)1 << logn;
    auto grid_for = [&](size_t items) {
        unsigned g = fr_grid(c, items, 4);
        return g < pcap ? g : pcap;
    };
    FrPtrs P;
    memset(&P, 0, sizeof P);
    for (int k = 0; k < NC; k++) P.in[k] = in[k];
    fr_sc_round_kernel<NC><<<grid_for(n / 2), FR_THREADS, 0, c->stream>>>(P, n / 2, 1, c->d_ctl, partials, nullptr, msgs,
                                                                         chals, lab);
    Fr* dst = bufA;
    size_t cur_n = n;
    for (uint32_t r = 1; r < logn; r++) {
        const size_t out_n = cur_n / 2;
        for (int k = 0; k < NC; k++) P.out[k] = dst + (size_t)k * out_n;
        fr_sc_round_kernel<NC><<<grid_for(cur_n / 4), FR_THREADS, 0, c->stream>>>(
            P, cur_n / 4, 0, c->d_ctl, partials, chals + (r - 1), msgs + (size_t)r * NT, chals + r, lab);
        for (int k = 0; k < NC; k++) P.in[k] = P.out[k];
        dst = (dst == bufA) ? bufB : bufA;
        cur_n = out_n;
    }
    fr_sc_finals_kernel<<<1, 32, 0, c->stream>>>(P, NC, chals + (logn - 1), finals);
    return cudaGetLastError() == cudaSuccess ? ZKH_OK : zkh_fail(c, ZKH_ERR_CUDA, "fr sumcheck launch");
}

extern "C" int zkh_fr_sumcheck(zkh_ctx* c, const void* const* cols_dev, int nc, uint32_t logn, const char* const* labels,
                               uint8_t state[32], void* evals, void* chals, void* finals) {
    if (!c) return ZKH_ERR_ARG;
    if (!cols_dev || !labels || !state || !evals || !chals) return zkh_fail(c, ZKH_ERR_ARG, "fr_sumcheck: null pointer");
    if (nc < 2 || nc > FR_MAXC) return zkh_fail(c, ZKH_ERR_ARG, "fr_sumcheck: 2..4 columns");
    if (logn < 1 || logn > 30) return zkh_fail(c, ZKH_ERR_ARG, "fr_sumcheck: logn must be 1..30");
    const int nt = nc + 1;
    FrLabels lab;
    memset(&lab, 0, sizeof lab);
    for (int t = 0; t < nt; t++) {
        if (!labels[t] || strlen(labels[t]) > ZKH_TR_MAX_LABEL) return zkh_fail(c, ZKH_ERR_LIMIT, "fr_sumcheck: bad label");
        lab.t[t] = zkh_make_tag(labels[t]);
    }
    ZKH_CUDA(c, cudaSetDevice(c->device));
    const size_t n = (size_t)1 << logn;
    const unsigned pcap = 4 * (unsigned)c->sm_count;
    const size_t szA = zkh_align((size_t)nc * (n / 2 + 1) * 32), szB = zkh_align((size_t)nc * (n / 4 + 1) * 32);
    const size_t szP = zkh_align((size_t)pcap * nt * 32), szM = zkh_align((size_t)logn * nt * 32);
    const size_t szC = zkh_align((size_t)logn * 32), szF = zkh_align((size_t)nc * 32);
    ZKH_TRY(zkh_ws_reserve(c, szA + szB + szP + szM + szC + szF));
    char* w = (char*)c->ws;
    Fr* bufA = (Fr*)w; w += szA;
    Fr* bufB = (Fr*)w; w += szB;
    Fr* part = (Fr*)w; w += szP;
    Fr* msgs = (Fr*)w; w += szM;
    Fr* chl = (Fr*)w; w += szC;
    Fr* fin = (Fr*)w;
    ZkhCtl* h = c->h_ctl;
    digest_from_bytes(state, h->st);
    h->counter = 0;
    h->err = 0;
    for (int i = 0; i < 8; i++) h->par[i] = 0;
    ZKH_CUDA(c, cudaMemcpyAsync(c->d_ctl, h, offsetof(ZkhCtl, local), cudaMemcpyHostToDevice, c->stream));
    const Fr* in[FR_MAXC];
    for (int k = 0; k < nc; k++) {
        if (!cols_dev[k]) return zkh_fail(c, ZKH_ERR_ARG, "fr_sumcheck: null column");
        in[k] = (const Fr*)cols_dev[k];
    }
    int rc = nc == 2 ? fr_sc_enqueue<2>(c, in, logn, lab, bufA, bufB, part, pcap, msgs, chl, fin)
           : nc == 3 ? fr_sc_enqueue<3>(c, in, logn, lab, bufA, bufB, part, pcap, msgs, chl, fin)
                     : fr_sc_enqueue<4>(c, in, logn, lab, bufA, bufB, part, pcap, msgs, chl, fin);
    ZKH_TRY(rc);
    ZKH_CUDA(c, cudaMemcpyAsync(h, c->d_ctl, offsetof(ZkhCtl, local), cudaMemcpyDeviceToHost, c->stream));
    ZKH_CUDA(c, cudaMemcpyAsync(evals, msgs, (size_t)logn * nt * 32, cudaMemcpyDeviceToHost, c->stream));
    ZKH_CUDA(c, cudaMemcpyAsync(chals, chl, (size_t)logn * 32, cudaMemcpyDeviceToHost, c->stream));
    if (finals) ZKH_CUDA(c, cudaMemcpyAsync(finals, fin, (size_t)nc * 32, cudaMemcpyDeviceToHost, c->stream));
    ZKH_CUDA(c, cudaStreamSynchronize(c->stream));
    if (h->err) return zkh_fail(c, ZKH_ERR_DEVICE, "fr_sumcheck: device error flag set");
    digest_to_bytes(h->st, state);
    return ZKH_OK;
}

extern "C" int zkh_fr_mul_throughput(zkh_ctx* c, uint32_t iters, double* gmul_per_s) {
    if (!c || !gmul_per_s || iters == 0 || iters > (1u << 20)) return zkh_fail(c, ZKH_ERR_ARG, "fr_mul_throughput: bad arguments");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    ZKH_TRY(zkh_ws_reserve(c, 64));
    cudaEvent_t e0, e1;
    ZKH_CUDA(c, cudaEventCreate(&e0));
    ZKH_CUDA(c, cudaEventCreate(&e1));
    Fr seed;
    for (int i = 0; i < 8; i++) seed.v[i] = 0x01234567u + 0x11111111u * i;
    seed.v[7] &= 0x3fffffffu;
    const unsigned grid = (unsigned)c->sm_count * 8;
    fr_mul_probe_kernel<<<grid, 256, 0, c->stream>>>(seed, 16, (Fr*)c->ws);   // warm-up
    cudaEventRecord(e0, c->stream);
    fr_mul_probe_kernel<<<grid, 256, 0, c->stream>>>(seed, iters, (Fr*)c->ws);
    cudaEventRecord(e1, c->stream);
    cudaError_t err = cudaEventSynchronize(e1);
    float ms = 0;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (err != cudaSuccess) return zkh_fail(c, ZKH_ERR_CUDA, "fr_mul_throughput: launch failed");
    *gmul_per_s = 4.0 * iters * grid * 256 / (ms * 1e6);
    return ZKH_OK;
}

extern "C" int zkh_fr_axpy(zkh_ctx* c, void* out_dev, const void* in_dev, const void* c32, uint64_t n) {
    if (!c) return ZKH_ERR_ARG;
    if (!out_dev || !in_dev || !c32 || !n) return zkh_fail(c, ZKH_ERR_ARG, "fr_axpy: bad arguments");
    if (!fr_canonical((const uint32_t*)c32)) return zkh_fail(c, ZKH_ERR_DOMAIN, "fr_axpy: scalar not below p");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    Fr cv;
    memcpy(cv.v, c32, 32);
    fr_axpy_plain_kernel<<<fr_grid(c, n, 8), FR_THREADS, 0, c->stream>>>((Fr*)out_dev, (const Fr*)in_dev, cv, (size_t)n);
    return cudaGetLastError() == cudaSuccess ? ZKH_OK : zkh_fail(c, ZKH_ERR_CUDA, "fr_axpy launch");
}

extern "C" int zkh_fr_mul(zkh_ctx* c, void* out_dev, const void* a_dev, const void* b_dev, uint64_t n) {
    if (!c) return ZKH_ERR_ARG;
    if (!out_dev || !a_dev || !b_dev) return zkh_fail(c, ZKH_ERR_ARG, "fr_mul: bad arguments");
    if (!n) return ZKH_OK;
    ZKH_CUDA(c, cudaSetDevice(c->device));
    fr_mul_plain_kernel<<<fr_grid(c, n, 8), FR_THREADS, 0, c->stream>>>((Fr*)out_dev, (const Fr*)a_dev, (const Fr*)b_dev, (size_t)n);
    return cudaGetLastError() == cudaSuccess ? ZKH_OK : zkh_fail(c, ZKH_ERR_CUDA, "fr_mul launch");
}

extern "C" int zkh_fr_round_sums(zkh_ctx* c, const void* a_dev, const void* b_dev, uint64_t h, void* out96) {
    if (!c) return ZKH_ERR_ARG;
    if (!a_dev || !b_dev || !out96 || !h) return zkh_fail(c, ZKH_ERR_ARG, "fr_round_sums: bad arguments");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    const unsigned g = fr_grid(c, h, 8);
    ZKH_TRY(zkh_ws_reserve(c, (size_t)g * 96 + 96));
    Fr* part = (Fr*)c->ws;
    Fr* res = part + (size_t)g * 3;
    fr_round_sums_kernel<<<g, FR_THREADS, 0, c->stream>>>((const Fr*)a_dev, (const Fr*)b_dev, (size_t)h, part);
    fr_sum3_fix_kernel<<<1, FR_THREADS, 0, c->stream>>>(part, g, res);
    ZKH_CUDA(c, cudaMemcpyAsync(out96, res, 96, cudaMemcpyDeviceToHost, c->stream));
    ZKH_CUDA(c, cudaStreamSynchronize(c->stream));
    return ZKH_OK;
}
