// Goldilocks NTT / Reed-Solomon encode for sm_100a.
//
// The reference encodes with a bit-reversal pass plus ceil(logM/2) global-memory
// radix-4 passes (zkllm-src/p3_ntt.cuh:210-230).  Here the transform is split into
// at most four digits of up to 9 bits (Cooley-Tukey, most significant input digit
// first).  One pass = one kernel over HBM: a CTA owns a (2^W x T)-element tile (T <= 16
// neighbouring transforms, so that every global access is a 64..128-byte segment), each
// thread keeps EIGHT elements of one transform in registers and runs three butterfly
// stages on them (radix 8) between two exchanges through shared memory, so a 9-bit digit
// costs two shared-memory round trips instead of nine, and the index arithmetic is done
// once per three stages.  After the last stage the inter-digit twiddle is applied and the
// digit is written bit-reversed; the last pass writes the digit-reversed (natural-order)
// result.  A 2^25 codeword takes 3 passes over HBM instead of 14.
// The zero padding of a Reed-Solomon encode (the upper half or three quarters of the first
// digit) is known at launch: those loads, additions and subtractions are left out.
//
// out[k] = sum_j in[j] * w^(jk), w = the primitive 2^logM-th root the reference uses
// (zkllm-src/p3_goldilocks.cuh:70-73).  The transform is exact field arithmetic, so the
// codeword is bit-identical to the reference's whatever the factorisation.
#include "ntt.cuh"

namespace zkh {

struct NttPass {
    uint32_t logM, W, ls, lb, logT, last, np;
    uint32_t ws[4];
    uint32_t tw_lb;
    const gl_t* tw_lo;
    const gl_t* tw_hi;
    uint64_t nin;  // input elements at positions >= nin are zero (only the first pass reads `in`)
};

__device__ __forceinline__ gl_t tw_pow(const NttPass& p, uint64_t e) {
    const uint64_t lo = e & ((1ull << p.tw_lb) - 1), hi = e >> p.tw_lb;
    gl_t a = p.tw_lo[lo];
    return hi ? gl_mul(a, p.tw_hi[hi]) : a;
}

__global__ void pow_table_kernel(gl_t* out, gl_t base, uint32_t cnt) {
    uint32_t k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k < cnt) out[k] = gl_pow(base, k);
}

// digits of fewer than three bits (transforms of 2 or 4 points, and the test hook that forces narrow digits): radix-2
// stages in shared memory
__global__ void __launch_bounds__(256) ntt_pass_small_kernel(const gl_t* in, gl_t* out, NttPass p) {
    extern __shared__ gl_t sm[];
    const uint32_t W = p.W, nW = 1u << W, T = 1u << p.logT, TP = T + 1, tid = threadIdx.x;
    gl_t* tile = sm;
    gl_t* tws = sm + (size_t)nW * TP;
    // tile origin: spread the CTA index over the index bits that are neither digit nor batch bits
    size_t base = 0;
    {
        size_t c = blockIdx.x;
        uint32_t cb = 0;
        for (uint32_t bit = 0; bit < p.logM; bit++) {
            if (bit >= p.ls && bit < p.ls + W) continue;
            if (p.logT && bit >= p.lb && bit < p.lb + p.logT) continue;
            base |= ((c >> cb) & 1) << bit;
            cb++;
        }
    }
    for (uint32_t e = tid; e < nW / 2; e += blockDim.x) tws[e] = tw_pow(p, (uint64_t)e << (p.logM - W));
    const uint32_t nel = nW << p.logT;
    if (p.ls == 0) {  // the digit is contiguous in memory: run along it
        for (uint32_t x = tid; x < nel; x += blockDim.x) {
            uint32_t d = x & (nW - 1), t = x >> W;
            size_t pos = base | d | ((size_t)t << p.lb);
            tile[d * TP + t] = pos < p.nin ? in[pos] : 0;
        }
    } else {  // batch elements are contiguous
        for (uint32_t x = tid; x < nel; x += blockDim.x) {
            uint32_t t = x & (T - 1), d = x >> p.logT;
            size_t pos = base | ((size_t)d << p.ls) | ((size_t)t << p.lb);
            tile[d * TP + t] = pos < p.nin ? in[pos] : 0;
        }
    }
    __syncthreads();
    // decimation in frequency: natural order in, bit-reversed digit out
    for (uint32_t s = 0; s < W; s++) {
        const uint32_t half = nW >> (s + 1);
        for (uint32_t b = tid; b < nel / 2; b += blockDim.x) {
            uint32_t t = b & (T - 1), q = b >> p.logT;
            uint32_t i = q & (half - 1), d0 = ((q - i) << 1) + i, d1 = d0 + half;
            gl_t u = tile[d0 * TP + t], v = tile[d1 * TP + t];
            tile[d0 * TP + t] = gl_add(u, v);
            gl_t df = gl_sub(u, v);
            tile[d1 * TP + t] = i ? gl_mul(df, tws[i << s]) : df;
        }
        __syncthreads();
    }
    for (uint32_t x = tid; x < nel; x += blockDim.x) {
        uint32_t t = x & (T - 1), k = x >> p.logT;
        gl_t val = tile[(__brev(k) >> (32 - W)) * TP + t];
        size_t pos = base | ((size_t)t << p.lb);
        if (!p.last) {
            uint64_t jlow = pos & (((size_t)1 << p.ls) - 1);
            uint64_t e = (jlow * k) << (p.logM - (W + p.ls));
            if (e) val = gl_mul(val, tw_pow(p, e));
            out[pos | ((size_t)k << p.ls)] = val;
        } else {
            // digits of pos, most significant first, become the least significant digits of the output index
            size_t outp = 0;
            uint32_t ph = p.logM, sh = 0;
            for (uint32_t j = 0; j + 1 < p.np; j++) {
                ph -= p.ws[j];
                outp |= ((pos >> ph) & (((size_t)1 << p.ws[j]) - 1)) << sh;
                sh += p.ws[j];
            }
            out[outp | ((size_t)k << sh)] = val;
        }
    }
}


// ---- radix-8 register pass ----
// Three decimation-in-frequency stages on the eight values a thread holds.  The values sit at digit indices
// d_j = (hi << (shift + 3)) | (j << shift) | lo, j = 0..7; stage s pairs indices that differ in bit W-1-s and multiplies
// the difference by w_nW^((d0 mod half) << s), half = nW >> (s + 1): for the three stages of one step that exponent
// depends on lo and on the low bits of j only.  s0 = index of the step's first stage; a_start > 0 skips stages (the last,
// partial step of a digit whose width is not a multiple of three).  ZB > 0 (first step of a zero-padded encode): the
// values x[j], j >= 8 >> ZB, are zero, so the first ZB stages only copy and scale.
template <int ZB>
__device__ __forceinline__ void r8_step(gl_t (&x)[8], const gl_t* tws, uint32_t shift, uint32_t lo, uint32_t s0, int a_start) {
    if (a_start <= 0) {
#pragma unroll
        for (int jl = 0; jl < 4; jl++) {
            if (ZB == 2 && jl >= 2) continue;                       // x[jl] and x[jl + 4] are both zero
            const gl_t tw = tws[(((uint32_t)jl << shift) | lo) << s0];
            const gl_t u = x[jl], v = x[jl + 4];
            if (ZB >= 1) {
                x[jl + 4] = gl_mul(u, tw);
            } else {
                x[jl] = gl_add(u, v);
                x[jl + 4] = gl_mul(gl_sub(u, v), tw);
            }
        }
    }
    if (a_start <= 1) {
#pragma unroll
        for (int jh = 0; jh < 8; jh += 4) {
#pragma unroll
            for (int jl = 0; jl < 2; jl++) {
                const gl_t tw = tws[(((uint32_t)jl << shift) | lo) << (s0 + 1)];
                const gl_t u = x[jh + jl], v = x[jh + jl + 2];
                if (ZB == 2) {
                    x[jh + jl + 2] = gl_mul(u, tw);
                } else {
                    x[jh + jl] = gl_add(u, v);
                    x[jh + jl + 2] = gl_mul(gl_sub(u, v), tw);
                }
            }
        }
    }
    if (shift == 0) {        // exponent 0: no twiddle in the last stage of a digit
#pragma unroll
        for (int m = 0; m < 4; m++) {
            const gl_t u = x[2 * m], v = x[2 * m + 1];
            x[2 * m] = gl_add(u, v);
            x[2 * m + 1] = gl_sub(u, v);
        }
    } else {
        const gl_t tw = tws[lo << (s0 + 2)];
#pragma unroll
        for (int m = 0; m < 4; m++) {
            const gl_t u = x[2 * m], v = x[2 * m + 1];
            x[2 * m] = gl_add(u, v);
            x[2 * m + 1] = gl_mul(gl_sub(u, v), tw);
        }
    }
}

// One digit (3 <= W <= 9 bits) of the transform.  blockDim.x = (2^W / 8) * 2^logT threads, one CTA per tile.
template <int ZB>
__global__ void __launch_bounds__(512, 2) ntt_pass_kernel(const gl_t* in, gl_t* out, NttPass p) {
    extern __shared__ gl_t sm[];
    const uint32_t W = p.W, nW = 1u << W, T = 1u << p.logT, TP = T + 1, tid = threadIdx.x, G = nW >> 3;
    gl_t* tile = sm;
    gl_t* tws = sm + (size_t)nW * TP;
    // tile origin: spread the CTA index over the index bits that are neither digit nor batch bits
    size_t base = 0;
    {
        size_t c = blockIdx.x;
        uint32_t cb = 0;
        for (uint32_t bit = 0; bit < p.logM; bit++) {
            if (bit >= p.ls && bit < p.ls + W) continue;
            if (p.logT && bit >= p.lb && bit < p.lb + p.logT) continue;
            base |= ((c >> cb) & 1) << bit;
            cb++;
        }
    }
    for (uint32_t e = tid; e < nW / 2; e += blockDim.x) tws[e] = tw_pow(p, (uint64_t)e << (p.logM - W));
    // thread -> (group g of eight digit values, transform t).  Where the digit is contiguous in memory (ls == 0) the lanes
    // run along g for the loads; every later step, and all stores, have the lanes along t.
    bool along_g = (p.ls == 0);
    uint32_t g, t;
    if (along_g) { g = tid & (G - 1); t = tid >> (W - 3); }
    else { t = tid & (T - 1); g = tid >> p.logT; }
    gl_t x[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
        if (j >= (8 >> ZB)) { x[j] = 0; continue; }
        const size_t pos = base | ((size_t)(((uint32_t)j << (W - 3)) | g) << p.ls) | ((size_t)t << p.lb);
        x[j] = pos < p.nin ? in[pos] : 0;
    }
    __syncthreads();    // twiddle table complete
    const uint32_t nfull = W / 3, rem = W % 3, nsteps = nfull + (rem ? 1 : 0);
    uint32_t shift = W - 3;
    r8_step<ZB>(x, tws, shift, g, 0, nfull ? 0 : 3 - (int)rem);   // W >= 3: the first step is always a full one
    for (uint32_t k = 1; k < nsteps; k++) {
        {   // hand the values over: write at this step's indices ...
            const uint32_t lo = g & ((1u << shift) - 1), hi = g >> shift;
#pragma unroll
            for (int j = 0; j < 8; j++) tile[((hi << (shift + 3)) | ((uint32_t)j << shift) | lo) * TP + t] = x[j];
        }
        __syncthreads();
        if (along_g) { along_g = false; t = tid & (T - 1); g = tid >> p.logT; }
        const bool full = k < nfull;
        shift = full ? W - 3 * (k + 1) : 0;
        const uint32_t lo = g & ((1u << shift) - 1), hi = g >> shift;
#pragma unroll
        for (int j = 0; j < 8; j++) x[j] = tile[((hi << (shift + 3)) | ((uint32_t)j << shift) | lo) * TP + t];   // ... read at the next
        __syncthreads();
        r8_step<0>(x, tws, shift, lo, full ? 3 * k : W - 3, full ? 0 : 3 - (int)rem);
    }
    // the thread now holds digit indices (g << 3) | j; output digit value k = bit reversal
    const size_t pos = base | ((size_t)t << p.lb);
    if (!p.last) {
        const uint64_t jlow = pos & (((size_t)1 << p.ls) - 1);
        const uint32_t esh = p.logM - (W + p.ls);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const uint32_t k = __brev((g << 3) | (uint32_t)j) >> (32 - W);
            const uint64_t e = (jlow * k) << esh;
            gl_t val = x[j];
            if (e) val = gl_mul(val, tw_pow(p, e));
            out[pos | ((size_t)k << p.ls)] = val;
        }
    } else {
        // digits of pos, most significant first, become the least significant digits of the output index
        size_t outp = 0;
        uint32_t ph = p.logM, sh = 0;
        for (uint32_t j = 0; j + 1 < p.np; j++) {
            ph -= p.ws[j];
            outp |= ((pos >> ph) & (((size_t)1 << p.ws[j]) - 1)) << sh;
            sh += p.ws[j];
        }
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const uint32_t k = __brev((g << 3) | (uint32_t)j) >> (32 - W);
            out[outp | ((size_t)k << sh)] = x[j];
        }
    }
}

__global__ void scale_kernel(gl_t* a, gl_t c, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) a[i] = gl_mul(a[i], c);
}

static int max_digit_bits() {
    const char* e = getenv("ZKH_NTT_MAX_DIGIT");  // test hook: force many passes at small sizes
    int v = e ? atoi(e) : 9;
    if (v < 2) v = 2;
    if (v > 9) v = 9;
    return v;
}

static int ntt_tables(zkh_ctx* c, uint32_t logM, bool inverse, const gl_t** lo, const gl_t** hi, uint32_t* lb_out) {
    zkh_ctx::Tw& t = c->tw[logM];
    gl_t*& tl = inverse ? t.lo_inv : t.lo;
    gl_t*& th = inverse ? t.hi_inv : t.hi;
    uint32_t lb = logM <= 13 ? logM : (logM + 1) / 2;
    if (lb < 1) lb = 1;
    if (!tl) {
        uint32_t nlo = 1u << lb, nhi = 1u << (logM > lb ? logM - lb : 0);
        gl_t* p = nullptr;
        cudaError_t e = cudaMalloc(&p, (size_t)(nlo + nhi) * 8);
        if (e != cudaSuccess) { cudaGetLastError(); return zkh_fail(c, ZKH_ERR_NOMEM, "ntt: twiddle table allocation failed"); }
        gl_t w = gl_root_of_unity(logM);
        if (inverse) w = gl_inv(w);
        pow_table_kernel<<<(nlo + 255) / 256, 256, 0, c->stream>>>(p, w, nlo);
        pow_table_kernel<<<(nhi + 255) / 256, 256, 0, c->stream>>>(p + nlo, gl_pow(w, (uint64_t)1 << lb), nhi);
        ZKH_CUDA(c, cudaGetLastError());
        tl = p;
        th = p + nlo;
        t.lb = lb;
    }
    *lo = tl;
    *hi = th;
    *lb_out = lb;
    return ZKH_OK;
}

int ntt_inverse_tables(zkh_ctx* c, uint32_t logM, const gl_t** lo, const gl_t** hi, uint32_t* lb) {
    return ntt_tables(c, logM, true, lo, hi, lb);
}

size_t ntt_scratch_bytes(uint32_t logM) {
    return (logM + max_digit_bits() - 1) / max_digit_bits() > 1 ? zkh_align(((size_t)8) << logM) : 256;
}

// in: nin valid elements (the rest of the 2^logM input is implicitly zero); out: 2^logM elements.
// in may equal out only when the transform needs more than one pass.
int ntt_enqueue(zkh_ctx* c, const gl_t* in, uint64_t nin, gl_t* out, uint32_t logM, bool inverse, void* scratch) {
    if (logM < 1 || logM > 32) return zkh_fail(c, ZKH_ERR_ARG, "ntt: logM must be 1..32");
    const int maxw = max_digit_bits();
    NttPass p;
    memset(&p, 0, sizeof p);
    p.logM = logM;
    p.np = (logM + maxw - 1) / maxw;
    if (p.np > 4) return zkh_fail(c, ZKH_ERR_LIMIT, "ntt: more than four digits");
    for (uint32_t i = 0; i < p.np; i++) p.ws[i] = logM / p.np + (i < logM % p.np ? 1 : 0);
    ZKH_TRY(ntt_tables(c, logM, inverse, &p.tw_lo, &p.tw_hi, &p.tw_lb));
    static ZkhOncePerDevice attr_set;
    zkh_once_on_device(attr_set, c->device, [] {
        cudaFuncSetAttribute(ntt_pass_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 80 * 1024);
        cudaFuncSetAttribute(ntt_pass_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 80 * 1024);
        cudaFuncSetAttribute(ntt_pass_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 80 * 1024);
        cudaFuncSetAttribute(ntt_pass_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 80 * 1024);
    });
    gl_t* tmp = (gl_t*)scratch;
    uint32_t pos_hi = logM;
    const gl_t* src = in;
    for (uint32_t i = 0; i < p.np; i++) {
        p.W = p.ws[i];
        p.ls = pos_hi - p.W;
        p.last = (i == p.np - 1);
        if (p.np == 1) { p.logT = 0; p.lb = 0; }
        else if (p.last) { p.logT = p.ws[0] < 4 ? p.ws[0] : 4; p.lb = logM - p.ws[0]; }
        else { p.logT = p.ls < 4 ? p.ls : 4; p.lb = 0; }
        if (p.W >= 3 && p.W + p.logT > 12) p.logT = 12 - p.W;       // at most 512 threads of eight values
        p.nin = (i == 0) ? nin : ((uint64_t)1 << logM);
        gl_t* dst = p.last ? out : tmp;
        size_t smem = ((size_t)(1u << p.W) * ((1u << p.logT) + 1) + (1u << p.W) / 2 + 1) * 8;
        unsigned grid = (unsigned)(((size_t)1 << logM) >> (p.W + p.logT));
        if (p.W < 3) {
            ntt_pass_small_kernel<<<grid, 256, smem, c->stream>>>(src, dst, p);
        } else {
            const unsigned threads = (1u << (p.W - 3)) << p.logT;
            // zero padding of an encode: nin = 2^logM >> r leaves the top r bits of the first digit empty
            int zb = 0;
            if (i == 0 && nin && !(nin & (nin - 1)) && nin < ((uint64_t)1 << logM)) {
                uint32_t r = 0;
                while ((nin << r) < ((uint64_t)1 << logM)) r++;
                zb = r >= 2 ? 2 : 1;
            }
            if (zb == 2) ntt_pass_kernel<2><<<grid, threads, smem, c->stream>>>(src, dst, p);
            else if (zb == 1) ntt_pass_kernel<1><<<grid, threads, smem, c->stream>>>(src, dst, p);
            else ntt_pass_kernel<0><<<grid, threads, smem, c->stream>>>(src, dst, p);
        }
        src = dst;
        pos_hi = p.ls;
    }
    if (inverse) {
        size_t n = (size_t)1 << logM;
        scale_kernel<<<(unsigned)((n + 255) / 256), 256, 0, c->stream>>>(out, gl_inv((gl_t)n), n);
    }
    ZKH_CUDA(c, cudaGetLastError());
    return ZKH_OK;
}

}  // namespace zkh

using namespace zkh;

extern "C" int zkh_ntt(zkh_ctx* c, const uint64_t* in_dev, uint64_t* out_dev, uint32_t logn, int inverse) {
    if (!c || !in_dev || !out_dev) return zkh_fail(c, ZKH_ERR_ARG, "ntt: null pointer");
    if (in_dev == out_dev) return zkh_fail(c, ZKH_ERR_ARG, "ntt: in and out must differ");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    ZKH_TRY(zkh_ws_reserve(c, ntt_scratch_bytes(logn)));
    return ntt_enqueue(c, in_dev, (uint64_t)1 << logn, out_dev, logn, inverse != 0, c->ws);
}

extern "C" int zkh_rs_encode(zkh_ctx* c, const uint64_t* c_dev, uint32_t v, uint32_t R, uint64_t* cw_dev) {
    if (!c || !c_dev || !cw_dev) return zkh_fail(c, ZKH_ERR_ARG, "rs_encode: null pointer");
    if (v + R < 1 || v + R > 32 || R > 8) return zkh_fail(c, ZKH_ERR_ARG, "rs_encode: need 1 <= v+R <= 32, R <= 8");
    if (c_dev == cw_dev) return zkh_fail(c, ZKH_ERR_ARG, "rs_encode: in and out must differ");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    ZKH_TRY(zkh_ws_reserve(c, ntt_scratch_bytes(v + R)));
    return ntt_enqueue(c, c_dev, (uint64_t)1 << v, cw_dev, v + R, false, c->ws);
}
