// Witness replays of the integer decoder layer's gadgets for sm_100a: the element-wise and per-row integer arithmetic that
// p3itf::build_witness runs on the host (zkllm-src/p3_int_layer.cuh:182-318 through the gadgets' gen_witness functions in
// zkllm-src/p3_int_gadgets.cuh), one kernel per gadget, columns in and out as field-lifted signed integers:
//   residual add      p3iadd::gen_witness   p3_int_gadgets.cuh:690-710
//   SwiGLU product    p3iswg::gen_witness   p3_int_gadgets.cuh:1738-1788
//   RoPE              p3irope::gen_witness  p3_int_gadgets.cuh:1228-1273
//   RMSNorm           p3irms::gen_witness   p3_int_gadgets.cuh:830-916
//   causal softmax    p3ismx::gen_witness   p3_int_gadgets.cuh:1416-1512
// Exact integer arithmetic: every column equals the host replay's.  A value outside a gadget's range raises the device
// error flag and the call returns ZKH_ERR_DOMAIN (the reference throws "out of range").
// All kernels are HBM-bound streaming passes (8 bytes per column element read or written) except the two per-row ones,
// which hold a row in registers / shared memory between its reduction and its element-wise part.
#include <climits>
#include "common.cuh"

namespace zkh {

constexpr long long IG_ABND = 1ll << 19;     // RS20 window [-2^19, 2^19)

__device__ __forceinline__ long long igw_sig(gl_t v) { return (long long)(v >> 63 ? v + 0xFFFFFFFFull : v); }
__device__ __forceinline__ gl_t igw_lift(long long s) { return s < 0 ? (gl_t)s - 0xFFFFFFFFull : (gl_t)s; }

// out = a + b in the RS20 window; idx = out + 2^19
__global__ void __launch_bounds__(256) ig_add_kernel(const gl_t* __restrict__ a, const gl_t* __restrict__ b, size_t n,
                                                      gl_t* __restrict__ out, uint32_t* __restrict__ idx, unsigned int* err) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    bool bad = false;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const long long o = igw_sig(a[i]) + igw_sig(b[i]);
        bad |= (o < -IG_ABND) | (o >= IG_ABND);
        out[i] = igw_lift(o);
        idx[i] = (uint32_t)(o + IG_ABND);
    }
    if (bad) atomicOr(err, 32u);
}
// idx = v + 2^19 for a value in the RS20 window
__global__ void __launch_bounds__(256) ig_rs20_kernel(const gl_t* __restrict__ v, size_t n, uint32_t* __restrict__ idx, unsigned int* err) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    bool bad = false;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const long long s = igw_sig(v[i]);
        bad |= (s < -IG_ABND) | (s >= IG_ABND);
        idx[i] = (uint32_t)(s + IG_ABND);
    }
    if (bad) atomicOr(err, 32u);
}
// sil = SILU[g + 2^19]; m = sil * u; mo = round(m / 2^16); rem = m + 2^15 - mo * 2^16
__global__ void __launch_bounds__(256)
ig_swiglu_kernel(const gl_t* __restrict__ g, const gl_t* __restrict__ u, const gl_t* __restrict__ silu, size_t n, gl_t* __restrict__ sil_out,
                 gl_t* __restrict__ rem_out, gl_t* __restrict__ mo_out, uint32_t* __restrict__ idxG, uint32_t* __restrict__ idxR,
                 uint32_t* __restrict__ idxM, unsigned int* err) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    bool bad = false;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const long long gv = igw_sig(g[i]), uv = igw_sig(u[i]);
        const bool in = (gv >= -IG_ABND) & (gv < IG_ABND);
        bad |= !in;
        const gl_t sl = silu[in ? gv + IG_ABND : 0];
        const long long m64 = igw_sig(sl) * uv;
        const long long mo = (m64 + (1ll << 15)) >> 16, rem = (m64 + (1ll << 15)) - (mo << 16);
        bad |= (mo < -IG_ABND) | (mo >= IG_ABND);
        sil_out[i] = sl;
        rem_out[i] = (gl_t)rem;
        mo_out[i] = igw_lift(mo);
        idxG[i] = (uint32_t)(gv + IG_ABND);
        idxR[i] = (uint32_t)rem;
        idxM[i] = (uint32_t)(mo + IG_ABND);
    }
    if (bad) atomicOr(err, 32u);
}
// RoPE over the (batch, position, head, lane) layout: u = j | t << ld, position s = t mod 2^lseq, lane jj = j mod 2^ldh;
// Y = round((q * C + q[u ^ half] * S2) / 2^14) with C = cos[s][jj mod half], S2 = -/+ sin[s][jj mod half] for the first / second half
__global__ void __launch_bounds__(256)
ig_rope_kernel(const gl_t* __restrict__ q, const int* __restrict__ ct, const int* __restrict__ st, uint32_t lseq, uint32_t ldh, uint32_t ld,
               size_t n, gl_t* __restrict__ Y, gl_t* __restrict__ rem_out, uint32_t* __restrict__ idxR, uint32_t* __restrict__ idxY,
               long long* __restrict__ C_out, long long* __restrict__ S_out, unsigned int* err) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const uint32_t fb = ldh - 1;
    bool bad = false;
    for (size_t u = (size_t)blockIdx.x * blockDim.x + threadIdx.x; u < n; u += stride) {
        const size_t j = u & (((size_t)1 << ld) - 1), t = u >> ld;
        const size_t s = t & (((size_t)1 << lseq) - 1), jj = j & (((size_t)1 << ldh) - 1);
        const size_t ti = (s << fb) + (jj & (((size_t)1 << fb) - 1));
        const long long C = ct[ti], S2 = ((jj >> fb) & 1) ? (long long)st[ti] : -(long long)st[ti];
        const long long y64 = igw_sig(q[u]) * C + igw_sig(q[u ^ ((size_t)1 << fb)]) * S2;
        const long long yv = (y64 + (1ll << 13)) >> 14, rem = (y64 + (1ll << 13)) - (yv << 14);
        bad |= (yv < -IG_ABND) | (yv >= IG_ABND);
        Y[u] = igw_lift(yv);
        rem_out[u] = (gl_t)rem;
        idxR[u] = (uint32_t)(rem & 0x3FFF);
        idxY[u] = (uint32_t)(yv + IG_ABND);
        C_out[u] = C;
        S_out[u] = S2;
    }
    if (bad) atomicOr(err, 32u);
}

// ---- per-row gadgets: one CTA per row ----
__device__ __forceinline__ long long igw_block_sum(long long v, long long* sh) {
    for (int d = 16; d > 0; d >>= 1) v += __shfl_down_sync(0xffffffffu, v, d);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    long long t = 0;
    for (int w = 0; w < nw; w++) t += sh[w];
    return t;
}
__device__ __forceinline__ long long igw_block_max(long long v, long long* sh) {
    for (int d = 16; d > 0; d >>= 1) { const long long o = __shfl_down_sync(0xffffffffu, v, d); v = o > v ? o : v; }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    long long t = sh[0];
    for (int w = 1; w < nw; w++) t = sh[w] > t ? sh[w] : t;
    return t;
}

// RMSNorm: per row M = 2^14 + sum x^2, normalised m = M >> 2e in [2^14, 2^16), R = round(ISQ[m] / 2^e); per element
// W = round(R g / 2^16), Y = round(W x / 2^16).  db: the 18 per-row columns, de: W, remW, remY.
struct IgRms {
    gl_t* db[18];
    gl_t* de[3];
    gl_t* y;
    uint32_t* irow[14];   // e, m, m - 2^14, m (ISQ row), L40 L41 L42 D40 D41 D42 L20 D20 LR0, LR1
    uint32_t* iel[4];     // remW, W + 2^19, remY, Y + 2^19
};
__global__ void __launch_bounds__(256)
ig_rms_kernel(const gl_t* __restrict__ x, const gl_t* __restrict__ g, const gl_t* __restrict__ isq, uint32_t d, IgRms O, unsigned int* err) {
    __shared__ long long sh[8];
    __shared__ long long shR;
    const size_t row = blockIdx.x;
    const gl_t* xr = x + row * d;
    long long ss = 0;
    for (uint32_t j = threadIdx.x; j < d; j += blockDim.x) { const long long v = igw_sig(xr[j]); ss += v * v; }
    const long long M = (1ll << 14) + igw_block_sum(ss, sh);
    bool bad = false;
    if (threadIdx.x == 0) {
        long long e = 0;
        while ((M >> (2 * e)) >= (1ll << 16)) e++;
        const long long m = M >> (2 * e), p4 = 1ll << (2 * e), p2 = 1ll << e, h2 = e > 0 ? 1ll << (e - 1) : 0;
        const long long r4 = M - m * p4, d4 = p4 - 1 - r4;
        const long long RP = igw_sig(isq[m]);
        const long long Rr = (RP + h2) >> e, r2 = RP + h2 - (Rr << e), d2 = p2 - 1 - r2;
        const long long v[18] = {M, m, m - (1ll << 14), p4, p2, h2, RP, r4 & 0xFFFF, (r4 >> 16) & 0xFFFF, r4 >> 32,
                                 d4 & 0xFFFF, (d4 >> 16) & 0xFFFF, d4 >> 32, Rr, r2, d2, Rr & 0xFFFF, Rr >> 16};
        for (int k = 0; k < 18; k++) O.db[k][row] = igw_lift(v[k]);
        const long long ir[14] = {e, m, m - (1ll << 14), m, v[7], v[8], v[9], v[10], v[11], v[12], r2 & 0xFFFF, d2 & 0xFFFF, v[16], v[17]};
        for (int k = 0; k < 14; k++) O.irow[k][row] = (uint32_t)ir[k];
        shR = Rr;
    }
    __syncthreads();
    const long long Rr = shR;
    for (uint32_t j = threadIdx.x; j < d; j += blockDim.x) {
        const size_t u = row * d + j;
        const long long w64 = Rr * igw_sig(g[j]);
        const long long Wv = (w64 + (1ll << 15)) >> 16, remW = (w64 + (1ll << 15)) - (Wv << 16);
        const long long y64 = Wv * igw_sig(xr[j]);
        const long long Yv = (y64 + (1ll << 15)) >> 16, remY = (y64 + (1ll << 15)) - (Yv << 16);
        bad |= (Wv < -IG_ABND) | (Wv >= IG_ABND) | (Yv < -IG_ABND) | (Yv >= IG_ABND);
        O.de[0][u] = igw_lift(Wv); O.de[1][u] = (gl_t)remW; O.de[2][u] = (gl_t)remY;
        O.y[u] = igw_lift(Yv);
        O.iel[0][u] = (uint32_t)remW; O.iel[1][u] = (uint32_t)(Wv + IG_ABND);
        O.iel[2][u] = (uint32_t)remY; O.iel[3][u] = (uint32_t)(Yv + IG_ABND);
    }
    if (bad) atomicOr(err, 32u);
}

// causal softmax: row = (head-batch a, query i), key j; mx = max_{j <= i} z, dm = mx - z (2^16 where masked),
// E = EXPT[dm], S = sum_j E, P = floor((2^17 E + S) / 2S), remainders r1, r2 in 16-bit limbs; `first` marks the first
// key attaining the maximum.
struct IgSmx {
    gl_t* xe[7];          // first, dm, E, r1 lo, r1 hi, r2 lo, r2 hi
    gl_t* xb[2];          // per row: mx, S
    gl_t* p;
    uint32_t* idm;
    uint32_t* il[4];
    uint32_t* imx;
};
__global__ void __launch_bounds__(256)
ig_softmax_kernel(const gl_t* __restrict__ z, const gl_t* __restrict__ expt, uint32_t lseq, IgSmx O, unsigned int* err) {
    __shared__ long long sh[8];
    const uint32_t seq = 1u << lseq;
    const size_t row = blockIdx.x;
    const uint32_t i = (uint32_t)(row & (seq - 1));
    const gl_t* zr = z + row * seq;
    long long mx = LLONG_MIN;
    for (uint32_t j = threadIdx.x; j <= i; j += blockDim.x) { const long long v = igw_sig(zr[j]); mx = v > mx ? v : mx; }
    mx = igw_block_max(mx, sh);
    bool bad = false;
    long long ssum = 0, firstj = seq;
    for (uint32_t j = threadIdx.x; j < seq; j += blockDim.x) {
        const long long dm = j <= i ? mx - igw_sig(zr[j]) : (1ll << 16);
        const bool in = (dm >= 0) & (dm < (1ll << 17));
        bad |= !in;
        ssum += igw_sig(expt[in ? dm : 0]);
        if (j <= i && dm == 0 && (long long)j < firstj) firstj = j;
    }
    const long long S = igw_block_sum(ssum, sh);
    const long long fj = -igw_block_max(-firstj, sh);
    if (S <= 0) bad = true;
    for (uint32_t j = threadIdx.x; j < seq; j += blockDim.x) {
        const size_t u = row * seq + j;
        const long long dm = j <= i ? mx - igw_sig(zr[j]) : (1ll << 16);
        const bool in = (dm >= 0) & (dm < (1ll << 17));
        const long long E = igw_sig(expt[in ? dm : 0]);
        const long long num = (1ll << 17) * E + S, den = S > 0 ? 2 * S : 1;
        long long P = num / den;
        if (num - P * den < 0) P--;                     // floor for a negative numerator
        const long long r1 = num - 2 * P * S, r2 = 2 * S - 1 - r1;
        O.xe[0][u] = (gl_t)(j == fj);
        O.xe[1][u] = igw_lift(dm); O.xe[2][u] = igw_lift(E);
        O.xe[3][u] = igw_lift(r1 & 0xFFFF); O.xe[4][u] = igw_lift(r1 >> 16);
        O.xe[5][u] = igw_lift(r2 & 0xFFFF); O.xe[6][u] = igw_lift(r2 >> 16);
        O.p[u] = igw_lift(P);
        O.idm[u] = (uint32_t)dm;
        O.il[0][u] = (uint32_t)(r1 & 0xFFFF); O.il[1][u] = (uint32_t)(r1 >> 16);
        O.il[2][u] = (uint32_t)(r2 & 0xFFFF); O.il[3][u] = (uint32_t)(r2 >> 16);
    }
    if (threadIdx.x == 0) {
        O.xb[0][row] = igw_lift(mx);
        O.xb[1][row] = igw_lift(S);
        O.imx[row] = (uint32_t)(mx + (1ll << 15));
    }
    if (bad) atomicOr(err, 32u);
}

static unsigned igw_grid(zkh_ctx* c, size_t n) {
    size_t b = (n + 255) / 256, cap = (size_t)c->sm_count * 8;
    return (unsigned)(b < cap ? (b ? b : 1) : cap);
}
static int igw_finish(zkh_ctx* c, const char* what) {
    unsigned int* err = &c->d_ctl->err;
    ZKH_CUDA(c, cudaGetLastError());
    ZKH_CUDA(c, cudaMemcpyAsync(&c->h_ctl->err, err, 4, cudaMemcpyDeviceToHost, c->stream));
    ZKH_CUDA(c, cudaStreamSynchronize(c->stream));
    if (c->h_ctl->err) return zkh_fail(c, ZKH_ERR_DOMAIN, std::string(what) + ": a value lies outside the gadget's range");
    return ZKH_OK;
}

}  // namespace zkh

using namespace zkh;

extern "C" int zkh_ig_add_witness(zkh_ctx* c, const uint64_t* a_dev, const uint64_t* b_dev, uint64_t n, uint64_t* out_dev,
                                  uint32_t* idx_dev) {
    if (!c || !a_dev || !b_dev || !out_dev || !idx_dev || !n) return zkh_fail(c, ZKH_ERR_ARG, "ig_add_witness: null pointer or empty column");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    ZKH_CUDA(c, cudaMemsetAsync(&c->d_ctl->err, 0, 4, c->stream));
    ig_add_kernel<<<igw_grid(c, n), 256, 0, c->stream>>>(a_dev, b_dev, (size_t)n, out_dev, idx_dev, &c->d_ctl->err);
    return igw_finish(c, "ig_add_witness");
}
// signed integers -> field elements (v, or p - |v|): how weights, activations and the RoPE gadget's public columns enter
__global__ void ig_lift_i32_kernel(const int32_t* __restrict__ in, size_t n, gl_t* __restrict__ out) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const long long v = in[i];
        out[i] = v < 0 ? (gl_t)v - 0xFFFFFFFFull : (gl_t)v;        // v + p (mod 2^64)
    }
}
__global__ void ig_lift_i64_kernel(const long long* in, size_t n, gl_t* out) {     // in == out allowed
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const long long v = in[i];
        out[i] = v < 0 ? (gl_t)v - 0xFFFFFFFFull : (gl_t)v;
    }
}
extern "C" int zkh_gl_lift_i32(zkh_ctx* c, const int32_t* in_dev, uint64_t n, uint64_t* out_dev) {
    if (!c || !in_dev || !out_dev || !n) return zkh_fail(c, ZKH_ERR_ARG, "lift_i32: null pointer or empty column");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    ig_lift_i32_kernel<<<igw_grid(c, n), 256, 0, c->stream>>>(in_dev, (size_t)n, out_dev);
    ZKH_CUDA(c, cudaGetLastError());
    return ZKH_OK;
}
extern "C" int zkh_gl_lift_i64(zkh_ctx* c, const int64_t* in_dev, uint64_t n, uint64_t* out_dev) {
    if (!c || !in_dev || !out_dev || !n) return zkh_fail(c, ZKH_ERR_ARG, "lift_i64: null pointer or empty column");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    ig_lift_i64_kernel<<<igw_grid(c, n), 256, 0, c->stream>>>((const long long*)in_dev, (size_t)n, out_dev);
    ZKH_CUDA(c, cudaGetLastError());
    return ZKH_OK;
}
extern "C" int zkh_ig_rs20_index(zkh_ctx* c, const uint64_t* v_dev, uint64_t n, uint32_t* idx_dev) {
    if (!c || !v_dev || !idx_dev || !n) return zkh_fail(c, ZKH_ERR_ARG, "ig_rs20_index: null pointer or empty column");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    ZKH_CUDA(c, cudaMemsetAsync(&c->d_ctl->err, 0, 4, c->stream));
    ig_rs20_kernel<<<igw_grid(c, n), 256, 0, c->stream>>>(v_dev, (size_t)n, idx_dev, &c->d_ctl->err);
    return igw_finish(c, "ig_rs20_index");
}
extern "C" int zkh_ig_swiglu_witness(zkh_ctx* c, const uint64_t* g_dev, const uint64_t* u_dev, const uint64_t* silu_col_dev, uint64_t n,
                                     uint64_t* sil_dev, uint64_t* rem_dev, uint64_t* mo_dev, uint32_t* idxG_dev, uint32_t* idxRem_dev,
                                     uint32_t* idxMo_dev) {
    if (!c || !g_dev || !u_dev || !silu_col_dev || !sil_dev || !rem_dev || !mo_dev || !idxG_dev || !idxRem_dev || !idxMo_dev || !n)
        return zkh_fail(c, ZKH_ERR_ARG, "ig_swiglu_witness: null pointer or empty column");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    ZKH_CUDA(c, cudaMemsetAsync(&c->d_ctl->err, 0, 4, c->stream));
    ig_swiglu_kernel<<<igw_grid(c, n), 256, 0, c->stream>>>(g_dev, u_dev, silu_col_dev, (size_t)n, sil_dev, rem_dev, mo_dev, idxG_dev,
                                                           idxRem_dev, idxMo_dev, &c->d_ctl->err);
    return igw_finish(c, "ig_swiglu_witness");
}
extern "C" int zkh_ig_rope_witness(zkh_ctx* c, const uint64_t* q_dev, const int32_t* cos_dev, const int32_t* sin_dev, uint32_t lseq,
                                   uint32_t ldh, uint32_t lT, uint32_t ld, uint64_t* y_dev, uint64_t* rem_dev, uint32_t* idxRem_dev,
                                   uint32_t* idxY_dev, int64_t* c_dev, int64_t* s2_dev) {
    if (!c || !q_dev || !cos_dev || !sin_dev || !y_dev || !rem_dev || !idxRem_dev || !idxY_dev || !c_dev || !s2_dev)
        return zkh_fail(c, ZKH_ERR_ARG, "ig_rope_witness: null pointer");
    if (ldh < 1 || ldh > ld || lseq > lT || lT + ld > 40) return zkh_fail(c, ZKH_ERR_ARG, "ig_rope_witness: need 1 <= ldh <= ld, lseq <= lT");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    ZKH_CUDA(c, cudaMemsetAsync(&c->d_ctl->err, 0, 4, c->stream));
    const size_t n = (size_t)1 << (lT + ld);
    ig_rope_kernel<<<igw_grid(c, n), 256, 0, c->stream>>>(q_dev, cos_dev, sin_dev, lseq, ldh, ld, n, y_dev, rem_dev, idxRem_dev, idxY_dev,
                                                         (long long*)c_dev, (long long*)s2_dev, &c->d_ctl->err);
    return igw_finish(c, "ig_rope_witness");
}

// db: 18 per-row columns (2^lT each), de: 3 per-element columns, y, irow: 14 per-row index arrays, iel: 4 per-element ones;
// orders as in the kernel's IgRms
extern "C" int zkh_ig_rms_witness(zkh_ctx* c, const uint64_t* x_dev, const uint64_t* g_dev, const uint64_t* isq_col_dev, uint32_t lT,
                                  uint32_t ld, uint64_t* const db_dev[18], uint64_t* const de_dev[3], uint64_t* y_dev,
                                  uint32_t* const irow_dev[14], uint32_t* const iel_dev[4]) {
    if (!c || !x_dev || !g_dev || !isq_col_dev || !db_dev || !de_dev || !y_dev || !irow_dev || !iel_dev)
        return zkh_fail(c, ZKH_ERR_ARG, "ig_rms_witness: null pointer");
    if (lT + ld > 40 || ld > 20) return zkh_fail(c, ZKH_ERR_ARG, "ig_rms_witness: dimensions out of range");
    IgRms O;
    for (int k = 0; k < 18; k++) O.db[k] = db_dev[k];
    for (int k = 0; k < 3; k++) O.de[k] = de_dev[k];
    O.y = y_dev;
    for (int k = 0; k < 14; k++) O.irow[k] = irow_dev[k];
    for (int k = 0; k < 4; k++) O.iel[k] = iel_dev[k];
    ZKH_CUDA(c, cudaSetDevice(c->device));
    ZKH_CUDA(c, cudaMemsetAsync(&c->d_ctl->err, 0, 4, c->stream));
    ig_rms_kernel<<<1u << lT, 256, 0, c->stream>>>(x_dev, g_dev, isq_col_dev, 1u << ld, O, &c->d_ctl->err);
    return igw_finish(c, "ig_rms_witness");
}
// xe: 7 per-element columns, xb: mx and S per row, p, idxDM, idxL[4] per element, idxMX per row
extern "C" int zkh_ig_softmax_witness(zkh_ctx* c, const uint64_t* z_dev, const uint64_t* expt_col_dev, uint32_t la, uint32_t lseq,
                                      uint64_t* const xe_dev[7], uint64_t* const xb_dev[2], uint64_t* p_dev, uint32_t* idxDM_dev,
                                      uint32_t* const idxL_dev[4], uint32_t* idxMX_dev) {
    if (!c || !z_dev || !expt_col_dev || !xe_dev || !xb_dev || !p_dev || !idxDM_dev || !idxL_dev || !idxMX_dev)
        return zkh_fail(c, ZKH_ERR_ARG, "ig_softmax_witness: null pointer");
    if (la + lseq > 30 || lseq > 16) return zkh_fail(c, ZKH_ERR_ARG, "ig_softmax_witness: dimensions out of range");
    IgSmx O;
    for (int k = 0; k < 7; k++) O.xe[k] = xe_dev[k];
    O.xb[0] = xb_dev[0]; O.xb[1] = xb_dev[1];
    O.p = p_dev; O.idm = idxDM_dev; O.imx = idxMX_dev;
    for (int k = 0; k < 4; k++) O.il[k] = idxL_dev[k];
    ZKH_CUDA(c, cudaSetDevice(c->device));
    ZKH_CUDA(c, cudaMemsetAsync(&c->d_ctl->err, 0, 4, c->stream));
    ig_softmax_kernel<<<1u << (la + lseq), 256, 0, c->stream>>>(z_dev, expt_col_dev, lseq, O, &c->d_ctl->err);
    return igw_finish(c, "ig_softmax_witness");
}
