// Exact integer matrix products of the integer decoder layer's witness chain for sm_100a.
//
// p3itf::build_witness (zkllm-src/p3_int_layer.cuh:182-318) computes the seven weight matmuls of a layer and, per
// head, the score and attention-output products with host loops over int64 (p3imm::matmul_i64,
// zkllm-src/p3_int_gadgets.cuh:493-508).  Here they are one kernel: operands are columns of field-lifted signed
// integers (v or p - |v|), read through strided views so that the per-head slices of the (batch, position, head, lane)
// activations need no gather, multiplied exactly in 64-bit integers and written back lifted.
//
// Two kernels: the tensor-core one (ig_matmul_tc.cu) for full-size shapes, and this integer-pipe one for everything else
// (small or ragged shapes, operands beyond 2^20).
// Tiling: a CTA of 256 threads owns a 128 x 64 tile of C; operands are converted to int32 while they are staged in
// shared memory (k-major), every thread accumulates an 8 x 4 block in 64-bit registers with one 32 x 32 + 64 multiply-add
// per product.  The next k-slab is fetched into registers while the current one is multiplied.
// Bound: the integer pipe (one multiply-add per product; 2^13-term sums of 38-bit products stay below 2^51).
#include "common.cuh"

namespace zkh {

struct MatView { long long sb0, sb1, sr, sc; };   // element strides: outer batch, inner batch, row, column

constexpr int IGM_BM = 128, IGM_BN = 64, IGM_BK = 16, IGM_T = 256;

// field element -> signed 32-bit integer; values outside (-2^24, 2^24) raise the flag (sums of 2^15 products of such
// operands cannot leave 64 bits)
__device__ __forceinline__ int igm_sig(gl_t v, unsigned int& bad) {
    const long long s = (long long)(v >> 63 ? v + 0xFFFFFFFFull : v);   // v - p == v + 2^32 - 1 (mod 2^64)
    if (s <= -(1ll << 24) || s >= (1ll << 24)) bad = 1u;
    return (int)s;
}

__global__ void __launch_bounds__(IGM_T) ig_matmul_kernel(const gl_t* __restrict__ A, MatView va, const gl_t* __restrict__ B,
                                                         MatView vb, gl_t* __restrict__ C, MatView vc, uint32_t nb1,
                                                         uint32_t I, uint32_t J, uint32_t K, unsigned int* err) {
    __shared__ int As[IGM_BK][IGM_BM + 4];
    __shared__ int Bs[IGM_BK][IGM_BN + 4];
    const uint32_t tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const uint32_t b0 = blockIdx.z / nb1, b1 = blockIdx.z % nb1;
    const uint32_t i0 = blockIdx.y * IGM_BM, k0 = blockIdx.x * IGM_BN;
    A += (long long)b0 * va.sb0 + (long long)b1 * va.sb1;
    B += (long long)b0 * vb.sb0 + (long long)b1 * vb.sb1;
    C += (long long)b0 * vc.sb0 + (long long)b1 * vc.sb1;
    // staging maps: the fastest thread index runs along whichever of the two tile dimensions has the smaller stride
    const bool a_by_col = va.sc <= va.sr, b_by_col = vb.sc <= vb.sr;
    unsigned int bad = 0;
    int ra[8], rb[4];

    auto fetch = [&](uint32_t j0) {
#pragma unroll
        for (int q = 0; q < 8; q++) {            // A tile: 128 rows x 16 columns
            const uint32_t e = tid + q * IGM_T;
            const uint32_t r = a_by_col ? e / IGM_BK : e % IGM_BM, c = a_by_col ? e % IGM_BK : e / IGM_BM;
            const uint32_t i = i0 + r, j = j0 + c;
            ra[q] = (i < I && j < J) ? igm_sig(A[(long long)i * va.sr + (long long)j * va.sc], bad) : 0;
        }
#pragma unroll
        for (int q = 0; q < 4; q++) {            // B tile: 16 rows x 64 columns
            const uint32_t e = tid + q * IGM_T;
            const uint32_t r = b_by_col ? e / IGM_BN : e % IGM_BK, c = b_by_col ? e % IGM_BN : e / IGM_BK;
            const uint32_t j = j0 + r, k = k0 + c;
            rb[q] = (j < J && k < K) ? igm_sig(B[(long long)j * vb.sr + (long long)k * vb.sc], bad) : 0;
        }
    };
    auto stage = [&]() {
#pragma unroll
        for (int q = 0; q < 8; q++) {
            const uint32_t e = tid + q * IGM_T;
            const uint32_t r = a_by_col ? e / IGM_BK : e % IGM_BM, c = a_by_col ? e % IGM_BK : e / IGM_BM;
            As[c][r] = ra[q];
        }
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const uint32_t e = tid + q * IGM_T;
            const uint32_t r = b_by_col ? e / IGM_BN : e % IGM_BK, c = b_by_col ? e % IGM_BN : e / IGM_BK;
            Bs[r][c] = rb[q];
        }
    };

    long long acc[8][4];
#pragma unroll
    for (int r = 0; r < 8; r++)
#pragma unroll
        for (int c = 0; c < 4; c++) acc[r][c] = 0;

    fetch(0);
    for (uint32_t j0 = 0; j0 < J; j0 += IGM_BK) {
        stage();
        __syncthreads();
        if (j0 + IGM_BK < J) fetch(j0 + IGM_BK);
#pragma unroll
        for (int kk = 0; kk < IGM_BK; kk++) {
            // rows ty*4..+3 and 64 + ty*4..+3, columns tx*4..+3: 16-byte shared loads, conflict-free
            const int4 a_lo = *reinterpret_cast<const int4*>(&As[kk][ty * 4]);
            const int4 a_hi = *reinterpret_cast<const int4*>(&As[kk][64 + ty * 4]);
            const int4 bv = *reinterpret_cast<const int4*>(&Bs[kk][tx * 4]);
            const int av[8] = {a_lo.x, a_lo.y, a_lo.z, a_lo.w, a_hi.x, a_hi.y, a_hi.z, a_hi.w};
            const int bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int r = 0; r < 8; r++)
#pragma unroll
                for (int c = 0; c < 4; c++) acc[r][c] += (long long)av[r] * (long long)bw[c];
        }
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < 8; r++) {
        const uint32_t i = i0 + (r < 4 ? ty * 4 + r : 64 + ty * 4 + (r - 4));
        if (i >= I) continue;
#pragma unroll
        for (int c = 0; c < 4; c++) {
            const uint32_t k = k0 + tx * 4 + c;
            if (k >= K) continue;
            const long long s = acc[r][c];
            C[(long long)i * vc.sr + (long long)k * vc.sc] = s < 0 ? (gl_t)s - 0xFFFFFFFFull : (gl_t)s;   // s + p (mod 2^64)
        }
    }
    if (bad) atomicOr(err, 16u);
}

int ig_matmul_tc(zkh_ctx* c, const gl_t* A, const long long sa[4], const gl_t* B, const long long sb[4], gl_t* Cc, const long long sc[4],
                 uint32_t nb0, uint32_t nb1, uint32_t I, uint32_t J, uint32_t K);

}  // namespace zkh

using namespace zkh;

extern "C" int zkh_ig_matmul(zkh_ctx* c, const uint64_t* A_dev, const int64_t a_strides[4], const uint64_t* B_dev,
                             const int64_t b_strides[4], uint64_t* C_dev, const int64_t c_strides[4], uint32_t nb0,
                             uint32_t nb1, uint32_t I, uint32_t J, uint32_t K) {
    if (!c || !A_dev || !B_dev || !C_dev || !a_strides || !b_strides || !c_strides)
        return zkh_fail(c, ZKH_ERR_ARG, "ig_matmul: null pointer");
    if (!nb0 || !nb1 || !I || !J || !K) return zkh_fail(c, ZKH_ERR_ARG, "ig_matmul: empty dimension");
    if (J > (1u << 15)) return zkh_fail(c, ZKH_ERR_LIMIT, "ig_matmul: more than 2^15 terms per output");
    if ((uint64_t)nb0 * nb1 > 65535) return zkh_fail(c, ZKH_ERR_LIMIT, "ig_matmul: more than 65535 batch entries");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    // full-size shapes run on the tensor cores (three 7-bit limbs per operand, exact); ZKH_IG_MATMUL=imad / tc forces a path
    const char* force = getenv("ZKH_IG_MATMUL");
    if (!force || strcmp(force, "imad")) {
        const long long sa[4] = {a_strides[0], a_strides[1], a_strides[2], a_strides[3]}, sb[4] = {b_strides[0], b_strides[1], b_strides[2], b_strides[3]},
                        sc[4] = {c_strides[0], c_strides[1], c_strides[2], c_strides[3]};
        const int rc = ig_matmul_tc(c, A_dev, sa, B_dev, sb, C_dev, sc, nb0, nb1, I, J, K);
        if (rc != 1) return rc;
        if (force && !strcmp(force, "tc")) return zkh_fail(c, ZKH_ERR_ARG, "ig_matmul: shape or operand range outside the tensor-core path");
    }
    MatView va{a_strides[0], a_strides[1], a_strides[2], a_strides[3]};
    MatView vb{b_strides[0], b_strides[1], b_strides[2], b_strides[3]};
    MatView vc{c_strides[0], c_strides[1], c_strides[2], c_strides[3]};
    unsigned int* err = &c->d_ctl->err;
    ZKH_CUDA(c, cudaMemsetAsync(err, 0, 4, c->stream));
    dim3 grid((K + IGM_BN - 1) / IGM_BN, (I + IGM_BM - 1) / IGM_BM, nb0 * nb1);
    ig_matmul_kernel<<<grid, IGM_T, 0, c->stream>>>(A_dev, va, B_dev, vb, C_dev, vc, nb1, I, J, K, err);
    ZKH_CUDA(c, cudaGetLastError());
    ZKH_CUDA(c, cudaMemcpyAsync(&c->h_ctl->err, err, 4, cudaMemcpyDeviceToHost, c->stream));
    ZKH_CUDA(c, cudaStreamSynchronize(c->stream));
    if (c->h_ctl->err) return zkh_fail(c, ZKH_ERR_DOMAIN, "ig_matmul: an operand lies outside (-2^24, 2^24)");
    return ZKH_OK;
}
