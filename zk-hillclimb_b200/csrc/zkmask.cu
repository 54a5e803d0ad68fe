// Randomness of the hiding (zk) mode on the GPU: the two generators the reference defines (zkllm-src/p3_zkc.cuh:100-123,
// :471-534) and the augmented column [real values | mask slices] that every hiding commitment encodes (:158-185).
//
//   random-access stream  out[i] = mix(seed + golden * (i + 1)) mod p       (zprng_at; blind columns)
//   LCG chain             s <- a*s + c, out = (s ^ s>>31) mod p             (zprng / zprng_fill; masks)
//
// The chain is sequential on the host; here a thread jumps to its first state with the binary ladder
// A_2k = A_k^2, C_2k = C_k (A_k + 1) and then walks CHAIN_RUN consecutive states, so the ladder's conditional steps are paid
// once per run; the block transposes the runs through shared memory so that global stores are coalesced.
#include "common.cuh"

namespace {

constexpr int CHAIN_RUN = 8;
constexpr int CHAIN_T = 256;

struct Ladder { uint64_t A[40], C[40]; };

Ladder make_ladder() {
    Ladder L;
    L.A[0] = 6364136223846793005ULL; L.C[0] = 1442695040888963407ULL;
    for (int k = 1; k < 40; k++) { L.A[k] = L.A[k - 1] * L.A[k - 1]; L.C[k] = L.C[k - 1] * (L.A[k - 1] + 1); }
    return L;
}

__device__ __forceinline__ gl_t mix_at(uint64_t seed, uint64_t i) {
    uint64_t z = seed + 0x9E3779B97F4A7C15ULL * (i + 1);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    z ^= z >> 31;
    return z % GL_P;
}

__global__ void __launch_bounds__(256) fill_at_kernel(gl_t* out, uint64_t seed, uint64_t i0, size_t n) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = mix_at(seed, i0 + i);
}

// out[i] = element k0 + i of the chain from s0 (element 0 is the output of the first step)
__global__ void __launch_bounds__(CHAIN_T) chain_kernel(gl_t* out, uint64_t s0, uint64_t k0, size_t n, Ladder L) {
    __shared__ gl_t tile[CHAIN_T * CHAIN_RUN];
    const size_t base = (size_t)blockIdx.x * CHAIN_T * CHAIN_RUN;
    const size_t first = base + (size_t)threadIdx.x * CHAIN_RUN;
    if (first < n) {
        uint64_t s = s0, steps = k0 + first;
        for (int k = 0; steps; k++, steps >>= 1)
            if (steps & 1) s = L.A[k] * s + L.C[k];
#pragma unroll
        for (int j = 0; j < CHAIN_RUN; j++) {
            s = s * 6364136223846793005ULL + 1442695040888963407ULL;
            tile[threadIdx.x * CHAIN_RUN + j] = (s ^ (s >> 31)) % GL_P;
        }
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < CHAIN_RUN; j++) {
        const size_t e = (size_t)j * CHAIN_T + threadIdx.x;
        if (base + e < n) out[base + e] = tile[e];
    }
}

int chain_enqueue(zkh_ctx* c, gl_t* out, uint64_t s0, uint64_t k0, size_t n) {
    static const Ladder L = make_ladder();
    if (!n) return ZKH_OK;
    const size_t per = (size_t)CHAIN_T * CHAIN_RUN;
    chain_kernel<<<(unsigned)((n + per - 1) / per), CHAIN_T, 0, c->stream>>>(out, s0, k0, n, L);
    return cudaGetLastError() == cudaSuccess ? ZKH_OK : zkh_fail(c, ZKH_ERR_CUDA, "zk chain fill launch");
}
}  // namespace

extern "C" int zkh_zk_fill_at(zkh_ctx* c, uint64_t seed, uint64_t i0, uint64_t n, uint64_t* out_dev) {
    if (!c || (n && !out_dev)) return zkh_fail(c, ZKH_ERR_ARG, "zk_fill_at: null pointer");
    if (!n) return ZKH_OK;
    ZKH_CUDA(c, cudaSetDevice(c->device));
    const size_t want = (n + 255) / 256, cap = (size_t)c->sm_count * 16;
    fill_at_kernel<<<(unsigned)(want < cap ? want : cap), 256, 0, c->stream>>>(out_dev, seed, i0, (size_t)n);
    ZKH_CUDA(c, cudaGetLastError());
    return ZKH_OK;
}

extern "C" int zkh_zk_fill_chain(zkh_ctx* c, uint64_t s0, uint64_t k0, uint64_t n, uint64_t* out_dev) {
    if (!c || (n && !out_dev)) return zkh_fail(c, ZKH_ERR_ARG, "zk_fill_chain: null pointer");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    return chain_enqueue(c, out_dev, s0, k0, (size_t)n);
}

extern "C" int zkh_zk_augment(zkh_ctx* c, const uint64_t* col_dev, uint32_t v, uint32_t e, uint64_t mask_seed, uint64_t* out_dev) {
    if (!c || !col_dev || !out_dev) return zkh_fail(c, ZKH_ERR_ARG, "zk_augment: null pointer");
    if (e < 1 || v + e > 34) return zkh_fail(c, ZKH_ERR_ARG, "zk_augment: need e >= 1 and v + e <= 34");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    const size_t N = (size_t)1 << v, tot = (size_t)1 << (v + e);
    ZKH_CUDA(c, cudaMemcpyAsync(out_dev, col_dev, N * 8, cudaMemcpyDeviceToDevice, c->stream));
    if (mask_seed == 0) {      // masks off (the reference's negative control): zero mask slices
        ZKH_CUDA(c, cudaMemsetAsync(out_dev + N, 0, (tot - N) * 8, c->stream));
        return ZKH_OK;
    }
    return chain_enqueue(c, out_dev + N, mask_seed, 0, tot - N);
}
