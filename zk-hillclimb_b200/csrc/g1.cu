// Pedersen row commitments over BLS12-381 G1 for sm_100a: out[r] = sum_i scalars[r][i] * gen[i], the commitment of the
// reference's first proof stack (Commitment::commit -> commit_pippenger, zkllm-src/commitment.cu:41-103).
//
// The reference's bucket method fixes the Jacobian representative of every commitment: 4-bit windows of the scalar's raw limbs,
// per (row, window) sixteen buckets filled in generator order, the running-sum reduction from bucket 15 down to 1, windows
// combined by Horner from the top.  The files the orchestrator compares byte by byte hold those triples, so the same sums are
// formed in the same order here: one thread per (row, window) with its sixteen buckets in local memory (m * 64 threads), then
// one thread per row for the Horner step.  Integer-pipe bound (a Jacobian addition is sixteen 384-bit Montgomery products).
#include "common.cuh"
#include "g1.cuh"

namespace zkh {

constexpr uint32_t PIP_C = 4, PIP_NB = 1u << PIP_C, PIP_W = 64;      // 64 windows of 4 bits cover the 256-bit scalar

// the w-th 4-bit window of the scalar's raw limbs (no Montgomery conversion: the reference multiplies by val[] directly)
__device__ __forceinline__ uint32_t pip_digit(const uint32_t* s, uint32_t w) {
    const uint32_t bit = w * PIP_C;
    return (s[bit >> 5] >> (bit & 31)) & (PIP_NB - 1);
}
// thread = (row, window), as in the reference: sixteen buckets in local memory filled in generator order, then
// sum_b b * bucket[b] by the running-sum trick from bucket 15 down.  (A thread per BUCKET gives fifteen times the threads but at
// every generator only one of a window's fifteen bucket threads has work: two active lanes per warp, measured 13x slower.)
__global__ void __launch_bounds__(64, 7) pedersen_bucket_kernel(const G1* __restrict__ gen, const uint32_t* __restrict__ scalars,
                                                             G1* __restrict__ partials, uint32_t m, uint32_t n) {
    const size_t rw = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (rw >= (size_t)m * PIP_W) return;
    const uint32_t w = (uint32_t)(rw % PIP_W);
    const size_t row = rw / PIP_W;
    const uint32_t* srow = scalars + row * (size_t)n * 8;
    G1 bucket[PIP_NB];
    for (uint32_t b = 0; b < PIP_NB; b++) bucket[b] = g1_zero();
    for (uint32_t i = 0; i < n; i++) {
        const uint32_t d = pip_digit(srow + (size_t)i * 8, w);
        if (d) bucket[d] = g1_add(bucket[d], g1_load(gen + i));
    }
    G1 acc = g1_zero(), run = g1_zero();
    for (int b = (int)PIP_NB - 1; b >= 1; b--) {
        acc = g1_add(acc, bucket[b]);
        run = g1_add(run, acc);
    }
    partials[rw] = run;
}
// thread = row: Horner over the windows from the top: four doublings, then the window's partial
__global__ void __launch_bounds__(64) pedersen_combine_kernel(const G1* __restrict__ partials, G1* __restrict__ out, uint32_t m) {
    const uint32_t row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= m) return;
    G1 acc = g1_zero();
    for (int w = (int)PIP_W - 1; w >= 0; w--) {
        for (uint32_t k = 0; k < PIP_C; k++) acc = g1_double(acc);
        acc = g1_add(acc, g1_load(partials + (size_t)row * PIP_W + w));
    }
    out[row] = acc;
}

}  // namespace zkh

using namespace zkh;

extern "C" int zkh_g1_pedersen_commit(zkh_ctx* c, const void* gens_dev, const void* scalars_dev, uint32_t m, uint32_t n, void* out_dev) {
    if (!c || !gens_dev || !scalars_dev || !out_dev) return zkh_fail(c, ZKH_ERR_ARG, "g1_pedersen_commit: null pointer");
    if (!m || !n) return zkh_fail(c, ZKH_ERR_ARG, "g1_pedersen_commit: empty dimension");
    if (((uintptr_t)gens_dev | (uintptr_t)scalars_dev | (uintptr_t)out_dev) & 15)
        return zkh_fail(c, ZKH_ERR_ARG, "g1_pedersen_commit: buffers must be 16-byte aligned");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    const size_t nrw = (size_t)m * PIP_W;
    ZKH_TRY(zkh_ws_reserve(c, zkh_align(nrw * sizeof(G1))));
    G1* partials = (G1*)c->ws;
    pedersen_bucket_kernel<<<(unsigned)((nrw + 63) / 64), 64, 0, c->stream>>>((const G1*)gens_dev, (const uint32_t*)scalars_dev, partials, m, n);
    pedersen_combine_kernel<<<(m + 63) / 64, 64, 0, c->stream>>>(partials, (G1*)out_dev, m);
    ZKH_CUDA(c, cudaGetLastError());
    return ZKH_OK;
}
