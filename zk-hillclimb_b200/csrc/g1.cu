// Pedersen row commitments over BLS12-381 G1 for sm_100a: out[r] = sum_i scalars[r][i] * gen[i], the commitment of the
// reference's first proof stack (Commitment::commit -> commit_pippenger, zkllm-src/commitment.cu:41-103).
//
// The reference's bucket method fixes the Jacobian representative of every commitment: 4-bit windows of the scalar's raw limbs,
// per (row, window) sixteen buckets filled in generator order, the running-sum reduction from bucket 15 down to 1, windows
// combined by Horner from the top.  The files the orchestrator compares byte by byte hold those triples, so the same sums are
// formed in the same order here.  What is free is the schedule: a bucket's sum depends only on the order of its own generators,
// so the generator indices of a (row, window) are first grouped by digit (a counting sort), then every bucket is summed by a
// thread of its own with its accumulator in registers (m * 64 * 15 threads, each about n / 16 additions), then the running sum
// per (row, window) and the Horner step per row, both with each point operation on four lanes.
// Integer-pipe bound (a Jacobian addition is sixteen 384-bit Montgomery products).
#include <algorithm>

#include "common.cuh"
#define ZKH_FP_PAIR_AS_SINGLE      // 80 registers per thread in the bucket kernel: two plain products instead of a paired one
#include "g1.cuh"

namespace zkh {

constexpr uint32_t PIP_C = 4, PIP_NB = 1u << PIP_C, PIP_W = 64;      // 64 windows of 4 bits cover the 256-bit scalar

// the w-th 4-bit window of the scalar's raw limbs (no Montgomery conversion: the reference multiplies by val[] directly)
__device__ __forceinline__ uint32_t pip_digit(const uint32_t* s, uint32_t w) {
    const uint32_t bit = w * PIP_C;
    return (s[bit >> 5] >> (bit & 31)) & (PIP_NB - 1);
}
// Step 1, thread = (row, window): counting sort of the generator indices by the window's digit.  A bucket's sum depends only
// on the order of its own generators, so each bucket can be summed on its own once its index list is known.
// idx[rw * n + ..] = the indices grouped by digit (ascending inside a group), off[rw * 17 + d] = start of digit d's group.
__global__ void __launch_bounds__(64) pedersen_sort_kernel(const uint32_t* __restrict__ scalars, uint32_t rows, uint32_t n, uint32_t* __restrict__ idx,
                                                         uint32_t* __restrict__ off) {
    const size_t rw = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (rw >= (size_t)rows * PIP_W) return;
    const uint32_t w = (uint32_t)(rw % PIP_W);
    const uint32_t* srow = scalars + (rw / PIP_W) * (size_t)n * 8;
    uint32_t cnt[PIP_NB];
#pragma unroll
    for (uint32_t d = 0; d < PIP_NB; d++) cnt[d] = 0;
    for (uint32_t i = 0; i < n; i++) {
        const uint32_t dg = pip_digit(srow + (size_t)i * 8, w);
#pragma unroll
        for (uint32_t d = 0; d < PIP_NB; d++) cnt[d] += (dg == d);
    }
    uint32_t pos[PIP_NB], run = 0;
#pragma unroll
    for (uint32_t d = 0; d < PIP_NB; d++) {
        pos[d] = run;
        off[rw * (PIP_NB + 1) + d] = run;
        run += cnt[d];
    }
    off[rw * (PIP_NB + 1) + PIP_NB] = run;
    uint32_t* out = idx + rw * (size_t)n;
    for (uint32_t i = 0; i < n; i++) {
        const uint32_t dg = pip_digit(srow + (size_t)i * 8, w);
        uint32_t p = 0;
#pragma unroll
        for (uint32_t d = 0; d < PIP_NB; d++)
            if (dg == d) { p = pos[d]; pos[d] = p + 1; }
        out[p] = i;
    }
}
// Step 2: every bucket 1..15 of every (row, window) summed in generator order with the accumulator in registers.
// (With all sixteen buckets of a window in one thread's local memory, as the reference has them, 3.7 KB per thread go through
// L1 and L2 at every addition.)  The lists differ in length (n / 16 on average, a standard deviation of a quarter of the
// square root of n), so a warp takes the buckets of per_warp (row, window) pairs as a queue: a lane that finishes a bucket
// fetches the next one, and the lanes stay busy until the queue is empty.  per_warp is chosen on the host so that all warps
// are resident at once (24 per SM).
__global__ void __launch_bounds__(64, 12) pedersen_bucket_kernel(const G1* __restrict__ gen, const uint32_t* __restrict__ idx, const uint32_t* __restrict__ off,
                                                              uint32_t rows, uint32_t n, uint32_t per_warp, G1* __restrict__ buckets) {
    __shared__ unsigned int next[2];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t nrw = (size_t)rows * PIP_W, rw0 = ((size_t)blockIdx.x * 2 + warp) * per_warp;
    if (rw0 >= nrw) return;
    const uint32_t total = (uint32_t)((nrw - rw0 < per_warp ? nrw - rw0 : per_warp) * (PIP_NB - 1));
    if (lane == 0) next[warp] = 32;                  // buckets 0..31 of the queue are handed out below
    __syncwarp();
    // One addition per lane and iteration, all lanes at the same call site (lanes that drift apart in a loop of their own would
    // execute the 16-product addition one group after the other); a lane whose list is finished stores the sum and takes the
    // next bucket of the queue before the iteration's addition.
    uint32_t b = lane, pos = 0, end = 0, d = 0;
    size_t rw = 0;
    const uint32_t* list = idx;
    bool have = false;
    G1 acc = g1_zero();
    for (;;) {
        while (!have || pos == end) {
            if (have) {
                g1_store(buckets + rw * PIP_NB + d, acc);
                have = false;
                b = atomicAdd(&next[warp], 1u);
            }
            if (b >= total) break;
            rw = rw0 + b / (PIP_NB - 1);
            d = b % (PIP_NB - 1) + 1;
            pos = off[rw * (PIP_NB + 1) + d];
            end = off[rw * (PIP_NB + 1) + d + 1];
            list = idx + rw * (size_t)n;
            acc = g1_zero();
            have = true;
        }
        if (!__any_sync(0xffffffffu, have)) break;
        if (have) {
            acc = g1_add(acc, g1_load(gen + list[pos]));
            pos++;
        }
        __syncwarp();
    }
}
// Step 3, quad = (row, window): sum_b b * bucket[b] by the running sum from bucket 15 down
__global__ void __launch_bounds__(32) pedersen_runsum_kernel(const G1* __restrict__ buckets, uint32_t rows, G1* __restrict__ partials) {
    const size_t rw = (size_t)blockIdx.x * 8 + (threadIdx.x >> 2);
    if (rw >= (size_t)rows * PIP_W) return;
    const uint32_t qm = g1q_mask();
    G1 acc = g1_zero(), run = g1_zero();
    for (int b = (int)PIP_NB - 1; b >= 1; b--) {
        acc = g1q_add(acc, g1_load(buckets + rw * PIP_NB + b), qm);
        run = g1q_add(run, acc, qm);
    }
    if ((threadIdx.x & 3) == 0) g1_store(partials + rw, run);
}
// Step 4, quad = row: Horner over the windows from the top: four doublings, then the window's partial
__global__ void __launch_bounds__(32) pedersen_combine_kernel(const G1* __restrict__ partials, G1* __restrict__ out, uint32_t rows) {
    const uint32_t row = blockIdx.x * 8 + (threadIdx.x >> 2);
    if (row >= rows) return;
    const uint32_t qm = g1q_mask();
    G1 acc = g1_zero();
    for (int w = (int)PIP_W - 1; w >= 0; w--) {
        for (uint32_t k = 0; k < PIP_C; k++) acc = g1q_double(acc, qm);
        acc = g1q_add(acc, g1_load(partials + (size_t)row * PIP_W + w), qm);
    }
    if ((threadIdx.x & 3) == 0) g1_store(out + row, acc);
}

}  // namespace zkh

using namespace zkh;

extern "C" int zkh_g1_pedersen_commit(zkh_ctx* c, const void* gens_dev, const void* scalars_dev, uint32_t m, uint32_t n, void* out_dev) {
    if (!c || !gens_dev || !scalars_dev || !out_dev) return zkh_fail(c, ZKH_ERR_ARG, "g1_pedersen_commit: null pointer");
    if (!m || !n) return zkh_fail(c, ZKH_ERR_ARG, "g1_pedersen_commit: empty dimension");
    if (((uintptr_t)gens_dev | (uintptr_t)scalars_dev | (uintptr_t)out_dev) & 15)
        return zkh_fail(c, ZKH_ERR_ARG, "g1_pedersen_commit: buffers must be 16-byte aligned");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    // rows in chunks, so that the index lists (4 n bytes per row and window) stay within about 2 GB of workspace
    const size_t per_row = (size_t)PIP_W * ((size_t)n * 4 + (PIP_NB + 1) * 4 + (PIP_NB + 1) * sizeof(G1));
    uint32_t chunk = (uint32_t)std::max<size_t>(1, std::min<size_t>(m, ((size_t)2 << 30) / per_row));
    const size_t szI = zkh_align((size_t)chunk * PIP_W * n * 4), szO = zkh_align((size_t)chunk * PIP_W * (PIP_NB + 1) * 4);
    const size_t szB = zkh_align((size_t)chunk * PIP_W * PIP_NB * sizeof(G1)), szP = zkh_align((size_t)chunk * PIP_W * sizeof(G1));
    ZKH_TRY(zkh_ws_reserve(c, szI + szO + szB + szP));
    char* w = (char*)c->ws;
    uint32_t* idx = (uint32_t*)w; w += szI;
    uint32_t* off = (uint32_t*)w; w += szO;
    G1* buckets = (G1*)w; w += szB;
    G1* partials = (G1*)w;
    for (uint32_t r0 = 0; r0 < m; r0 += chunk) {
        const uint32_t rows = std::min(chunk, m - r0);
        const size_t nrw = (size_t)rows * PIP_W;
        const uint32_t* sc = (const uint32_t*)scalars_dev + (size_t)r0 * n * 8;
        pedersen_sort_kernel<<<(unsigned)((nrw + 63) / 64), 64, 0, c->stream>>>(sc, rows, n, idx, off);
        const size_t slots = (size_t)c->sm_count * 24;               // resident warps at 12 blocks of two warps per SM
        const uint32_t per_warp = (uint32_t)std::max<size_t>(1, std::min<size_t>(32, (nrw + slots - 1) / slots));
        const size_t warps = (nrw + per_warp - 1) / per_warp;
        pedersen_bucket_kernel<<<(unsigned)((warps + 1) / 2), 64, 0, c->stream>>>((const G1*)gens_dev, idx, off, rows, n, per_warp, buckets);
        pedersen_runsum_kernel<<<(unsigned)((nrw + 7) / 8), 32, 0, c->stream>>>(buckets, rows, partials);
        pedersen_combine_kernel<<<(rows + 7) / 8, 32, 0, c->stream>>>(partials, (G1*)out_dev + r0, rows);
    }
    ZKH_CUDA(c, cudaGetLastError());
    return ZKH_OK;
}
