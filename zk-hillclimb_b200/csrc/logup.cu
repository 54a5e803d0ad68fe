// logUp primitives over Goldilocks for sm_100a: multiplicity histogram, batched inversion,
// gamma-combination of columns, and the fraction-tree level combine.
//   histogram    zkllm-src/p3_logup.cuh:149-172 (p3lu_cntg/cnts_kernel), host loop :1412-1475
//   inversion    zkllm-src/p3_logup.cuh:636-660 (inv_all_add, host OpenMP Montgomery trick)
//   combine      zkllm-src/p3_logup.cuh:663-672 (combine), :93-107 (device Am build)
#include <cooperative_groups.h>
#include "common.cuh"

namespace zkh {

// Counting is order-free integer accumulation, so the bins equal the host loop's exactly.
// Tables of up to 2^15 rows are counted in shared memory (32-bit sub-histograms flushed with
// 64-bit atomics).  Tables of up to 2^18 rows are counted by thread-block clusters: the 2, 4 or 8 CTAs of a
// cluster each hold 2^15 bins in their shared memory (128 KB), the cluster scans its slice of the indices ONCE
// and every increment is a shared-memory atomic, on the CTA's own bins or on a neighbour's through distributed
// shared memory (skewed lookups such as range checks of Gaussian activations serialise in L2 otherwise).
// Where a cluster cannot be launched the same tables are cut into windows of 2^15 bins, blockIdx.y picking the
// window (the indices are then read once per window).  Larger tables go straight to 64-bit global atomics.
__global__ void __launch_bounds__(512)
hist_shared_kernel(const uint32_t* __restrict__ idx, size_t n, uint32_t M, unsigned long long* bins,
                   unsigned int* oob) {
    extern __shared__ uint32_t shc[];
    for (uint32_t t = threadIdx.x; t < M; t += blockDim.x) shc[t] = 0;
    __syncthreads();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        uint32_t r = idx[i];
        if (r >= M) atomicAdd(oob, 1u);
        else atomicAdd(&shc[r], 1u);
    }
    __syncthreads();
    for (uint32_t t = threadIdx.x; t < M; t += blockDim.x)
        if (shc[t]) atomicAdd(&bins[t], (unsigned long long)shc[t]);
}
__global__ void __launch_bounds__(512)
hist_window_kernel(const uint32_t* __restrict__ idx, size_t n, uint32_t M, unsigned long long* bins,
                   unsigned int* oob) {
    extern __shared__ uint32_t shc[];
    constexpr uint32_t W = 1u << 15;
    const uint32_t base = blockIdx.y * W;
    for (uint32_t t = threadIdx.x; t < W; t += blockDim.x) shc[t] = 0;
    __syncthreads();
    const size_t n4 = n / 4, stride = (size_t)gridDim.x * blockDim.x;
    const uint4* idx4 = reinterpret_cast<const uint4*>(idx);
    unsigned bad = 0;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        const uint4 v = __ldg(idx4 + i);
        const uint32_t r[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint32_t d = r[j] - base;
            if (d < W) atomicAdd(&shc[d], 1u);
            bad += r[j] >= M;
        }
    }
    for (size_t i = 4 * n4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const uint32_t d = idx[i] - base;
        if (d < W) atomicAdd(&shc[d], 1u);
        bad += idx[i] >= M;
    }
    if (bad && blockIdx.y == 0) atomicAdd(oob, bad);
    __syncthreads();
    for (uint32_t t = threadIdx.x; t < W && base + t < M; t += blockDim.x)
        if (shc[t]) atomicAdd(&bins[base + t], (unsigned long long)shc[t]);
}
// One cluster = ceil(M / 2^15) CTAs (a power of two, at most 8); CTA `rank` owns bins [rank * 2^15, (rank + 1) * 2^15).
// 1024 threads per CTA and four independent 16-byte loads in flight per thread cover the DRAM latency.
// REMOTE: the CTAs split the cluster's slice of the indices and increment whichever member owns the bin (half of the
// increments of a pair cross to the neighbour's shared memory).  Otherwise every member scans the whole slice and counts
// only its own bins: the slice is read once from DRAM and once more from L2, and every increment is local.
constexpr uint32_t HC_BINS = 1u << 15;
template <bool REMOTE>
__global__ void __launch_bounds__(1024)
hist_cluster_kernel(const uint32_t* __restrict__ idx, size_t n, uint32_t M, unsigned long long* bins, unsigned int* oob) {
    namespace cg = cooperative_groups;
    extern __shared__ uint32_t shc[];
    cg::cluster_group cluster = cg::this_cluster();
    const unsigned rank = cluster.block_rank(), csize = cluster.num_blocks();
    for (uint32_t t = threadIdx.x; t < HC_BINS; t += blockDim.x) shc[t] = 0;
    cluster.sync();                                     // every member's bins are zero before anyone increments them
    const size_t nclusters = gridDim.x / csize, cid = blockIdx.x / csize;
    const size_t lane = REMOTE ? (cid * csize + rank) * blockDim.x + threadIdx.x : cid * blockDim.x + threadIdx.x;
    const size_t stride = REMOTE ? nclusters * csize * blockDim.x : nclusters * blockDim.x;
    const size_t n4 = n / 4;
    const uint4* idx4 = reinterpret_cast<const uint4*>(idx);
    const uint32_t base = rank * HC_BINS;
    unsigned bad = 0;
    auto count = [&](uint32_t r) {
        if (r >= M) { bad++; return; }
        if (REMOTE) {
            uint32_t* dst = cluster.map_shared_rank(shc, r >> 15);
            atomicAdd(dst + (r & (HC_BINS - 1)), 1u);
        } else {
            const uint32_t d = r - base;
            if (d < HC_BINS) atomicAdd(&shc[d], 1u);
        }
    };
    for (size_t i = lane; i < n4; i += 4 * stride) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const size_t k = i + (size_t)u * stride;
            v[u] = k < n4 ? __ldg(idx4 + k) : make_uint4(~0u, ~0u, ~0u, ~0u);
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
            if (i + (size_t)u * stride >= n4) break;
            count(v[u].x); count(v[u].y); count(v[u].z); count(v[u].w);
        }
    }
    for (size_t i = 4 * n4 + lane; i < n; i += stride) count(idx[i]);
    if (bad && (REMOTE || rank == 0)) atomicAdd(oob, bad);
    cluster.sync();                                     // all increments, the neighbours' too, have landed
    for (uint32_t t = threadIdx.x; t < HC_BINS && base + t < M; t += blockDim.x)
        if (shc[t]) atomicAdd(&bins[base + t], (unsigned long long)shc[t]);
}
__global__ void __launch_bounds__(256)
hist_global_kernel(const uint32_t* __restrict__ idx, size_t n, uint32_t M, unsigned long long* bins,
                   unsigned int* oob) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        uint32_t r = idx[i];
        if (r >= M) atomicAdd(oob, 1u);
        else atomicAdd(&bins[r], 1ULL);
    }
}

// out[i] = 1/(A[i]+beta).  Each thread inverts INV_K strided elements with one Fermat
// inversion: prefix products, invert the total, peel off backwards (3 multiplies per element).
#define INV_K 16
__global__ void __launch_bounds__(256)
inv_add_kernel(const gl_t* __restrict__ A, gl_t* __restrict__ out, size_t n, gl_t beta, unsigned int* zero) {
    const size_t nthreads = (size_t)gridDim.x * blockDim.x, t = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    gl_t d[INV_K], pre[INV_K];
    gl_t acc = 1;
#pragma unroll
    for (int k = 0; k < INV_K; k++) {
        size_t i = t + (size_t)k * nthreads;
        gl_t v = 1;
        if (i < n) {
            v = gl_add(A[i], beta);
            if (v == 0) { atomicAdd(zero, 1u); v = 1; }
        }
        d[k] = v;
        pre[k] = acc;
        acc = gl_mul(acc, v);
    }
    gl_t inv = gl_inv(acc);
#pragma unroll
    for (int k = INV_K - 1; k >= 0; k--) {
        size_t i = t + (size_t)k * nthreads;
        if (i < n) out[i] = gl_mul(pre[k], inv);
        inv = gl_mul(inv, d[k]);
    }
}

struct CombCols { const gl_t* col[8]; gl_t gk[8]; int c; gl_t addend; };
__global__ void __launch_bounds__(256) combine_kernel(CombCols cc, gl_t* __restrict__ out, size_t n) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        Acc192 acc;
        acc.clear();
        acc.add_val(cc.addend);
        for (int k = 0; k < cc.c; k++) acc.add_prod(cc.gk[k], cc.col[k][i]);
        out[i] = acc.reduce();
    }
}

}  // namespace zkh

using namespace zkh;

extern "C" int zkh_histogram(zkh_ctx* c, const uint32_t* idx_dev, uint64_t n, uint32_t M, uint64_t* cnt_dev) {
    if (!c || !idx_dev || !cnt_dev) return zkh_fail(c, ZKH_ERR_ARG, "histogram: null pointer");
    if (M == 0) return zkh_fail(c, ZKH_ERR_ARG, "histogram: empty table");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    unsigned int* oob = (unsigned int*)&c->d_ctl->err;
    ZKH_CUDA(c, cudaMemsetAsync(cnt_dev, 0, (size_t)M * 8, c->stream));
    ZKH_CUDA(c, cudaMemsetAsync(oob, 0, 4, c->stream));
    if (n) {
        if (M <= (1u << 15)) {
            static ZkhOncePerDevice attr;
            zkh_once_on_device(attr, c->device, [] { cudaFuncSetAttribute(hist_shared_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024); });
            size_t blocks = (n + 512 * 64 - 1) / (512 * 64), cap = (size_t)c->sm_count;
            if (blocks < 1) blocks = 1;
            hist_shared_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 512, (size_t)M * 4, c->stream>>>(
                idx_dev, (size_t)n, M, (unsigned long long*)cnt_dev, oob);
        } else if (M <= (1u << 18) && ((uintptr_t)idx_dev & 15) == 0) {
            static ZkhOncePerDevice attr;
            zkh_once_on_device(attr, c->device, [] {
                cudaFuncSetAttribute(hist_window_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024);
                cudaFuncSetAttribute(hist_cluster_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024);
                cudaFuncSetAttribute(hist_cluster_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024);
            });
            const unsigned windows = (M + (1u << 15) - 1) >> 15;
            unsigned csize = 1;
            while (csize < windows) csize <<= 1;
            // clusters: one pass over the indices
            size_t ncl = (size_t)c->sm_count / csize, want = (n / 4 + (size_t)1024 * 4 * csize - 1) / ((size_t)1024 * 4 * csize);
            if (ncl < 1) ncl = 1;
            if (want < 1) want = 1;
            if (want < ncl) ncl = want;
            cudaLaunchConfig_t cfg;
            memset(&cfg, 0, sizeof cfg);
            cfg.gridDim = dim3((unsigned)(ncl * csize));
            cfg.blockDim = dim3(1024);
            cfg.dynamicSmemBytes = 128 * 1024;
            cfg.stream = c->stream;
            cudaLaunchAttribute at[1];
            at[0].id = cudaLaunchAttributeClusterDimension;
            at[0].val.clusterDim.x = csize;
            at[0].val.clusterDim.y = 1;
            at[0].val.clusterDim.z = 1;
            cfg.attrs = at;
            cfg.numAttrs = 1;
            // pairs: every member scans the pair's slice (second read from L2) and all increments are local; larger clusters
            // split the slice and increment across the cluster.  ZKH_HIST_REMOTE=0/1 overrides (measurement hook).
            bool remote = csize > 2;
            if (const char* e = getenv("ZKH_HIST_REMOTE")) remote = atoi(e) != 0;
            cudaError_t le = remote
                ? cudaLaunchKernelEx(&cfg, hist_cluster_kernel<true>, idx_dev, (size_t)n, M, (unsigned long long*)cnt_dev, oob)
                : cudaLaunchKernelEx(&cfg, hist_cluster_kernel<false>, idx_dev, (size_t)n, M, (unsigned long long*)cnt_dev, oob);
            if (le != cudaSuccess) {        // no room for such a cluster on this device: windows, one read of the indices each
                cudaGetLastError();
                size_t blocks = (n + 512 * 64 - 1) / (512 * 64), cap = (size_t)c->sm_count / windows;
                if (cap < 1) cap = 1;
                if (blocks < 1) blocks = 1;
                hist_window_kernel<<<dim3((unsigned)(blocks < cap ? blocks : cap), windows), 512, 128 * 1024, c->stream>>>(
                    idx_dev, (size_t)n, M, (unsigned long long*)cnt_dev, oob);
            }
        } else {
            size_t blocks = (n + 255) / 256, cap = (size_t)c->sm_count * 8;
            hist_global_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, c->stream>>>(
                idx_dev, (size_t)n, M, (unsigned long long*)cnt_dev, oob);
        }
        ZKH_CUDA(c, cudaGetLastError());
    }
    ZKH_CUDA(c, cudaMemcpyAsync(&c->h_ctl->err, oob, 4, cudaMemcpyDeviceToHost, c->stream));
    ZKH_CUDA(c, cudaStreamSynchronize(c->stream));
    if (c->h_ctl->err) return zkh_fail(c, ZKH_ERR_DOMAIN, "histogram: lookup index outside the table");
    return ZKH_OK;
}

extern "C" int zkh_gl_inv_all_add(zkh_ctx* c, const uint64_t* A_dev, uint64_t n, uint64_t beta, uint64_t* out_dev) {
    if (!c || (n && (!A_dev || !out_dev))) return zkh_fail(c, ZKH_ERR_ARG, "inv_all_add: null pointer");
    if (beta >= GL_P) return zkh_fail(c, ZKH_ERR_ARG, "inv_all_add: beta not canonical");
    if (!n) return ZKH_OK;
    ZKH_CUDA(c, cudaSetDevice(c->device));
    unsigned int* zero = (unsigned int*)&c->d_ctl->err;
    ZKH_CUDA(c, cudaMemsetAsync(zero, 0, 4, c->stream));
    size_t threads = (n + INV_K - 1) / INV_K, blocks = (threads + 255) / 256;
    inv_add_kernel<<<(unsigned)blocks, 256, 0, c->stream>>>(A_dev, out_dev, (size_t)n, beta, zero);
    ZKH_CUDA(c, cudaGetLastError());
    ZKH_CUDA(c, cudaMemcpyAsync(&c->h_ctl->err, zero, 4, cudaMemcpyDeviceToHost, c->stream));
    ZKH_CUDA(c, cudaStreamSynchronize(c->stream));
    if (c->h_ctl->err) return zkh_fail(c, ZKH_ERR_DOMAIN, "inv_all_add: zero denominator (resample beta)");
    return ZKH_OK;
}

extern "C" int zkh_gl_affine(zkh_ctx* c, const uint64_t* const* cols_dev, int ncols, uint64_t n, uint64_t g,
                             uint64_t addend, uint64_t* out_dev);
extern "C" int zkh_gl_combine(zkh_ctx* c, const uint64_t* const* cols_dev, int ncols, uint64_t n, uint64_t g,
                              uint64_t* out_dev) {
    return zkh_gl_affine(c, cols_dev, ncols, n, g, 0, out_dev);
}
extern "C" int zkh_gl_affine(zkh_ctx* c, const uint64_t* const* cols_dev, int ncols, uint64_t n, uint64_t g,
                             uint64_t addend, uint64_t* out_dev) {
    if (!c || (ncols > 0 && !cols_dev) || !out_dev) return zkh_fail(c, ZKH_ERR_ARG, "combine: null pointer");
    if (ncols < 0 || ncols > 8) return zkh_fail(c, ZKH_ERR_LIMIT, "combine: 0..8 columns");
    if (g >= GL_P || addend >= GL_P) return zkh_fail(c, ZKH_ERR_ARG, "combine: gamma / addend not canonical");
    if (!n) return ZKH_OK;
    ZKH_CUDA(c, cudaSetDevice(c->device));
    CombCols cc;
    memset(&cc, 0, sizeof cc);
    cc.c = ncols;
    cc.addend = addend;
    gl_t gk = 1;
    for (int k = 0; k < ncols; k++) { cc.col[k] = cols_dev[k]; cc.gk[k] = gk; gk = gl_mul(gk, g); }
    size_t blocks = (n + 255) / 256, cap = (size_t)c->sm_count * 8;
    combine_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, c->stream>>>(cc, out_dev, (size_t)n);
    ZKH_CUDA(c, cudaGetLastError());
    return ZKH_OK;
}

// ---------------------------------------------------------------- small dense helpers
// Matrix-vector products over the field, used to bind one index group of a committed matrix
// (partial multilinear evaluation): rows: out[r] = sum_c M[r*C+c]*w[c]; cols: out[c] = sum_r w[r]*M[r*C+c].
namespace zkh {
__global__ void __launch_bounds__(256)
matvec_rows_kernel(const gl_t* __restrict__ M, const gl_t* __restrict__ w, size_t C, gl_t* out) {
    __shared__ gl_t sh[32];
    const gl_t* row = M + (size_t)blockIdx.x * C;
    Acc192 acc;
    acc.clear();
    for (size_t c = threadIdx.x; c < C; c += blockDim.x) acc.add_prod(row[c], w[c]);
    gl_t s[1] = {acc.reduce()};
    block_sum<1>(s, sh);
    if (threadIdx.x == 0) out[blockIdx.x] = s[0];
}
// blockIdx.y selects a chunk of rows: out[chunk * C + c] = sum over the chunk's rows of w[r] * M[r][c].  A matrix with few
// columns (2048 columns fill 8 blocks) still covers the GPU; matvec_cols_sum_kernel adds the chunks.
__global__ void __launch_bounds__(256)
matvec_cols_kernel(const gl_t* __restrict__ M, const gl_t* __restrict__ w, size_t R, size_t C, size_t rows_per_chunk, gl_t* out) {
    size_t c = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const size_t r0 = (size_t)blockIdx.y * rows_per_chunk, r1 = r0 + rows_per_chunk < R ? r0 + rows_per_chunk : R;
    Acc192 acc;
    acc.clear();
    for (size_t r = r0; r < r1; r++) acc.add_prod(w[r], M[r * C + c]);
    out[(size_t)blockIdx.y * C + c] = acc.reduce();
}
__global__ void __launch_bounds__(256) matvec_cols_sum_kernel(const gl_t* __restrict__ part, size_t chunks, size_t C, gl_t* out) {
    size_t c = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    gl_t s = 0;
    for (size_t k = 0; k < chunks; k++) s = gl_add(s, part[k * C + c]);
    out[c] = s;
}
__global__ void __launch_bounds__(256) scale_vec_kernel(const gl_t* __restrict__ in, gl_t s, size_t n, gl_t* out) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = gl_mul(in[i], s);
}
}  // namespace zkh

extern "C" int zkh_gl_matvec(zkh_ctx* c, const uint64_t* M_dev, uint64_t rows, uint64_t cols, const uint64_t* w_dev,
                             int along_rows, uint64_t* out_dev) {
    if (!c || !M_dev || !w_dev || !out_dev) return zkh_fail(c, ZKH_ERR_ARG, "matvec: null pointer");
    if (!rows || !cols || rows > ((uint64_t)1 << 31) || cols > ((uint64_t)1 << 40))
        return zkh_fail(c, ZKH_ERR_ARG, "matvec: bad shape");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    if (along_rows)
        matvec_rows_kernel<<<(unsigned)rows, cols >= 256 ? 256 : 32, 0, c->stream>>>(M_dev, w_dev, (size_t)cols, out_dev);
    else {
        const size_t col_blocks = (cols + 255) / 256, want = (size_t)c->sm_count * 4;
        size_t chunks = col_blocks >= want ? 1 : (want + col_blocks - 1) / col_blocks;
        if (chunks > rows) chunks = rows;
        if (chunks > 65535) chunks = 65535;
        const size_t rpc = (rows + chunks - 1) / chunks;
        chunks = (rows + rpc - 1) / rpc;
        if (chunks == 1) {
            matvec_cols_kernel<<<dim3((unsigned)col_blocks, 1), 256, 0, c->stream>>>(M_dev, w_dev, (size_t)rows, (size_t)cols, rpc, out_dev);
        } else {
            ZKH_TRY(zkh_ws_reserve(c, chunks * cols * 8));
            gl_t* part = (gl_t*)c->ws;
            matvec_cols_kernel<<<dim3((unsigned)col_blocks, (unsigned)chunks), 256, 0, c->stream>>>(M_dev, w_dev, (size_t)rows, (size_t)cols, rpc, part);
            matvec_cols_sum_kernel<<<(unsigned)col_blocks, 256, 0, c->stream>>>(part, chunks, (size_t)cols, out_dev);
        }
    }
    ZKH_CUDA(c, cudaGetLastError());
    return ZKH_OK;
}
namespace zkh {
// C[i][k] = sum_j A[i][j] * B[j][k] mod p (row-major).  One thread owns four rows of one output column: a B element is
// loaded once per four products (coalesced over k), the A elements are warp-wide broadcasts; products accumulate in 192 bits
// and reduce once.  Used for the linked first mask slices of matmul accumulators (zkllm-src/p3_int_gadgets.cuh:512-527).
constexpr int MM_ROWS = 4;
__global__ void __launch_bounds__(256) matmul_kernel(const gl_t* __restrict__ A, const gl_t* __restrict__ B, size_t I, size_t J,
                                                     size_t K, gl_t* __restrict__ C) {
    const size_t k = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t i0 = (size_t)blockIdx.y * MM_ROWS;
    if (k >= K) return;
    Acc192 acc[MM_ROWS];
#pragma unroll
    for (int r = 0; r < MM_ROWS; r++) acc[r].clear();
    for (size_t j = 0; j < J; j++) {
        const gl_t b = B[j * K + k];
#pragma unroll
        for (int r = 0; r < MM_ROWS; r++)
            if (i0 + r < I) acc[r].add_prod(A[(i0 + r) * J + j], b);
    }
#pragma unroll
    for (int r = 0; r < MM_ROWS; r++)
        if (i0 + r < I) C[(i0 + r) * K + k] = acc[r].reduce();
}
__global__ void __launch_bounds__(256) mul_vec_kernel(const gl_t* __restrict__ a, const gl_t* __restrict__ b, size_t n, gl_t* out) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = gl_mul(a[i], b[i]);
}
}  // namespace zkh
extern "C" int zkh_gl_matmul(zkh_ctx* c, const uint64_t* A_dev, const uint64_t* B_dev, uint64_t I, uint64_t J, uint64_t K,
                             uint64_t* C_dev) {
    if (!c || !A_dev || !B_dev || !C_dev) return zkh_fail(c, ZKH_ERR_ARG, "matmul: null pointer");
    if (!I || !J || !K || I > ((uint64_t)1 << 24) || J > ((uint64_t)1 << 30) || K > ((uint64_t)1 << 30))
        return zkh_fail(c, ZKH_ERR_ARG, "matmul: bad shape");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    const unsigned gy = (unsigned)((I + MM_ROWS - 1) / MM_ROWS);
    if (gy > 65535) return zkh_fail(c, ZKH_ERR_LIMIT, "matmul: more than 262140 rows");
    matmul_kernel<<<dim3((unsigned)((K + 255) / 256), gy), 256, 0, c->stream>>>(A_dev, B_dev, (size_t)I, (size_t)J, (size_t)K, C_dev);
    ZKH_CUDA(c, cudaGetLastError());
    return ZKH_OK;
}
extern "C" int zkh_gl_mul(zkh_ctx* c, const uint64_t* a_dev, const uint64_t* b_dev, uint64_t n, uint64_t* out_dev) {
    if (!c || !a_dev || !b_dev || !out_dev) return zkh_fail(c, ZKH_ERR_ARG, "mul: null pointer");
    if (!n) return ZKH_OK;
    ZKH_CUDA(c, cudaSetDevice(c->device));
    size_t blocks = (n + 255) / 256, cap = (size_t)c->sm_count * 16;
    mul_vec_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, c->stream>>>(a_dev, b_dev, (size_t)n, out_dev);
    ZKH_CUDA(c, cudaGetLastError());
    return ZKH_OK;
}
extern "C" int zkh_gl_scale(zkh_ctx* c, const uint64_t* in_dev, uint64_t n, uint64_t s, uint64_t* out_dev) {
    if (!c || !in_dev || !out_dev) return zkh_fail(c, ZKH_ERR_ARG, "scale: null pointer");
    if (s >= GL_P) return zkh_fail(c, ZKH_ERR_ARG, "scale: factor not canonical");
    if (!n) return ZKH_OK;
    ZKH_CUDA(c, cudaSetDevice(c->device));
    scale_vec_kernel<<<(unsigned)((n + 255) / 256), 256, 0, c->stream>>>(in_dev, s, (size_t)n, out_dev);
    ZKH_CUDA(c, cudaGetLastError());
    return ZKH_OK;
}

// ---------------------------------------------------------------- operand views as bit maps
// The operand views of the per-head matmuls (p3imm::op_off / y_off, zkllm-src/p3_int_gadgets.cuh:448-470) and the broadcast
// columns of the hiding mode address a committed grid through a map on index BITS: element index = c | OR over the set
// bits b of u of m[b].  One kernel gathers (out[u] = col[idx(u)]) or scatters (out[idx(u)] = vals[u]) through such a map.
struct BitMap { uint64_t c; uint64_t m[32]; uint32_t nb; };
template <bool SCATTER>
__global__ void bitmap_move_kernel(const gl_t* __restrict__ src, size_t n, BitMap bm, gl_t* __restrict__ dst) {
    for (size_t u = (size_t)blockIdx.x * blockDim.x + threadIdx.x; u < n; u += (size_t)gridDim.x * blockDim.x) {
        uint64_t idx = bm.c;
        for (uint32_t b = 0; b < bm.nb; b++)
            if ((u >> b) & 1) idx |= bm.m[b];
        if (SCATTER) dst[idx] = src[u];
        else dst[u] = src[idx];
    }
}
static int bitmap_move(zkh_ctx* c, bool scatter, const uint64_t* src, uint64_t n, uint64_t konst, const uint64_t* masks, uint32_t nbits,
                       uint64_t other_len, uint64_t* dst, const char* what) {
    if (!c || !src || !dst || (nbits && !masks)) return zkh_fail(c, ZKH_ERR_ARG, what);
    if (nbits > 32 || (nbits < 64 && n > ((uint64_t)1 << nbits))) return zkh_fail(c, ZKH_ERR_ARG, "bit map: n beyond 2^nbits, or more than 32 index bits");
    BitMap bm;
    bm.c = konst;
    bm.nb = nbits;
    uint64_t top = konst;
    for (uint32_t b = 0; b < 32; b++) {
        bm.m[b] = b < nbits ? masks[b] : 0;
        top |= bm.m[b];
    }
    if (top >= other_len) return zkh_fail(c, ZKH_ERR_DOMAIN, "bit map: an index reaches beyond the addressed column");
    if (!n) return ZKH_OK;
    ZKH_CUDA(c, cudaSetDevice(c->device));
    size_t blocks = (n + 255) / 256, cap = (size_t)c->sm_count * 16;
    const unsigned grid = (unsigned)(blocks < cap ? blocks : cap);
    if (scatter) bitmap_move_kernel<true><<<grid, 256, 0, c->stream>>>(src, (size_t)n, bm, dst);
    else bitmap_move_kernel<false><<<grid, 256, 0, c->stream>>>(src, (size_t)n, bm, dst);
    ZKH_CUDA(c, cudaGetLastError());
    return ZKH_OK;
}
extern "C" int zkh_gl_gather_bits(zkh_ctx* c, const uint64_t* col_dev, uint64_t col_len, uint64_t n, uint64_t konst, const uint64_t* masks,
                                  uint32_t nbits, uint64_t* out_dev) {
    return bitmap_move(c, false, col_dev, n, konst, masks, nbits, col_len, out_dev, "gather_bits: null pointer");
}
// out[u] = col[u ^ x]: the rotate-half partner column of RoPE (zkllm-src/p3_int_gadgets.cuh:1297-1298)
__global__ void gather_xor_kernel(const gl_t* __restrict__ col, size_t n, uint64_t x, gl_t* __restrict__ out) {
    for (size_t u = (size_t)blockIdx.x * blockDim.x + threadIdx.x; u < n; u += (size_t)gridDim.x * blockDim.x) out[u] = col[u ^ x];
}
extern "C" int zkh_gl_gather_xor(zkh_ctx* c, const uint64_t* col_dev, uint64_t n, uint64_t xor_mask, uint64_t* out_dev) {
    if (!c || !col_dev || !out_dev) return zkh_fail(c, ZKH_ERR_ARG, "gather_xor: null pointer");
    if (!n || (n & (n - 1)) || xor_mask >= n) return zkh_fail(c, ZKH_ERR_ARG, "gather_xor: n must be a power of two above the mask");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    size_t blocks = (n + 255) / 256, cap = (size_t)c->sm_count * 16;
    gather_xor_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, c->stream>>>(col_dev, (size_t)n, xor_mask, out_dev);
    ZKH_CUDA(c, cudaGetLastError());
    return ZKH_OK;
}
// p3ismx::mask_col (zkllm-src/p3_int_gadgets.cuh:1490-1498): 1 where key j <= query i over u = j | i << lseq | a << 2 lseq
__global__ void causal_mask_kernel(uint32_t lseq, size_t n, gl_t* __restrict__ out) {
    const uint64_t m = ((uint64_t)1 << lseq) - 1;
    for (size_t u = (size_t)blockIdx.x * blockDim.x + threadIdx.x; u < n; u += (size_t)gridDim.x * blockDim.x)
        out[u] = (u & m) <= ((u >> lseq) & m) ? 1 : 0;
}
extern "C" int zkh_ig_causal_mask(zkh_ctx* c, uint32_t la, uint32_t lseq, uint64_t* out_dev) {
    if (!c || !out_dev) return zkh_fail(c, ZKH_ERR_ARG, "causal_mask: null pointer");
    if (la + 2 * lseq > 34) return zkh_fail(c, ZKH_ERR_LIMIT, "causal_mask: more than 2^34 elements");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    const size_t n = (size_t)1 << (la + 2 * lseq);
    size_t blocks = (n + 255) / 256, cap = (size_t)c->sm_count * 16;
    causal_mask_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, c->stream>>>(lseq, n, out_dev);
    ZKH_CUDA(c, cudaGetLastError());
    return ZKH_OK;
}
extern "C" int zkh_gl_scatter_bits(zkh_ctx* c, const uint64_t* vals_dev, uint64_t n, uint64_t konst, const uint64_t* masks, uint32_t nbits,
                                   uint64_t* out_dev, uint64_t out_len) {
    return bitmap_move(c, true, vals_dev, n, konst, masks, nbits, out_len, out_dev, "scatter_bits: null pointer");
}

// ---------------------------------------------------------------- rescale witness
// y = floor((acc + 2^(sf-1)) / 2^sf) on the signed value of acc, rem = acc + 2^(sf-1) - y*2^sf split into
// 16-bit limbs, plus the lookup row indices of the limbs and of y in its signed window
// (zkllm-src/p3_int_gadgets.cuh:230-275 gen_witness).  window = 2^19 (rng 1), 2^15 (rng 2), none (rng 0).
namespace zkh {
__global__ void __launch_bounds__(256)
irs_witness_kernel(const gl_t* __restrict__ acc, size_t n, uint32_t sf, int rng, gl_t* y, gl_t* L0, gl_t* L1,
                   uint32_t* iL0, uint32_t* iL1, uint32_t* iY, unsigned int* bad) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const gl_t v = acc[i];
    const long long a = v > (GL_P >> 1) ? (long long)v - (long long)GL_P : (long long)v;
    const long long H = 1LL << (sf - 1), win = rng == 1 ? (1LL << 19) : (1LL << 15);
    const long long yv = (a + H) >> sf, rem = (a + H) - (yv << sf);
    if (rng != 0 && (yv < -win || yv >= win)) { atomicAdd(bad, 1u); }
    y[i] = yv >= 0 ? (gl_t)yv : GL_P - (gl_t)(-yv);
    const long long r0 = rem & 0xFFFF, r1 = rem >> 16;   // rem >= 0 for an honest witness
    L0[i] = (gl_t)r0;
    iL0[i] = (uint32_t)r0;
    if (L1) { L1[i] = (gl_t)r1; iL1[i] = (uint32_t)r1; }
    if (iY) iY[i] = (uint32_t)(yv + win);
}
}  // namespace zkh

extern "C" int zkh_irs_witness(zkh_ctx* c, const uint64_t* acc_dev, uint64_t n, uint32_t sf, int rng, uint64_t* y_dev,
                               uint64_t* L0_dev, uint64_t* L1_dev, uint32_t* idxL0_dev, uint32_t* idxL1_dev,
                               uint32_t* idxY_dev) {
    if (!c || !acc_dev || !y_dev || !L0_dev || !idxL0_dev) return zkh_fail(c, ZKH_ERR_ARG, "irs_witness: null pointer");
    if (sf < 1 || sf > 32 || rng < 0 || rng > 2) return zkh_fail(c, ZKH_ERR_ARG, "irs_witness: sf must be 1..32, rng 0..2");
    if ((sf > 16) != (L1_dev != nullptr) || (sf > 16) != (idxL1_dev != nullptr))
        return zkh_fail(c, ZKH_ERR_ARG, "irs_witness: the second limb is present exactly when sf > 16");
    if ((rng != 0) != (idxY_dev != nullptr)) return zkh_fail(c, ZKH_ERR_ARG, "irs_witness: idxY is present exactly when rng != 0");
    if (!n) return ZKH_OK;
    ZKH_CUDA(c, cudaSetDevice(c->device));
    unsigned int* bad = (unsigned int*)&c->d_ctl->err;
    ZKH_CUDA(c, cudaMemsetAsync(bad, 0, 4, c->stream));
    irs_witness_kernel<<<(unsigned)((n + 255) / 256), 256, 0, c->stream>>>(acc_dev, (size_t)n, sf, rng, y_dev, L0_dev, L1_dev,
                                                                         idxL0_dev, idxL1_dev, idxY_dev, bad);
    ZKH_CUDA(c, cudaGetLastError());
    ZKH_CUDA(c, cudaMemcpyAsync(&c->h_ctl->err, bad, 4, cudaMemcpyDeviceToHost, c->stream));
    ZKH_CUDA(c, cudaStreamSynchronize(c->stream));
    if (c->h_ctl->err) return zkh_fail(c, ZKH_ERR_DOMAIN, "irs_witness: y out of range (data too large)");
    return ZKH_OK;
}
