// SHA-256 Merkle trees over Goldilocks codewords for sm_100a.
//
// Leaf = SHA-256 of the 8 little-endian bytes of one element; node = a single compression of
// the 64 bytes (left|right) from the IV (zkllm-src/p3_fri.cuh:33-39, p3_merkle.cuh:69-104,
// :161-207).  The reference launches one kernel per level pair; here each thread carries four
// leaves (or four digests) through two tree levels in registers, with 128-bit loads and
// stores, so a tree of 2^25 leaves takes 13 launches and the commitment path can skip storing
// the lower levels altogether when only the root is wanted.
#include "merkle.cuh"

namespace zkh {

// thread i: leaves 4i..4i+3 -> level-1 nodes 2i, 2i+1 -> level-2 node i
template <bool SALT>
__global__ void __launch_bounds__(256)
merkle_leaf4_kernel(const gl_t* __restrict__ cw, uint32_t* lv0, uint32_t* lv1, uint32_t* lv2, size_t quads, uint64_t sseed) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= quads) return;
    ulonglong2 a = ld2(cw + 4 * i), b = ld2(cw + 4 * i + 2);
    uint32_t h0[8], h1[8], n0[8], n1[8], top[8];
    leaf_digest<SALT>(a.x, sseed, 4 * i, h0);
    leaf_digest<SALT>(a.y, sseed, 4 * i + 1, h1);
    if (lv0) { store_digest(lv0 + (4 * i) * 8, h0); store_digest(lv0 + (4 * i + 1) * 8, h1); }
    sha256_node<true>(h0, h1, n0);
    leaf_digest<SALT>(b.x, sseed, 4 * i + 2, h0);
    leaf_digest<SALT>(b.y, sseed, 4 * i + 3, h1);
    if (lv0) { store_digest(lv0 + (4 * i + 2) * 8, h0); store_digest(lv0 + (4 * i + 3) * 8, h1); }
    sha256_node<true>(h0, h1, n1);
    if (lv1) { store_digest(lv1 + (2 * i) * 8, n0); store_digest(lv1 + (2 * i + 1) * 8, n1); }
    sha256_node<true>(n0, n1, top);
    store_digest(lv2 + i * 8, top);
}
// thread i: digests 4i..4i+3 of one level -> two parents -> one grandparent
__global__ void __launch_bounds__(256)
merkle_node4_kernel(const uint32_t* __restrict__ in, uint32_t* up1, uint32_t* up2, size_t quads) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= quads) return;
    uint32_t a[8], b[8], n0[8], n1[8], top[8];
    load_digest(in + (4 * i) * 8, a);
    load_digest(in + (4 * i + 1) * 8, b);
    sha256_node<true>(a, b, n0);
    load_digest(in + (4 * i + 2) * 8, a);
    load_digest(in + (4 * i + 3) * 8, b);
    sha256_node<true>(a, b, n1);
    if (up1) { store_digest(up1 + (2 * i) * 8, n0); store_digest(up1 + (2 * i + 1) * 8, n1); }
    sha256_node<true>(n0, n1, top);
    store_digest(up2 + i * 8, top);
}
// single level (used for the odd level at the top and for 2-leaf trees)
__global__ void merkle_node2_kernel(const uint32_t* __restrict__ in, uint32_t* up, size_t cnt) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= cnt) return;
    uint32_t a[8], b[8], n[8];
    load_digest(in + (2 * i) * 8, a);
    load_digest(in + (2 * i + 1) * 8, b);
    sha256_node<true>(a, b, n);
    store_digest(up + i * 8, n);
}
template <bool SALT>
__global__ void merkle_leaf1_kernel(const gl_t* __restrict__ cw, uint32_t* lv0, size_t M, uint64_t sseed) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= M) return;
    uint32_t h[8];
    leaf_digest<SALT>(cw[i], sseed, i, h);
    store_digest(lv0 + i * 8, h);
}
__global__ void copy32_kernel(const uint32_t* src, uint32_t* dst) {
    if (threadIdx.x < 8) dst[threadIdx.x] = src[threadIdx.x];
}

// One CTA of 2^cut threads per opened position: thread t hashes leaf t of the aligned 2^cut-leaf block around the position,
// the block is reduced level by level in shared memory, and at every level the sibling of the position's ancestor is written out.
template <bool SALT>
__global__ void merkle_low_paths_kernel(const gl_t* __restrict__ cw, uint32_t cut, const uint32_t* __restrict__ pos, uint32_t pstride,
                                        uint32_t padd, uint64_t sseed, uint8_t* out, size_t stride) {
    __shared__ uint32_t dg[1 << MERKLE_CUT][8];
    const uint32_t t = threadIdx.x, W = 1u << cut;
    const size_t p = (size_t)pos[(size_t)blockIdx.x * pstride] + padd, base = p & ~(size_t)(W - 1);
    {
        uint32_t h[8];
        leaf_digest<SALT>(cw[base + t], sseed, base + t, h);
#pragma unroll
        for (int k = 0; k < 8; k++) dg[t][k] = h[k];
    }
    __syncthreads();
    uint32_t rel = (uint32_t)(p & (W - 1));
    for (uint32_t l = 0; l < cut; l++) {
        const uint32_t half = W >> (l + 1);
        if (t < 8) reinterpret_cast<uint32_t*>(out + (size_t)blockIdx.x * stride + (size_t)l * 32)[t] = bswap32(dg[rel ^ 1][t]);
        uint32_t n[8];
        if (t < half) sha256_node<true>(dg[2 * t], dg[2 * t + 1], n);
        __syncthreads();
        if (t < half) {
#pragma unroll
            for (int k = 0; k < 8; k++) dg[t][k] = n[k];
        }
        __syncthreads();
        rel >>= 1;
    }
}

int merkle_low_paths_enqueue(zkh_ctx* c, const gl_t* cw, uint32_t cut, const uint32_t* pos_dev, uint32_t n, const uint64_t* sseed,
                             uint8_t* out_dev, size_t stride, uint32_t pstride, uint32_t padd) {
    if (!cut || !n) return ZKH_OK;
    if (cut > MERKLE_CUT) return zkh_fail(c, ZKH_ERR_ARG, "merkle: cut beyond the supported subtree size");
    if (sseed) merkle_low_paths_kernel<true><<<n, 1u << cut, 0, c->stream>>>(cw, cut, pos_dev, pstride, padd, *sseed, out_dev, stride);
    else merkle_low_paths_kernel<false><<<n, 1u << cut, 0, c->stream>>>(cw, cut, pos_dev, pstride, padd, 0, out_dev, stride);
    ZKH_CUDA(c, cudaGetLastError());
    return ZKH_OK;
}

int merkle_enqueue(zkh_ctx* c, const gl_t* cw, size_t M, uint8_t* tree, void* scratch, uint8_t* root_dev, const uint64_t* sseed,
                   uint32_t cut) {
    if (M < 2 || (M & (M - 1))) return zkh_fail(c, ZKH_ERR_ARG, "merkle: leaf count must be a power of two >= 2");
    if ((cut & 1) || (cut && (M >> cut) < 4)) return zkh_fail(c, ZKH_ERR_ARG, "merkle: cut must be even and leave at least 4 nodes");
    if ((!tree || cut) && !scratch) return zkh_fail(c, ZKH_ERR_ARG, "merkle: scratch needed for the levels that are not stored");
    cudaStream_t s = c->stream;
    const size_t Mt = M >> cut;                                 // nodes of the lowest stored level
    auto stored = [&](size_t cnt_at_level) -> uint32_t* {       // start of the level that has cnt nodes, or null when it is not kept
        // levels are stored Mt, Mt/2, ...: offset = 2 Mt - 2 cnt nodes
        return (tree && cnt_at_level <= Mt) ? (uint32_t*)(tree + (2 * Mt - 2 * cnt_at_level) * 32) : nullptr;
    };
    uint32_t* sA = (uint32_t*)scratch;
    uint32_t* sB = scratch ? (uint32_t*)((char*)scratch + merkle_scratch_a(M)) : nullptr;
    bool flip = false;                                          // next scratch target for a level that is not stored
    auto target = [&](size_t cnt_at_level) -> uint32_t* {       // where a level that the next kernel reads goes
        uint32_t* t = stored(cnt_at_level);
        if (!t) { t = flip ? sB : sA; flip = !flip; }
        return t;
    };
    const uint32_t* cur;  // current top level
    size_t cnt;
    if (M >= 4) {
        uint32_t* l2 = target(M / 4);
        const unsigned grid = (unsigned)((M / 4 + 255) / 256);
        if (sseed) merkle_leaf4_kernel<true><<<grid, 256, 0, s>>>(cw, stored(M), stored(M / 2), l2, M / 4, *sseed);
        else merkle_leaf4_kernel<false><<<grid, 256, 0, s>>>(cw, stored(M), stored(M / 2), l2, M / 4, 0);
        cur = l2;
        cnt = M / 4;
    } else {
        uint32_t* l0 = target(M);
        if (sseed) merkle_leaf1_kernel<true><<<1, 32, 0, s>>>(cw, l0, M, *sseed);
        else merkle_leaf1_kernel<false><<<1, 32, 0, s>>>(cw, l0, M, 0);
        cur = l0;
        cnt = M;
    }
    while (cnt > 1) {
        if (cnt >= 4) {
            uint32_t* up2 = target(cnt / 4);
            merkle_node4_kernel<<<(unsigned)((cnt / 4 + 255) / 256), 256, 0, s>>>(cur, stored(cnt / 2), up2, cnt / 4);
            cur = up2;
            cnt /= 4;
        } else {
            uint32_t* up = target(cnt / 2);
            merkle_node2_kernel<<<1, 32, 0, s>>>(cur, up, cnt / 2);
            cur = up;
            cnt /= 2;
        }
    }
    if (root_dev) copy32_kernel<<<1, 32, 0, s>>>(cur, (uint32_t*)root_dev);
    ZKH_CUDA(c, cudaGetLastError());
    return ZKH_OK;
}

// thread per (index, level): sibling digest of the path (zkllm-src/p3_fri.cuh:156-163)
__global__ void path_gather_kernel(const uint8_t* tree, size_t M, uint32_t logM, const uint32_t* idx, uint32_t n,
                                   uint4* out) {
    uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n * logM * 2) return;
    uint32_t half = t & 1, e = t >> 1, i = e / logM, l = e % logM;
    size_t cnt = M >> l;
    size_t sib = ((size_t)idx[i] >> l) ^ 1;
    const uint4* src = reinterpret_cast<const uint4*>(tree + (2 * M - 2 * cnt + sib) * 32);
    out[(size_t)e * 2 + half] = src[half];
}

}  // namespace zkh

using namespace zkh;

extern "C" size_t zkh_merkle_tree_bytes(uint64_t M) { return merkle_tree_bytes((size_t)M); }

extern "C" int zkh_merkle_build(zkh_ctx* c, const uint64_t* cw_dev, uint64_t M, uint8_t* tree_dev, uint8_t root[32]) {
    if (!c || !cw_dev) return zkh_fail(c, ZKH_ERR_ARG, "merkle_build: null pointer");
    if (M < 2 || (M & (M - 1)) || M > ((uint64_t)1 << 32))
        return zkh_fail(c, ZKH_ERR_ARG, "merkle_build: leaf count must be a power of two in [2, 2^32]");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    void* scratch = nullptr;
    if (!tree_dev) {
        ZKH_TRY(zkh_ws_reserve(c, merkle_scratch_bytes(M)));
        scratch = c->ws;
    }
    uint8_t* root_dev = (uint8_t*)c->d_ctl->aux;
    ZKH_TRY(merkle_enqueue(c, cw_dev, M, tree_dev, scratch, root ? root_dev : nullptr));
    if (root) {
        ZKH_CUDA(c, cudaMemcpyAsync(c->h_ctl->aux, root_dev, 32, cudaMemcpyDeviceToHost, c->stream));
        ZKH_CUDA(c, cudaStreamSynchronize(c->stream));
        memcpy(root, c->h_ctl->aux, 32);
    }
    return ZKH_OK;
}

extern "C" int zkh_merkle_paths(zkh_ctx* c, const uint8_t* tree_dev, uint64_t M, const uint32_t* idx, uint32_t n,
                                uint8_t* out) {
    if (!c || !tree_dev || !idx || !out) return zkh_fail(c, ZKH_ERR_ARG, "merkle_paths: null pointer");
    if (M < 2 || (M & (M - 1))) return zkh_fail(c, ZKH_ERR_ARG, "merkle_paths: bad leaf count");
    uint32_t logM = 0;
    while (((uint64_t)1 << logM) < M) logM++;
    for (uint32_t i = 0; i < n; i++)
        if (idx[i] >= M) return zkh_fail(c, ZKH_ERR_DOMAIN, "merkle_paths: index beyond the tree");
    if (n == 0) return ZKH_OK;
    ZKH_CUDA(c, cudaSetDevice(c->device));
    size_t ob = (size_t)n * logM * 32, ib = zkh_align((size_t)n * 4);
    ZKH_TRY(zkh_ws_reserve(c, ib + ob));
    uint32_t* d_idx = (uint32_t*)c->ws;
    uint4* d_out = (uint4*)((char*)c->ws + ib);
    ZKH_CUDA(c, cudaMemcpyAsync(d_idx, idx, (size_t)n * 4, cudaMemcpyHostToDevice, c->stream));
    uint32_t threads = n * logM * 2;
    path_gather_kernel<<<(threads + 255) / 256, 256, 0, c->stream>>>(tree_dev, (size_t)M, logM, d_idx, n, d_out);
    ZKH_CUDA(c, cudaGetLastError());
    ZKH_CUDA(c, cudaMemcpyAsync(out, d_out, ob, cudaMemcpyDeviceToHost, c->stream));
    ZKH_CUDA(c, cudaStreamSynchronize(c->stream));
    return ZKH_OK;
}
