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

__device__ __forceinline__ void store_digest(uint32_t* dst, const uint32_t h[8]) {
    uint4 a = make_uint4(bswap32(h[0]), bswap32(h[1]), bswap32(h[2]), bswap32(h[3]));
    uint4 b = make_uint4(bswap32(h[4]), bswap32(h[5]), bswap32(h[6]), bswap32(h[7]));
    reinterpret_cast<uint4*>(dst)[0] = a;
    reinterpret_cast<uint4*>(dst)[1] = b;
}
__device__ __forceinline__ void load_digest(const uint32_t* src, uint32_t h[8]) {
    uint4 a = __ldg(reinterpret_cast<const uint4*>(src)), b = __ldg(reinterpret_cast<const uint4*>(src) + 1);
    h[0] = bswap32(a.x); h[1] = bswap32(a.y); h[2] = bswap32(a.z); h[3] = bswap32(a.w);
    h[4] = bswap32(b.x); h[5] = bswap32(b.y); h[6] = bswap32(b.z); h[7] = bswap32(b.w);
}

// leaf digest: plain, or salted with (seed, leaf index) for hiding commitments (zkllm-src/p3_zkc.cuh:272-279)
template <bool SALT>
__device__ __forceinline__ void leaf_digest(gl_t v, uint64_t sseed, size_t idx, uint32_t h[8]) {
    if (SALT) sha256_salted_leaf(v, sseed, (uint64_t)idx, h);
    else sha256_leaf(v, h);
}
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
    sha256_node(h0, h1, n0);
    leaf_digest<SALT>(b.x, sseed, 4 * i + 2, h0);
    leaf_digest<SALT>(b.y, sseed, 4 * i + 3, h1);
    if (lv0) { store_digest(lv0 + (4 * i + 2) * 8, h0); store_digest(lv0 + (4 * i + 3) * 8, h1); }
    sha256_node(h0, h1, n1);
    if (lv1) { store_digest(lv1 + (2 * i) * 8, n0); store_digest(lv1 + (2 * i + 1) * 8, n1); }
    sha256_node(n0, n1, top);
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
    sha256_node(a, b, n0);
    load_digest(in + (4 * i + 2) * 8, a);
    load_digest(in + (4 * i + 3) * 8, b);
    sha256_node(a, b, n1);
    if (up1) { store_digest(up1 + (2 * i) * 8, n0); store_digest(up1 + (2 * i + 1) * 8, n1); }
    sha256_node(n0, n1, top);
    store_digest(up2 + i * 8, top);
}
// single level (used for the odd level at the top and for 2-leaf trees)
__global__ void merkle_node2_kernel(const uint32_t* __restrict__ in, uint32_t* up, size_t cnt) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= cnt) return;
    uint32_t a[8], b[8], n[8];
    load_digest(in + (2 * i) * 8, a);
    load_digest(in + (2 * i + 1) * 8, b);
    sha256_node(a, b, n);
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

int merkle_enqueue(zkh_ctx* c, const gl_t* cw, size_t M, uint8_t* tree, void* scratch, uint8_t* root_dev, const uint64_t* sseed) {
    if (M < 2 || (M & (M - 1))) return zkh_fail(c, ZKH_ERR_ARG, "merkle: leaf count must be a power of two >= 2");
    cudaStream_t s = c->stream;
    auto level_ptr = [&](size_t cnt_at_level) -> uint32_t* {  // start of the level that has cnt nodes
        // levels are stored M, M/2, ...: offset = 2M - 2*cnt nodes
        return (uint32_t*)(tree + (2 * M - 2 * cnt_at_level) * 32);
    };
    uint32_t* sA = (uint32_t*)scratch;
    uint32_t* sB = scratch ? (uint32_t*)((char*)scratch + merkle_scratch_a(M)) : nullptr;
    const uint32_t* cur;  // current top level
    size_t cnt;
    if (M >= 4) {
        uint32_t* l2 = tree ? level_ptr(M / 4) : sA;
        uint32_t* l0 = tree ? level_ptr(M) : nullptr;
        uint32_t* l1 = tree ? level_ptr(M / 2) : nullptr;
        const unsigned grid = (unsigned)((M / 4 + 255) / 256);
        if (sseed) merkle_leaf4_kernel<true><<<grid, 256, 0, s>>>(cw, l0, l1, l2, M / 4, *sseed);
        else merkle_leaf4_kernel<false><<<grid, 256, 0, s>>>(cw, l0, l1, l2, M / 4, 0);
        cur = l2;
        cnt = M / 4;
    } else {
        uint32_t* l0 = tree ? level_ptr(M) : sA;
        if (sseed) merkle_leaf1_kernel<true><<<1, 32, 0, s>>>(cw, l0, M, *sseed);
        else merkle_leaf1_kernel<false><<<1, 32, 0, s>>>(cw, l0, M, 0);
        cur = l0;
        cnt = M;
    }
    bool flip = true;  // next scratch target when no tree is kept
    while (cnt > 1) {
        if (cnt >= 4) {
            uint32_t* up2 = tree ? level_ptr(cnt / 4) : (flip ? sB : sA);
            merkle_node4_kernel<<<(unsigned)((cnt / 4 + 255) / 256), 256, 0, s>>>(
                cur, tree ? level_ptr(cnt / 2) : nullptr, up2, cnt / 4);
            cur = up2;
            cnt /= 4;
        } else {
            uint32_t* up = tree ? level_ptr(cnt / 2) : (flip ? sB : sA);
            merkle_node2_kernel<<<1, 32, 0, s>>>(cur, up, cnt / 2);
            cur = up;
            cnt /= 2;
        }
        flip = !flip;
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
