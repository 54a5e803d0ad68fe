// Internal interface of the SHA-256 Merkle tree builder.
#pragma once
#include "common.cuh"
#include "sha256.cuh"
namespace zkh {
// A full tree is stored level after level: M leaf digests, M/2, ..., 1 (root); 32 bytes each,
// in the byte form the reference uses.  (2M-1)*32 bytes.
inline size_t merkle_tree_bytes(size_t M) { return (2 * M - 1) * 32; }
inline size_t merkle_scratch_a(size_t M) { return zkh_align((M / 4 + 2) * 32); }
inline size_t merkle_scratch_bytes(size_t M) { return merkle_scratch_a(M) + zkh_align((M / 16 + 2) * 32); }
// A CAPPED tree keeps only the levels from 2^cut leaves per node upwards (the full-tree layout of M >> cut "leaves"):
// 64 / 2^cut bytes per codeword element instead of 64.  An authentication path takes its upper siblings from the
// capped tree and its lowest `cut` siblings from a rebuild of the 2^cut-leaf subtree around the opened position
// (merkle_low_paths_enqueue), which costs a few hundred compressions per opened leaf.
constexpr uint32_t MERKLE_CUT = 6;
inline uint32_t merkle_cut(size_t M) { return M >= ((size_t)4 << MERKLE_CUT) ? MERKLE_CUT : 0; }
inline size_t merkle_capped_bytes(size_t M) { return merkle_tree_bytes(M >> merkle_cut(M)); }
// Queue the tree build.  tree != nullptr: the levels with at most M >> cut nodes are stored there (cut = 0: every
// level) and the root is the last 32 bytes; the levels below live in `scratch` (merkle_scratch_bytes; needed when
// tree == nullptr or cut > 0).  tree == nullptr: only the root is produced.  root_dev (optional) receives a copy of
// the root digest bytes.  sseed != nullptr: salted leaves SHA-256(value | SHA-256(seed | index)) for hiding commitments.
// cut must be even.
int merkle_enqueue(zkh_ctx* c, const gl_t* cw, size_t M, uint8_t* tree, void* scratch, uint8_t* root_dev,
                   const uint64_t* sseed = nullptr, uint32_t cut = 0);
// For each of the n positions pos_dev[i * pstride] + padd (device array): the sibling digests of levels 0..cut-1 of its
// path, written to out_dev + i * stride + level * 32.  One CTA of 2^cut threads per position.
int merkle_low_paths_enqueue(zkh_ctx* c, const gl_t* cw, uint32_t cut, const uint32_t* pos_dev, uint32_t n,
                             const uint64_t* sseed, uint8_t* out_dev, size_t stride, uint32_t pstride = 1, uint32_t padd = 0);

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
    if (SALT) sha256_salted_leaf<true>(v, sseed, (uint64_t)idx, h);
    else sha256_leaf<true>(v, h);
}
}  // namespace zkh
