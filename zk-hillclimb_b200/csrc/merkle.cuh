// Internal interface of the SHA-256 Merkle tree builder.
#pragma once
#include "common.cuh"
namespace zkh {
// A full tree is stored level after level: M leaf digests, M/2, ..., 1 (root); 32 bytes each,
// in the byte form the reference uses.  (2M-1)*32 bytes.
inline size_t merkle_tree_bytes(size_t M) { return (2 * M - 1) * 32; }
inline size_t merkle_scratch_a(size_t M) { return zkh_align((M / 4 + 2) * 32); }
inline size_t merkle_scratch_bytes(size_t M) { return merkle_scratch_a(M) + zkh_align((M / 16 + 2) * 32); }
// Queue the tree build.  tree != nullptr: every level is stored there and the root is the
// last 32 bytes.  tree == nullptr: only the root is produced, levels live in `scratch`
// (merkle_scratch_bytes).  root_dev (optional) receives a copy of the root digest bytes.
// sseed != nullptr: salted leaves SHA-256(value | SHA-256(seed | index)) for hiding commitments.
int merkle_enqueue(zkh_ctx* c, const gl_t* cw, size_t M, uint8_t* tree, void* scratch, uint8_t* root_dev,
                   const uint64_t* sseed = nullptr);
}  // namespace zkh
