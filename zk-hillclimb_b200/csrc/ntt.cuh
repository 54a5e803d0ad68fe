// Internal interface of the NTT / Reed-Solomon encoder.
#pragma once
#include "common.cuh"
namespace zkh {
size_t ntt_scratch_bytes(uint32_t logM);
int ntt_enqueue(zkh_ctx* c, const gl_t* in, uint64_t nin, gl_t* out, uint32_t logM, bool inverse, void* scratch);
}  // namespace zkh
