// Device and host helpers shared by the BLS12-381 Fr translation units.
#pragma once
#include "common.cuh"
#include "fr.cuh"

namespace zkh {

constexpr int FR_THREADS = 128;
constexpr int FR_MAXC = 4;
constexpr int FR_MAXNT = 5;

struct FrPtrs {
    const Fr* in[FR_MAXC];
    Fr* out[FR_MAXC];
};
struct FrLabels { ZkhTag t[FR_MAXNT]; };

// ------------------------------------------------------------------ reductions
template <int NT>
__device__ __forceinline__ void fr_block_sum(Fr (&v)[NT], Fr* sh) {  // sh: NT*32 elements
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int t = 0; t < NT; t++)
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) v[t] = fr_add(v[t], fr_shfl_down(v[t], d));
    if (lane == 0)
#pragma unroll
        for (int t = 0; t < NT; t++) sh[t * 32 + warp] = v[t];
    __syncthreads();
    if (warp == 0) {
#pragma unroll
        for (int t = 0; t < NT; t++) {
            Fr x = lane < nwarp ? sh[t * 32 + lane] : fr_zero();
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) x = fr_add(x, fr_shfl_down(x, d));
            v[t] = x;
        }
    }
    __syncthreads();
}

// full 32 challenge bytes as eight little-endian limbs; st is ratcheted (fs::Transcript::challenge_bytes)
__device__ __forceinline__ void tr_warp_challenge_limbs(uint32_t st[8], uint32_t out[8]) {
    const uint32_t lane = threadIdx.x & 31;
    uint32_t w[16], o[8];
#pragma unroll
    for (int i = 0; i < 8; i++) w[i] = st[i];
    w[8] = (lane == 1) ? 0x72746368u : 0x6368616cu;  // "rtch" : "chal"
    w[9] = 0x80000000u;
#pragma unroll
    for (int i = 10; i < 15; i++) w[i] = 0;
    w[15] = 36 * 8;
    sha256_iv(o);
    sha256_compress_compact(o, w);
#pragma unroll
    for (int i = 0; i < 8; i++) {
        st[i] = __shfl_sync(0xffffffffu, o[i], 1);
        out[i] = bswap32(__shfl_sync(0xffffffffu, o[i], 0));
    }
}

static inline bool fr_canonical(const uint32_t* x) {
    static const uint32_t P[8] = {0x00000001u, 0xffffffffu, 0xfffe5bfeu, 0x53bda402u, 0x09a1d805u, 0x3339d808u, 0x299d7d48u, 0x73eda753u};
    for (int i = 7; i >= 0; i--) {
        if (x[i] < P[i]) return true;
        if (x[i] > P[i]) return false;
    }
    return false;
}
static inline unsigned fr_grid(zkh_ctx* c, size_t items, int per_sm) {
    size_t want = (items + FR_THREADS - 1) / FR_THREADS, cap = (size_t)c->sm_count * per_sm;
    if (want < 1) want = 1;
    return (unsigned)(want < cap ? want : cap);
}

// E (2^v entries) from the point u (device copy u_dev, host copy u_host); stream-ordered (fr_kernels.cu)
int fr_eq_enqueue(zkh_ctx* c, const Fr* u_dev, const Fr* u_host, uint32_t v, Fr* E);

}  // namespace zkh
