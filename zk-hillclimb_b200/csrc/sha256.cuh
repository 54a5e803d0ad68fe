// SHA-256 and the Fiat-Shamir transcript, usable from device and host code.
//
// Byte-exact with the reference's hashing:
//   * full SHA-256 (FIPS 180-4)                      zkllm-src/fs_transcript.hpp:24-99
//   * Merkle leaf  = SHA-256(8-byte LE value)         zkllm-src/p3_fri.cuh:33-35
//   * Merkle node  = ONE compression of l|r from the IV, no padding block
//                                                     zkllm-src/p3_merkle.cuh:69-104
//   * transcript   state' = H(state|LE32(|label|)|label|LE64(len)|data)
//                  challenge: out = H(state|"chal"), state' = H(state|"rtch")
//                                                     zkllm-src/fs_transcript.hpp:115-166
// A digest is kept as eight 32-bit words h[0..7]; its byte form is the big-endian
// serialisation of those words (what the reference stores and absorbs).
#pragma once
#include <cstdint>
#include "gl.cuh"

namespace zkh {

struct Digest { uint32_t h[8]; };

GL_HD uint32_t rotr32(uint32_t x, int n) {
#ifdef __CUDA_ARCH__
    return __funnelshift_r(x, x, n);
#else
    return (x >> n) | (x << (32 - n));
#endif
}
GL_HD uint32_t bswap32(uint32_t x) {
#ifdef __CUDA_ARCH__
    return __byte_perm(x, 0, 0x0123);
#else
    return (x >> 24) | ((x >> 8) & 0xff00u) | ((x << 8) & 0xff0000u) | (x << 24);
#endif
}

#define ZKH_SHA_K_LIST                                                                           \
    0x428a2f98u, 0x71374491u, 0xb5c0fbcfu, 0xe9b5dba5u, 0x3956c25bu, 0x59f111f1u, 0x923f82a4u,   \
    0xab1c5ed5u, 0xd807aa98u, 0x12835b01u, 0x243185beu, 0x550c7dc3u, 0x72be5d74u, 0x80deb1feu,   \
    0x9bdc06a7u, 0xc19bf174u, 0xe49b69c1u, 0xefbe4786u, 0x0fc19dc6u, 0x240ca1ccu, 0x2de92c6fu,   \
    0x4a7484aau, 0x5cb0a9dcu, 0x76f988dau, 0x983e5152u, 0xa831c66du, 0xb00327c8u, 0xbf597fc7u,   \
    0xc6e00bf3u, 0xd5a79147u, 0x06ca6351u, 0x14292967u, 0x27b70a85u, 0x2e1b2138u, 0x4d2c6dfcu,   \
    0x53380d13u, 0x650a7354u, 0x766a0abbu, 0x81c2c92eu, 0x92722c85u, 0xa2bfe8a1u, 0xa81a664bu,   \
    0xc24b8b70u, 0xc76c51a3u, 0xd192e819u, 0xd6990624u, 0xf40e3585u, 0x106aa070u, 0x19a4c116u,   \
    0x1e376c08u, 0x2748774cu, 0x34b0bcb5u, 0x391c0cb3u, 0x4ed8aa4au, 0x5b9cca4fu, 0x682e6ff3u,   \
    0x748f82eeu, 0x78a5636fu, 0x84c87814u, 0x8cc70208u, 0x90befffau, 0xa4506cebu, 0xbef9a3f7u,   \
    0xc67178f2u

#ifdef __CUDACC__
// The multiplier of the additions that sha256_compress<true> routes through the multiply-add pipe; a constant-bank
// operand the compiler cannot fold, so the instruction stays a multiply-add.
static __constant__ uint32_t zkh_sha_one = 1;
#endif
// a + b computed as a * 1 + b on the multiply-add pipe (device code), so that it does not queue behind the rotations and
// the three-input logic operations on the integer pipe
GL_HD uint32_t sha_fadd(uint32_t a, uint32_t b) {
#ifdef __CUDA_ARCH__
    uint32_t d;
    asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(zkh_sha_one), "r"(b));
    return d;
#else
    return a + b;
#endif
}

// One compression: h <- h + F(h, w).  w (16 words) is consumed as a rolling schedule.
// Fully unrolled so that round constants become immediates and w stays in registers.
// BAL (throughput-bound bulk hashing: Merkle leaves and nodes): three of the seven additions of a round go through the
// multiply-add pipe.  The integer pipe is the limit of bulk SHA-256 (96 % busy with the multiply-add pipe at 5 %); moving
// three additions measured 15.6 G compressions/s against 14.3 G, moving all seven or the rotations measured slower.
template <bool BAL = false>
GL_HD void sha256_compress(uint32_t h[8], uint32_t w[16]) {
    constexpr uint32_t K[64] = {ZKH_SHA_K_LIST};
    uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
#pragma unroll
    for (int i = 0; i < 64; i++) {
        uint32_t wi;
        if (i < 16) {
            wi = w[i];
        } else {
            uint32_t x = w[(i - 15) & 15], y = w[(i - 2) & 15];
            uint32_t s0 = rotr32(x, 7) ^ rotr32(x, 18) ^ (x >> 3);
            uint32_t s1 = rotr32(y, 17) ^ rotr32(y, 19) ^ (y >> 10);
            wi = w[i & 15] = w[i & 15] + s0 + w[(i - 7) & 15] + s1;
        }
        uint32_t t2 = (rotr32(a, 2) ^ rotr32(a, 13) ^ rotr32(a, 22)) + ((a & b) ^ (a & c) ^ (b & c));
        if (BAL) {
            uint32_t t1 = sha_fadd(hh + (rotr32(e, 6) ^ rotr32(e, 11) ^ rotr32(e, 25)) + ((e & f) ^ (~e & g)), K[i] + wi);
            hh = g; g = f; f = e; e = sha_fadd(d, t1);
            d = c; c = b; b = a; a = sha_fadd(t1, t2);
        } else {
            uint32_t t1 = hh + (rotr32(e, 6) ^ rotr32(e, 11) ^ rotr32(e, 25)) + ((e & f) ^ (~e & g)) + K[i] + wi;
            hh = g; g = f; f = e; e = d + t1;
            d = c; c = b; b = a; a = t1 + t2;
        }
    }
    h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += hh;
}
GL_HD void sha256_iv(uint32_t h[8]) {
    h[0] = 0x6a09e667u; h[1] = 0xbb67ae85u; h[2] = 0x3c6ef372u; h[3] = 0xa54ff53au;
    h[4] = 0x510e527fu; h[5] = 0x9b05688cu; h[6] = 0x1f83d9abu; h[7] = 0x5be0cd19u;
}

// Merkle leaf: SHA-256 of the 8 little-endian bytes of v (one padded block).
template <bool BAL = false>
GL_HD void sha256_leaf(gl_t v, uint32_t out[8]) {
    uint32_t w[16];
    w[0] = bswap32((uint32_t)v);
    w[1] = bswap32((uint32_t)(v >> 32));
    w[2] = 0x80000000u;
#pragma unroll
    for (int i = 3; i < 15; i++) w[i] = 0;
    w[15] = 64;  // message length in bits
    sha256_iv(out);
    sha256_compress<BAL>(out, w);
}
// Salted (hiding) Merkle leaf (zkllm-src/p3_zkc.cuh:230-270): salt = SHA-256(seed_le8 | index_le8), leaf =
// SHA-256(value_le8 | salt); both are single padded blocks, the salt's digest words feed the leaf block directly.
template <bool BAL = false>
GL_HD void sha256_salt(uint64_t sseed, uint64_t idx, uint32_t hs[8]) {
    uint32_t w[16];
    w[0] = bswap32((uint32_t)sseed); w[1] = bswap32((uint32_t)(sseed >> 32));
    w[2] = bswap32((uint32_t)idx); w[3] = bswap32((uint32_t)(idx >> 32));
    w[4] = 0x80000000u;
#pragma unroll
    for (int i = 5; i < 15; i++) w[i] = 0;
    w[15] = 128;  // 16-byte message
    sha256_iv(hs);
    sha256_compress<BAL>(hs, w);
}
template <bool BAL = false>
GL_HD void sha256_salted_leaf(gl_t v, uint64_t sseed, uint64_t idx, uint32_t out[8]) {
    uint32_t w[16], hs[8];
    sha256_salt<BAL>(sseed, idx, hs);
    w[0] = bswap32((uint32_t)v); w[1] = bswap32((uint32_t)(v >> 32));
#pragma unroll
    for (int i = 0; i < 8; i++) w[2 + i] = hs[i];
    w[10] = 0x80000000u;
#pragma unroll
    for (int i = 11; i < 15; i++) w[i] = 0;
    w[15] = 320;  // 40-byte message
    sha256_iv(out);
    sha256_compress<BAL>(out, w);
}
// Merkle node: compression of the two child digests, IV start, no length block.
template <bool BAL = false>
GL_HD void sha256_node(const uint32_t l[8], const uint32_t r[8], uint32_t out[8]) {
    uint32_t w[16];
#pragma unroll
    for (int i = 0; i < 8; i++) { w[i] = l[i]; w[8 + i] = r[i]; }
    sha256_iv(out);
    sha256_compress<BAL>(out, w);
}

// Generic SHA-256 of a short byte string held in words-addressable scratch.
// msg must have room for len rounded up to the next multiple of 64 (+64).
GL_HD void sha256_bytes(uint8_t* msg, uint32_t len, uint32_t out[8]) {
    uint32_t padded = ((len + 8) / 64 + 1) * 64;
    msg[len] = 0x80;
    for (uint32_t i = len + 1; i < padded - 8; i++) msg[i] = 0;
    uint64_t bits = (uint64_t)len * 8;
    for (int i = 0; i < 8; i++) msg[padded - 1 - i] = (uint8_t)(bits >> (8 * i));
    sha256_iv(out);
    for (uint32_t off = 0; off < padded; off += 64) {
        uint32_t w[16];
        for (int i = 0; i < 16; i++)
            w[i] = ((uint32_t)msg[off + 4 * i] << 24) | ((uint32_t)msg[off + 4 * i + 1] << 16) |
                   ((uint32_t)msg[off + 4 * i + 2] << 8) | (uint32_t)msg[off + 4 * i + 3];
        sha256_compress(out, w);
    }
}

// ---------------- transcript ----------------
#define ZKH_TR_MAX_LABEL 48
#define ZKH_TR_MAX_DATA 320

GL_HD void digest_to_bytes(const uint32_t h[8], uint8_t* b) {
    for (int i = 0; i < 8; i++) {
        b[4 * i] = (uint8_t)(h[i] >> 24); b[4 * i + 1] = (uint8_t)(h[i] >> 16);
        b[4 * i + 2] = (uint8_t)(h[i] >> 8); b[4 * i + 3] = (uint8_t)h[i];
    }
}
GL_HD void digest_from_bytes(const uint8_t* b, uint32_t h[8]) {
    for (int i = 0; i < 8; i++)
        h[i] = ((uint32_t)b[4 * i] << 24) | ((uint32_t)b[4 * i + 1] << 16) |
               ((uint32_t)b[4 * i + 2] << 8) | (uint32_t)b[4 * i + 3];
}

// state' = H(state | LE32(ll) | label | LE64(len) | data);  ll <= 48, len <= 320
GL_HD void tr_absorb(uint32_t st[8], const char* label, uint32_t ll, const void* data, uint32_t len) {
    uint8_t msg[32 + 4 + ZKH_TR_MAX_LABEL + 8 + ZKH_TR_MAX_DATA + 72];
    digest_to_bytes(st, msg);
    uint32_t p = 32;
    msg[p++] = (uint8_t)ll; msg[p++] = (uint8_t)(ll >> 8); msg[p++] = 0; msg[p++] = 0;
    for (uint32_t i = 0; i < ll; i++) msg[p++] = (uint8_t)label[i];
    msg[p++] = (uint8_t)len; msg[p++] = (uint8_t)(len >> 8);
    for (int i = 0; i < 6; i++) msg[p++] = 0;
    const uint8_t* d = (const uint8_t*)data;
    for (uint32_t i = 0; i < len; i++) msg[p++] = d[i];
    sha256_bytes(msg, p, st);
}
// out = H(state|"chal"); state' = H(state|"rtch").  36-byte messages: one block each.
GL_HD void tr_challenge(uint32_t st[8], uint32_t out[8]) {
    uint32_t w[16], w2[16];
#pragma unroll
    for (int i = 0; i < 8; i++) { w[i] = st[i]; w2[i] = st[i]; }
    w[8] = 0x6368616cu;   // "chal"
    w2[8] = 0x72746368u;  // "rtch"
    w[9] = w2[9] = 0x80000000u;
#pragma unroll
    for (int i = 10; i < 15; i++) { w[i] = 0; w2[i] = 0; }
    w[15] = w2[15] = 36 * 8;
    sha256_iv(out);
    sha256_compress(out, w);
    uint32_t ns[8];
    sha256_iv(ns);
    sha256_compress(ns, w2);
#pragma unroll
    for (int i = 0; i < 8; i++) st[i] = ns[i];
}
#ifdef __CUDACC__
// ---- warp-level transcript steps for the serial end of a round ----
// The fully unrolled compression above is ~30 KB of straight-line code per instance; run once
// by one thread at the end of a kernel it is an instruction-cache miss from start to end.  The
// transcript path therefore uses ONE shared, compact copy (16 rounds unrolled, looped 4 times,
// round constants from constant memory), and runs the two independent hashes of a challenge
// ("chal" and "rtch") on two lanes of the same warp.
static __constant__ uint32_t zkh_sha_k[64] = {ZKH_SHA_K_LIST};

static __device__ __noinline__ void sha256_compress_compact(uint32_t* h, uint32_t* wp) {
    uint32_t w[16];
#pragma unroll
    for (int i = 0; i < 16; i++) w[i] = wp[i];
    uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
#pragma unroll 1
    for (int r = 0; r < 4; r++) {
#pragma unroll
        for (int j = 0; j < 16; j++) {
            if (r) {
                uint32_t x = w[(j + 1) & 15], y = w[(j + 14) & 15];
                w[j] += (rotr32(x, 7) ^ rotr32(x, 18) ^ (x >> 3)) + w[(j + 9) & 15] +
                        (rotr32(y, 17) ^ rotr32(y, 19) ^ (y >> 10));
            }
            uint32_t t1 = hh + (rotr32(e, 6) ^ rotr32(e, 11) ^ rotr32(e, 25)) + ((e & f) ^ (~e & g)) +
                          zkh_sha_k[16 * r + j] + w[j];
            uint32_t t2 = (rotr32(a, 2) ^ rotr32(a, 13) ^ rotr32(a, 22)) + ((a & b) ^ (a & c) ^ (b & c));
            hh = g; g = f; f = e; e = d + t1;
            d = c; c = b; b = a; a = t1 + t2;
        }
    }
    h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += hh;
}

// state' = H(state|LE32(ll)|label|LE64(8*nvals)|vals).  Called by all 32 lanes of one warp with
// identical arguments (vals: nvals 64-bit words readable by every lane); buf is shared memory of
// at least 32+4+48+8+320+72 bytes.  Every lane ends with the same new state.
__device__ __forceinline__ void tr_warp_absorb(uint32_t st[8], const char* label, uint32_t ll,
                                               const uint64_t* vals, uint32_t nvals, uint32_t* buf) {
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t total = 32 + 4 + ll + 8 + nvals * 8, padded = ((total + 8) / 64 + 1) * 64;
    __syncwarp();
    if (lane == 0) {
        uint8_t* b = reinterpret_cast<uint8_t*>(buf);
        for (int i = 0; i < 8; i++) buf[i] = bswap32(st[i]);
        uint32_t p = 32;
        b[p++] = (uint8_t)ll; b[p++] = (uint8_t)(ll >> 8); b[p++] = 0; b[p++] = 0;
        for (uint32_t i = 0; i < ll; i++) b[p++] = (uint8_t)label[i];
        const uint32_t len = nvals * 8;
        b[p++] = (uint8_t)len; b[p++] = (uint8_t)(len >> 8);
        for (int i = 0; i < 6; i++) b[p++] = 0;
        for (uint32_t k = 0; k < nvals; k++) {
            uint64_t v = vals[k];
            for (int j = 0; j < 8; j++) b[p++] = (uint8_t)(v >> (8 * j));
        }
        b[p++] = 0x80;
        while (p < padded - 8) b[p++] = 0;
        const uint64_t bits = (uint64_t)total * 8;
        for (int i = 0; i < 8; i++) b[padded - 1 - i] = (uint8_t)(bits >> (8 * i));
    }
    __syncwarp();
    uint32_t h[8];
    sha256_iv(h);
    for (uint32_t off = 0; off < padded / 4; off += 16) {
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 16; i++) w[i] = bswap32(buf[off + i]);
        sha256_compress_compact(h, w);
    }
#pragma unroll
    for (int i = 0; i < 8; i++) st[i] = h[i];
    __syncwarp();
}
// Challenge by a full warp holding the same state on every lane: lane 0 hashes state|"chal",
// lane 1 hashes state|"rtch" in the same instruction stream.  Returns the first 8 digest bytes
// as a little-endian integer on every lane; st becomes the ratcheted state on every lane.
__device__ __forceinline__ uint64_t tr_warp_challenge(uint32_t st[8]) {
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
    for (int i = 0; i < 8; i++) st[i] = __shfl_sync(0xffffffffu, o[i], 1);
    uint32_t c0 = __shfl_sync(0xffffffffu, o[0], 0), c1 = __shfl_sync(0xffffffffu, o[1], 0);
    return (uint64_t)bswap32(c0) | ((uint64_t)bswap32(c1) << 32);
}
__device__ __forceinline__ gl_t tr_warp_chal_gl(uint32_t st[8]) {
    uint64_t v = tr_warp_challenge(st);
    return v >= GL_P ? v - GL_P : v;
}
#define ZKH_TRBUF_WORDS ((32 + 4 + ZKH_TR_MAX_LABEL + 8 + ZKH_TR_MAX_DATA + 72) / 4)
#endif

// first 8 digest bytes as a little-endian u64
GL_HD uint64_t digest_le64(const uint32_t out[8]) {
    return (uint64_t)bswap32(out[0]) | ((uint64_t)bswap32(out[1]) << 32);
}
// field challenge: zkllm-src/p3_scgpu.cuh:31-35
GL_HD gl_t tr_chal_gl(uint32_t st[8]) {
    uint32_t out[8];
    tr_challenge(st, out);
    uint64_t v = digest_le64(out);   // v < 2^64 < 2p: one conditional subtraction is the remainder
    return v >= GL_P ? v - GL_P : v;
}
// query index: zkllm-src/p3_fri.cuh:422-426
GL_HD uint64_t tr_chal_idx(uint32_t st[8], uint64_t mod) {
    uint32_t out[8];
    tr_challenge(st, out);
    return digest_le64(out) % mod;
}

}  // namespace zkh
