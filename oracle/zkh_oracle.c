/*
 * CPU oracle (TEST INFRASTRUCTURE ONLY) -- see zkh_oracle.h for what this is
 * and who may call it.  Plain C11 + unsigned __int128; OpenMP is optional and
 * only changes scheduling (all sums are exact field sums, so any partition
 * gives the same canonical result).
 */
#include "zkh_oracle.h"
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef unsigned __int128 u128;
#define P ORC_GL_P
#define EPS 0xFFFFFFFFULL

/* ======================= field ======================= */
/* zkllm-src/p3_goldilocks.cuh:35-46 -- canonical [0,p) add / sub */
uint64_t orc_gl_add(uint64_t a, uint64_t b) {
    u128 s = (u128)a + b;
    if (s >= P) s -= P;
    return (uint64_t)s;
}
uint64_t orc_gl_sub(uint64_t a, uint64_t b) {
    return a >= b ? a - b : (uint64_t)((u128)a + P - b);
}
/* zkllm-src/p3_goldilocks.cuh:21-57 -- the reference reduces hi:lo with
 * 2^64 = 2^32-1 and 2^96 = -1; the result is the canonical (a*b) mod p, which
 * is what the reference's own selftest pins it to (p3_field_bench.cu:20-22). */
uint64_t orc_gl_mul(uint64_t a, uint64_t b) {
    return (uint64_t)(((u128)a * b) % P);
}
/* zkllm-src/p3_goldilocks.cuh:59-63 */
uint64_t orc_gl_pow(uint64_t a, uint64_t e) {
    uint64_t r = 1, base = a;
    for (; e; e >>= 1) {
        if (e & 1) r = orc_gl_mul(r, base);
        base = orc_gl_mul(base, base);
    }
    return r;
}
/* zkllm-src/p3_goldilocks.cuh:66 -- Fermat */
uint64_t orc_gl_inv(uint64_t a) { return orc_gl_pow(a, P - 2); }
/* zkllm-src/p3_goldilocks.cuh:70-73 -- 7 generates F_p^*; 7^(2^32-1) has order 2^32 */
uint64_t orc_gl_root_of_unity(uint32_t logn) {
    uint64_t g = orc_gl_pow(7, EPS);
    return orc_gl_pow(g, 1ULL << (32 - logn));
}

/* ======================= SHA-256 ======================= */
static const uint32_t KK[64] = {
    0x428a2f98u, 0x71374491u, 0xb5c0fbcfu, 0xe9b5dba5u, 0x3956c25bu, 0x59f111f1u, 0x923f82a4u,
    0xab1c5ed5u, 0xd807aa98u, 0x12835b01u, 0x243185beu, 0x550c7dc3u, 0x72be5d74u, 0x80deb1feu,
    0x9bdc06a7u, 0xc19bf174u, 0xe49b69c1u, 0xefbe4786u, 0x0fc19dc6u, 0x240ca1ccu, 0x2de92c6fu,
    0x4a7484aau, 0x5cb0a9dcu, 0x76f988dau, 0x983e5152u, 0xa831c66du, 0xb00327c8u, 0xbf597fc7u,
    0xc6e00bf3u, 0xd5a79147u, 0x06ca6351u, 0x14292967u, 0x27b70a85u, 0x2e1b2138u, 0x4d2c6dfcu,
    0x53380d13u, 0x650a7354u, 0x766a0abbu, 0x81c2c92eu, 0x92722c85u, 0xa2bfe8a1u, 0xa81a664bu,
    0xc24b8b70u, 0xc76c51a3u, 0xd192e819u, 0xd6990624u, 0xf40e3585u, 0x106aa070u, 0x19a4c116u,
    0x1e376c08u, 0x2748774cu, 0x34b0bcb5u, 0x391c0cb3u, 0x4ed8aa4au, 0x5b9cca4fu, 0x682e6ff3u,
    0x748f82eeu, 0x78a5636fu, 0x84c87814u, 0x8cc70208u, 0x90befffau, 0xa4506cebu, 0xbef9a3f7u,
    0xc67178f2u};
static const uint32_t IV[8] = {0x6a09e667u, 0xbb67ae85u, 0x3c6ef372u, 0xa54ff53au,
                               0x510e527fu, 0x9b05688cu, 0x1f83d9abu, 0x5be0cd19u};

static inline uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }

/* FIPS 180-4 compression of one 64-byte block into h */
static void sha_block(uint32_t h[8], const uint8_t* blk) {
    uint32_t w[64];
    for (int i = 0; i < 16; i++)
        w[i] = ((uint32_t)blk[4 * i] << 24) | ((uint32_t)blk[4 * i + 1] << 16) |
               ((uint32_t)blk[4 * i + 2] << 8) | blk[4 * i + 3];
    for (int i = 16; i < 64; i++) {
        uint32_t a = w[i - 15], b = w[i - 2];
        w[i] = w[i - 16] + (rotr(a, 7) ^ rotr(a, 18) ^ (a >> 3)) + w[i - 7] +
               (rotr(b, 17) ^ rotr(b, 19) ^ (b >> 10));
    }
    uint32_t s[8];
    memcpy(s, h, sizeof s);
    for (int i = 0; i < 64; i++) {
        uint32_t t1 = s[7] + (rotr(s[4], 6) ^ rotr(s[4], 11) ^ rotr(s[4], 25)) +
                      ((s[4] & s[5]) ^ (~s[4] & s[6])) + KK[i] + w[i];
        uint32_t t2 = (rotr(s[0], 2) ^ rotr(s[0], 13) ^ rotr(s[0], 22)) +
                      ((s[0] & s[1]) ^ (s[0] & s[2]) ^ (s[1] & s[2]));
        s[7] = s[6]; s[6] = s[5]; s[5] = s[4]; s[4] = s[3] + t1;
        s[3] = s[2]; s[2] = s[1]; s[1] = s[0]; s[0] = t1 + t2;
    }
    for (int i = 0; i < 8; i++) h[i] += s[i];
}
static void put_be(const uint32_t h[8], uint8_t out[32]) {
    for (int i = 0; i < 8; i++) {
        out[4 * i] = (uint8_t)(h[i] >> 24); out[4 * i + 1] = (uint8_t)(h[i] >> 16);
        out[4 * i + 2] = (uint8_t)(h[i] >> 8); out[4 * i + 3] = (uint8_t)h[i];
    }
}
/* incremental form used by the transcript (several pieces hashed back to back) */
typedef struct { uint32_t h[8]; uint64_t len; uint8_t buf[64]; size_t fill; } sha_ctx;
static void sha_start(sha_ctx* c) { memcpy(c->h, IV, sizeof IV); c->len = 0; c->fill = 0; }
static void sha_feed(sha_ctx* c, const void* data, size_t n) {
    const uint8_t* p = (const uint8_t*)data;
    c->len += n;
    while (n) {
        size_t k = 64 - c->fill;
        if (k > n) k = n;
        memcpy(c->buf + c->fill, p, k);
        c->fill += k; p += k; n -= k;
        if (c->fill == 64) { sha_block(c->h, c->buf); c->fill = 0; }
    }
}
static void sha_finish(sha_ctx* c, uint8_t out[32]) {
    uint64_t bits = c->len * 8;
    uint8_t pad[72];
    size_t padn = (c->fill < 56 ? 56 : 120) - c->fill;
    memset(pad, 0, sizeof pad);
    pad[0] = 0x80;
    for (int i = 0; i < 8; i++) pad[padn + i] = (uint8_t)(bits >> (56 - 8 * i));
    sha_feed(c, pad, padn + 8);
    put_be(c->h, out);
}
/* zkllm-src/fs_transcript.hpp:95-97 */
void orc_sha256(const void* data, size_t n, uint8_t out[32]) {
    sha_ctx c; sha_start(&c); sha_feed(&c, data, n); sha_finish(&c, out);
}
/* zkllm-src/p3_merkle.cuh:69-104 -- ONE compression from the IV, no padding block */
void orc_sha256_compress64(const uint8_t in[64], uint8_t out[32]) {
    uint32_t h[8];
    memcpy(h, IV, sizeof IV);
    sha_block(h, in);
    put_be(h, out);
}

/* ======================= transcript ======================= */
/* zkllm-src/fs_transcript.hpp:118-120 */
void orc_tr_init(uint8_t st[32], const void* seed, size_t n) { orc_sha256(seed, n, st); }
/* zkllm-src/fs_transcript.hpp:121-134: state = H(state | LE32(|label|) | label | LE64(len) | data) */
void orc_tr_absorb(uint8_t st[32], const char* label, const void* data, uint64_t len) {
    sha_ctx c; sha_start(&c);
    sha_feed(&c, st, 32);
    uint32_t ll = (uint32_t)strlen(label);
    uint8_t b4[4] = {(uint8_t)ll, (uint8_t)(ll >> 8), (uint8_t)(ll >> 16), (uint8_t)(ll >> 24)};
    sha_feed(&c, b4, 4);
    sha_feed(&c, label, ll);
    uint8_t b8[8];
    for (int i = 0; i < 8; i++) b8[i] = (uint8_t)(len >> (8 * i));
    sha_feed(&c, b8, 8);
    sha_feed(&c, data, (size_t)len);
    sha_finish(&c, st);
}
/* zkllm-src/fs_transcript.hpp:149-165: out = H(state|"chal"); state = H(state|"rtch") */
void orc_tr_challenge_bytes(uint8_t st[32], uint8_t out[32]) {
    uint8_t m[36];
    memcpy(m, st, 32);
    memcpy(m + 32, "chal", 4);
    orc_sha256(m, 36, out);
    memcpy(m + 32, "rtch", 4);
    orc_sha256(m, 36, st);
}
static uint64_t le64(const uint8_t* b) {
    uint64_t v = 0;
    for (int i = 0; i < 8; i++) v |= (uint64_t)b[i] << (8 * i);
    return v;
}
/* zkllm-src/p3_scgpu.cuh:31-35 (same in p3_basefold.cuh:294-298, p3_gkr.cuh:127-131) */
uint64_t orc_tr_chal(uint8_t st[32]) {
    uint8_t b[32];
    orc_tr_challenge_bytes(st, b);
    return le64(b) % P;
}
/* zkllm-src/p3_fri.cuh:422-426 */
uint64_t orc_tr_idx(uint8_t st[32], uint64_t mod) {
    uint8_t b[32];
    orc_tr_challenge_bytes(st, b);
    return le64(b) % mod;
}

/* ======================= multilinear helpers ======================= */
/* zkllm-src/p3_basefold.cuh:125-136: eq(b,z) = prod_i (b_i ? z_i : 1-z_i), LSB = variable 0.
 * Built by doubling (same products, O(N) instead of O(N v)). */
void orc_build_eq(const uint64_t* z, uint32_t v, uint64_t* out) {
    out[0] = 1;
    for (uint32_t i = 0; i < v; i++) {
        size_t n = (size_t)1 << i;
        uint64_t zi = z[i], omz = orc_gl_sub(1, zi);
        for (size_t b = 0; b < n; b++) {
            uint64_t w = out[b];
            out[b + n] = orc_gl_mul(w, zi);   /* bit i set   */
            out[b] = orc_gl_mul(w, omz);      /* bit i clear */
        }
    }
}
/* zkllm-src/p3_basefold.cuh:139-155 */
uint64_t orc_eval_h(const uint64_t* c, const uint64_t* eq, size_t n) {
    uint64_t acc = 0;
    for (size_t i = 0; i < n; i++) acc = orc_gl_add(acc, orc_gl_mul(c[i], eq[i]));
    return acc;
}
uint64_t orc_mle_eval(const uint64_t* c, const uint64_t* z, uint32_t v) {
    size_t n = (size_t)1 << v;
    uint64_t* eq = (uint64_t*)malloc(n * 8);
    orc_build_eq(z, v, eq);
    uint64_t y = orc_eval_h(c, eq, n);
    free(eq);
    return y;
}
/* zkllm-src/p3_basefold.cuh:300-307: Lagrange through (0,s0),(1,s1),(2,s2) */
uint64_t orc_quad_eval(uint64_t s0, uint64_t s1, uint64_t s2, uint64_t t) {
    uint64_t i2 = orc_gl_inv(2), t1 = orc_gl_sub(t, 1), t2 = orc_gl_sub(t, 2);
    uint64_t L0 = orc_gl_mul(orc_gl_mul(t1, t2), i2);
    uint64_t L1 = orc_gl_sub(0, orc_gl_mul(t, t2));
    uint64_t L2 = orc_gl_mul(orc_gl_mul(t, t1), i2);
    return orc_gl_add(orc_gl_add(orc_gl_mul(s0, L0), orc_gl_mul(s1, L1)), orc_gl_mul(s2, L2));
}
/* zkllm-src/p3_logup.cuh:615-624 (same in p3_gkr.cuh:133-143) */
uint64_t orc_cubic_eval(uint64_t s0, uint64_t s1, uint64_t s2, uint64_t s3, uint64_t t) {
    uint64_t i2 = orc_gl_inv(2), i6 = orc_gl_inv(6);
    uint64_t t1 = orc_gl_sub(t, 1), t2 = orc_gl_sub(t, 2), t3 = orc_gl_sub(t, 3);
    uint64_t L0 = orc_gl_sub(0, orc_gl_mul(orc_gl_mul(orc_gl_mul(t1, t2), t3), i6));
    uint64_t L1 = orc_gl_mul(orc_gl_mul(orc_gl_mul(t, t2), t3), i2);
    uint64_t L2 = orc_gl_sub(0, orc_gl_mul(orc_gl_mul(orc_gl_mul(t, t1), t3), i2));
    uint64_t L3 = orc_gl_mul(orc_gl_mul(orc_gl_mul(t, t1), t2), i6);
    return orc_gl_add(orc_gl_add(orc_gl_mul(s0, L0), orc_gl_mul(s1, L1)),
                      orc_gl_add(orc_gl_mul(s2, L2), orc_gl_mul(s3, L3)));
}
/* zkllm-src/p3_hawkeye.cuh:642-655 */
uint64_t orc_quartic_eval(const uint64_t s[5], uint64_t t) {
    /* Lagrange basis on nodes 0..4: L_k(t) = prod_{j!=k}(t-j) / prod_{j!=k}(k-j) */
    static const int64_t den[5] = {24, -6, 4, -6, 24};
    uint64_t acc = 0;
    for (int k = 0; k < 5; k++) {
        uint64_t num = 1;
        for (int j = 0; j < 5; j++)
            if (j != k) num = orc_gl_mul(num, orc_gl_sub(t, (uint64_t)j));
        uint64_t d = den[k] > 0 ? (uint64_t)den[k] : orc_gl_sub(0, (uint64_t)(-den[k]));
        acc = orc_gl_add(acc, orc_gl_mul(s[k], orc_gl_mul(num, orc_gl_inv(d))));
    }
    return acc;
}
/* zkllm-src/p3_basefold.cuh:309-316 */
uint64_t orc_eq_point(const uint64_t* a, const uint64_t* z, uint32_t v) {
    uint64_t prod = 1;
    for (uint32_t i = 0; i < v; i++) {
        uint64_t t = orc_gl_add(orc_gl_mul(a[i], z[i]),
                                orc_gl_mul(orc_gl_sub(1, a[i]), orc_gl_sub(1, z[i])));
        prod = orc_gl_mul(prod, t);
    }
    return prod;
}
/* zkllm-src/p3_scgpu.cuh:41-44: f'[i] = f[2i] + a*(f[2i+1]-f[2i]) */
void orc_bind_lsb(uint64_t* f, size_t n, uint64_t a) {
    size_t h = n / 2;
    /* in place is safe serially: f[i] is written after f[2i],f[2i+1] (2i >= i) are read */
    for (size_t i = 0; i < h; i++)
        f[i] = orc_gl_add(f[2 * i], orc_gl_mul(a, orc_gl_sub(f[2 * i + 1], f[2 * i])));
}

/* ======================= generic sumcheck ======================= */
static inline uint64_t summand(int functor, const uint64_t* c, const uint64_t* p) {
    switch (functor) {
    case ORC_F_PROD2: /* zkllm-src/p3_basefold.cuh:319-330 */
        return orc_gl_mul(c[0], c[1]);
    case ORC_F_PROD3: /* zkllm-src/p3_int_gadgets.cuh:539-544 */
        return orc_gl_mul(c[0], orc_gl_mul(c[1], c[2]));
    case ORC_F_GKR:   /* zkllm-src/p3_gkr.cuh:48-53 */
        return orc_gl_mul(c[0], orc_gl_add(orc_gl_add(orc_gl_mul(c[1], c[4]), orc_gl_mul(c[2], c[3])),
                                           orc_gl_mul(p[0], orc_gl_mul(c[3], c[4]))));
    case ORC_F_IRS1: /* zkllm-src/p3_int_gadgets.cuh:316-325, one limb */
    case ORC_F_IRS2: {
        uint64_t t = orc_gl_sub(orc_gl_add(c[1], p[0]), orc_gl_mul(c[2], p[1]));
        t = orc_gl_sub(t, c[3]);
        if (functor == ORC_F_IRS2) t = orc_gl_sub(t, orc_gl_mul(c[4], 65536ULL));
        return orc_gl_mul(c[0], t);
    }
    case ORC_F_LOGUP: /* zkllm-src/p3_logup.cuh:49-54 */
        return orc_gl_add(orc_gl_mul(p[0], c[0]),
                          orc_gl_mul(c[2], orc_gl_sub(orc_gl_mul(c[0], orc_gl_add(c[1], p[1])), c[3])));
    }
    return 0;
}
static int functor_nc(int functor) {
    switch (functor) {
    case ORC_F_PROD2: return 2;
    case ORC_F_PROD3: return 3;
    case ORC_F_GKR: return 5;
    case ORC_F_LOGUP: return 4;
    case ORC_F_IRS1: return 4;
    case ORC_F_IRS2: return 5;
    }
    return -1;
}
#define ORC_MAXC 8
#define ORC_MAXNT 5
/* One round message over the current columns: evaluations at t=0..nt-1 of
 * sum_i F(lo_i + t*(hi_i-lo_i)), pairs (2i,2i+1): zkllm-src/p3_scgpu.cuh:56-83 */
static void round_message(int functor, int nt, uint64_t** cols, int nc, size_t half,
                          const uint64_t* par, uint64_t* s, int nthreads) {
    for (int t = 0; t < nt; t++) s[t] = 0;
    int nparts = 1;
#ifdef _OPENMP
    if (nthreads > 1 && half >= 4096) nparts = nthreads * 4;
#endif
    (void)nthreads;
    uint64_t* part = (uint64_t*)calloc((size_t)nparts * ORC_MAXNT, 8);
#ifdef _OPENMP
#pragma omp parallel for schedule(static) num_threads(nthreads > 1 ? nthreads : 1) if (nparts > 1)
#endif
    for (int pi = 0; pi < nparts; pi++) {
        size_t lo = half * (size_t)pi / nparts, hi = half * (size_t)(pi + 1) / nparts;
        uint64_t acc[ORC_MAXNT] = {0}, cur[ORC_MAXC], dd[ORC_MAXC];
        for (size_t i = lo; i < hi; i++) {
            for (int k = 0; k < nc; k++) {
                cur[k] = cols[k][2 * i];
                dd[k] = orc_gl_sub(cols[k][2 * i + 1], cur[k]);
            }
            for (int t = 0; t < nt; t++) {
                acc[t] = orc_gl_add(acc[t], summand(functor, cur, par));
                if (t + 1 < nt)
                    for (int k = 0; k < nc; k++) cur[k] = orc_gl_add(cur[k], dd[k]);
            }
        }
        for (int t = 0; t < nt; t++) part[(size_t)pi * ORC_MAXNT + t] = acc[t];
    }
    for (int pi = 0; pi < nparts; pi++)
        for (int t = 0; t < nt; t++) s[t] = orc_gl_add(s[t], part[(size_t)pi * ORC_MAXNT + t]);
    free(part);
}
static void bind_cols(uint64_t** cols, int nc, size_t half, uint64_t a, int nthreads) {
#ifdef _OPENMP
    if (nthreads > 1 && half >= 8192) {
        /* out-of-place per column so the pair reads never race the writes */
        for (int k = 0; k < nc; k++) {
            uint64_t* f = cols[k];
            uint64_t* tmp = (uint64_t*)malloc(half * 8);
#pragma omp parallel for schedule(static) num_threads(nthreads)
            for (size_t i = 0; i < half; i++)
                tmp[i] = orc_gl_add(f[2 * i], orc_gl_mul(a, orc_gl_sub(f[2 * i + 1], f[2 * i])));
            memcpy(f, tmp, half * 8);
            free(tmp);
        }
        return;
    }
#endif
    (void)nthreads;
    for (int k = 0; k < nc; k++) orc_bind_lsb(cols[k], half * 2, a);
}
/* zkllm-src/p3_scgpu.cuh:91-160 (driver loop), p3_hawkeye.cuh:659-695 (host twin):
 * per round: message -> absorb under `tag` -> one challenge -> bind every column */
int orc_sumcheck(uint8_t st[32], const char* tag, int functor, int nt, uint64_t** cols, int nc,
                 uint32_t logn, const uint64_t* par, uint64_t* msgs, uint64_t* chals,
                 uint64_t* finals, int nthreads) {
    if (nc != functor_nc(functor) || nt < 2 || nt > ORC_MAXNT || nc > ORC_MAXC) return -1;
    size_t n = (size_t)1 << logn;
    for (uint32_t rd = 0; rd < logn; rd++) {
        size_t half = n / 2;
        uint64_t s[ORC_MAXNT];
        round_message(functor, nt, cols, nc, half, par, s, nthreads);
        memcpy(msgs + (size_t)rd * nt, s, (size_t)nt * 8);
        orc_tr_absorb(st, tag, s, (uint64_t)nt * 8);
        uint64_t a = orc_tr_chal(st);
        chals[rd] = a;
        bind_cols(cols, nc, half, a, nthreads);
        n = half;
    }
    if (finals)
        for (int k = 0; k < nc; k++) finals[k] = cols[k][0];
    return 0;
}

/* ======================= Reed-Solomon / NTT ======================= */
/* zkllm-src/p3_basefold.cuh:162-172 -- cw[j] = poly(w^j), Horner, O(N*M) */
void orc_rs_encode_horner(const uint64_t* c, uint32_t v, uint32_t R, uint64_t* cw) {
    size_t N = (size_t)1 << v, M = (size_t)1 << (v + R);
    uint64_t w = orc_gl_root_of_unity(v + R);
    for (size_t j = 0; j < M; j++) {
        uint64_t x = orc_gl_pow(w, j), acc = 0;
        for (size_t i = N; i-- > 0;) acc = orc_gl_add(orc_gl_mul(acc, x), c[i]);
        cw[j] = acc;
    }
}
/* zkllm-src/p3_ntt.cuh:170-230 -- out[k] = sum_j a[j] w^(jk), natural order in and out.
 * Any correct transform yields the same canonical values; this one is a
 * textbook bit-reverse + decimation-in-time loop. */
void orc_ntt(uint64_t* a, uint32_t logn, int inverse) {
    size_t n = (size_t)1 << logn;
    for (size_t i = 0; i < n; i++) {
        size_t r = 0;
        for (uint32_t b = 0; b < logn; b++) r |= ((i >> b) & 1) << (logn - 1 - b);
        if (r > i) { uint64_t t = a[i]; a[i] = a[r]; a[r] = t; }
    }
    uint64_t w = orc_gl_root_of_unity(logn);
    if (inverse) w = orc_gl_inv(w);
    for (uint32_t s = 1; s <= logn; s++) {
        size_t m = (size_t)1 << s, h = m >> 1;
        uint64_t wm = orc_gl_pow(w, n / m);
        for (size_t base = 0; base < n; base += m) {
            uint64_t tw = 1;
            for (size_t i = 0; i < h; i++) {
                uint64_t u = a[base + i], t = orc_gl_mul(a[base + i + h], tw);
                a[base + i] = orc_gl_add(u, t);
                a[base + i + h] = orc_gl_sub(u, t);
                tw = orc_gl_mul(tw, wm);
            }
        }
    }
    if (inverse) {
        uint64_t ninv = orc_gl_inv((uint64_t)n);
        for (size_t i = 0; i < n; i++) a[i] = orc_gl_mul(a[i], ninv);
    }
}
/* zkllm-src/p3_basefold.cuh:188-197 -- zero-pad to 2^(v+R), forward NTT */
void orc_rs_encode(const uint64_t* c, uint32_t v, uint32_t R, uint64_t* cw) {
    size_t N = (size_t)1 << v, M = (size_t)1 << (v + R);
    memcpy(cw, c, N * 8);
    memset(cw + N, 0, (M - N) * 8);
    orc_ntt(cw, v + R, 0);
}

/* ======================= Merkle ======================= */
/* zkllm-src/p3_fri.cuh:33-35 -- full SHA-256 of the 8-byte little-endian value */
void orc_leaf_hash(uint64_t v, uint8_t out[32]) {
    uint8_t b[8];
    for (int k = 0; k < 8; k++) b[k] = (uint8_t)(v >> (8 * k));
    orc_sha256(b, 8, out);
}
/* zkllm-src/p3_fri.cuh:36-39 -- single compression of l|r from the IV */
/* salted leaf of the hiding commitment (zkllm-src/p3_zkc.cuh:235-249 salt_of, salted_leaf):
 * salt = SHA-256(seed_le8 | index_le8), leaf = SHA-256(value_le8 | salt) */
void orc_salt_of(uint64_t sseed, uint64_t idx, uint8_t out[32]) {
    uint8_t sb[16];
    for (int k = 0; k < 8; k++) { sb[k] = (uint8_t)(sseed >> (8 * k)); sb[8 + k] = (uint8_t)(idx >> (8 * k)); }
    orc_sha256(sb, 16, out);
}
void orc_salted_leaf_hash(uint64_t v, uint64_t sseed, uint64_t idx, uint8_t out[32]) {
    uint8_t b[40];
    orc_salt_of(sseed, idx, b + 8);
    for (int k = 0; k < 8; k++) b[k] = (uint8_t)(v >> (8 * k));
    orc_sha256(b, 40, out);
}
void orc_node_hash(const uint8_t l[32], const uint8_t r[32], uint8_t out[32]) {
    uint8_t b[64];
    memcpy(b, l, 32);
    memcpy(b + 32, r, 32);
    orc_sha256_compress64(b, out);
}
/* zkllm-src/p3_fri.cuh:42-56 */
void orc_merkle_build(const uint64_t* cw, size_t M, uint8_t* tree) {
#ifdef _OPENMP
#pragma omp parallel for schedule(static) if (M >= 4096)
#endif
    for (size_t i = 0; i < M; i++) orc_leaf_hash(cw[i], tree + i * 32);
    uint8_t* cur = tree;
    for (size_t cnt = M; cnt > 1; cnt /= 2) {
        uint8_t* nxt = cur + cnt * 32;
#ifdef _OPENMP
#pragma omp parallel for schedule(static) if (cnt >= 4096)
#endif
        for (size_t i = 0; i < cnt / 2; i++)
            orc_node_hash(cur + 2 * i * 32, cur + (2 * i + 1) * 32, nxt + i * 32);
        cur = nxt;
    }
}
/* tree with salted leaves; internal nodes as orc_merkle_build (zkllm-src/p3_zkc.cuh:294-318 SaltedDevMerkle) */
void orc_merkle_build_salted(const uint64_t* cw, size_t M, uint64_t sseed, uint8_t* tree) {
    for (size_t i = 0; i < M; i++) orc_salted_leaf_hash(cw[i], sseed, (uint64_t)i, tree + i * 32);
    uint8_t* cur = tree;
    for (size_t cnt = M; cnt > 1; cnt >>= 1) {
        uint8_t* nxt = cur + cnt * 32;
        for (size_t i = 0; i < cnt / 2; i++) orc_node_hash(cur + 2 * i * 32, cur + (2 * i + 1) * 32, nxt + i * 32);
        cur = nxt;
    }
}
void orc_merkle_root(const uint64_t* cw, size_t M, uint8_t root[32]) {
    uint8_t* tree = (uint8_t*)malloc((2 * M - 1) * 32);
    orc_merkle_build(cw, M, tree);
    memcpy(root, tree + (2 * M - 2) * 32, 32);
    free(tree);
}
/* zkllm-src/p3_fri.cuh:80-84 -- sibling at every level below the root */
void orc_merkle_path(const uint8_t* tree, size_t M, size_t idx, uint8_t* path) {
    const uint8_t* lvl = tree;
    size_t d = 0;
    for (size_t cnt = M; cnt > 1; cnt /= 2, d++) {
        memcpy(path + d * 32, lvl + (idx ^ 1) * 32, 32);
        idx >>= 1;
        lvl += cnt * 32;
    }
}
/* zkllm-src/p3_fri.cuh:87-91 */
int orc_merkle_verify_path(const uint8_t leaf[32], size_t idx, const uint8_t* path, uint32_t plen,
                           const uint8_t root[32]) {
    uint8_t h[32], t[32];
    memcpy(h, leaf, 32);
    for (uint32_t d = 0; d < plen; d++) {
        if (idx & 1) orc_node_hash(path + d * 32, h, t);
        else orc_node_hash(h, path + d * 32, t);
        memcpy(h, t, 32);
        idx >>= 1;
    }
    return memcmp(h, root, 32) == 0;
}

/* ======================= fold ======================= */
/* zkllm-src/p3_fri.cuh:396-402 */
uint64_t orc_fold_pair(uint64_t a, uint64_t b, uint64_t invx, uint64_t beta, int mle) {
    uint64_t i2 = orc_gl_inv(2);
    uint64_t E = orc_gl_mul(orc_gl_add(a, b), i2);
    uint64_t O = orc_gl_mul(orc_gl_mul(orc_gl_sub(a, b), i2), invx);
    if (mle) return orc_gl_add(orc_gl_mul(orc_gl_sub(1, beta), E), orc_gl_mul(beta, O));
    return orc_gl_add(E, orc_gl_mul(beta, O));
}
/* zkllm-src/p3_fri.cuh:405-415 -- pairs (c, c+M/2), x = wM^c */
void orc_fold(const uint64_t* f, size_t M, uint64_t wM, uint64_t beta, int mle, uint64_t* out) {
    size_t half = M / 2;
    uint64_t winv = orc_gl_inv(wM), i2 = orc_gl_inv(2), invx = 1;
    uint64_t omb = orc_gl_sub(1, beta);
    for (size_t c = 0; c < half; c++) {
        uint64_t E = orc_gl_mul(orc_gl_add(f[c], f[c + half]), i2);
        uint64_t O = orc_gl_mul(orc_gl_mul(orc_gl_sub(f[c], f[c + half]), i2), invx);
        out[c] = mle ? orc_gl_add(orc_gl_mul(omb, E), orc_gl_mul(beta, O))
                     : orc_gl_add(E, orc_gl_mul(beta, O));
        invx = orc_gl_mul(invx, winv);
    }
}

/* ======================= Basefold opening ======================= */
size_t orc_bf_proof_size(uint32_t v, uint32_t R, uint32_t Q) {
    size_t s = 12 + (size_t)v * 32 + (size_t)v * 24 + ((size_t)8 << R);
    for (uint32_t r = 0; r < v; r++) s += (size_t)Q * (16 + 2 * (size_t)(v + R - r) * 32);
    return s + (size_t)v * 8 + 8;
}
static void put32(uint8_t** p, uint32_t x) { memcpy(*p, &x, 4); *p += 4; }
static void put64(uint8_t** p, uint64_t x) { memcpy(*p, &x, 8); *p += 8; }

/* zkllm-src/p3_basefold.cuh:423-496 (host) == :355-420 (device-resident), A.5 schedule:
 * absorb "z","y"; per round: root -> "root", message -> "sc", alpha, bind c and eq,
 * fold the codeword with the same alpha; "final"; Q query indices. */
size_t orc_bf_prove_eval(const uint64_t* c, const uint64_t* z, uint32_t v, uint64_t y, uint32_t R,
                         uint32_t Q, const uint64_t* cw0, const char* seed, uint8_t* out,
                         size_t cap) {
    size_t need = orc_bf_proof_size(v, R, Q);
    if (!out) return need;
    if (cap < need) return 0;
    uint32_t logM0 = v + R;
    size_t M0 = (size_t)1 << logM0, N = (size_t)1 << v;
    uint8_t st[32];
    orc_tr_init(st, seed, strlen(seed));
    orc_tr_absorb(st, "z", z, (uint64_t)v * 8);
    orc_tr_absorb(st, "y", &y, 8);

    uint64_t** words = (uint64_t**)calloc(v + 1, sizeof(uint64_t*));
    uint8_t** trees = (uint8_t**)calloc(v + 1, sizeof(uint8_t*));
    words[0] = (uint64_t*)malloc(M0 * 8);
    memcpy(words[0], cw0, M0 * 8);
    uint64_t* cc = (uint64_t*)malloc(N * 8);
    uint64_t* ww = (uint64_t*)malloc(N * 8);
    memcpy(cc, c, N * 8);
    orc_build_eq(z, v, ww);

    uint8_t* p = out;
    put32(&p, v); put32(&p, R); put32(&p, Q);
    uint8_t* p_roots = p;
    uint8_t* p_msgs = p_roots + (size_t)v * 32;
    for (uint32_t r = 0; r < v; r++) {
        size_t Mr = M0 >> r, n = N >> r, half = n / 2;
        trees[r] = (uint8_t*)malloc((2 * Mr - 1) * 32);
        orc_merkle_build(words[r], Mr, trees[r]);
        const uint8_t* root = trees[r] + (2 * Mr - 2) * 32;
        memcpy(p_roots + (size_t)r * 32, root, 32);
        orc_tr_absorb(st, "root", root, 32);
        uint64_t s0 = 0, s1 = 0, s2 = 0;
        for (size_t b = 0; b < half; b++) {
            uint64_t cl = cc[2 * b], ch = cc[2 * b + 1], wl = ww[2 * b], wh = ww[2 * b + 1];
            s0 = orc_gl_add(s0, orc_gl_mul(cl, wl));
            s1 = orc_gl_add(s1, orc_gl_mul(ch, wh));
            uint64_t c2 = orc_gl_sub(orc_gl_add(ch, ch), cl), w2 = orc_gl_sub(orc_gl_add(wh, wh), wl);
            s2 = orc_gl_add(s2, orc_gl_mul(c2, w2));
        }
        uint64_t msg[3] = {s0, s1, s2};
        memcpy(p_msgs + (size_t)r * 24, msg, 24);
        orc_tr_absorb(st, "sc", msg, 24);
        uint64_t a = orc_tr_chal(st);
        orc_bind_lsb(cc, n, a);
        orc_bind_lsb(ww, n, a);
        words[r + 1] = (uint64_t*)malloc((Mr / 2) * 8);
        orc_fold(words[r], Mr, orc_gl_root_of_unity(logM0 - r), a, 1, words[r + 1]);
    }
    p = p_msgs + (size_t)v * 24;
    size_t fin = (size_t)1 << R;
    memcpy(p, words[v], fin * 8);
    orc_tr_absorb(st, "final", words[v], fin * 8);
    p += fin * 8;
    for (uint32_t q = 0; q < Q; q++) {
        size_t pos = (size_t)orc_tr_idx(st, M0 / 2);
        for (uint32_t r = 0; r < v; r++) {
            size_t Mr = M0 >> r, h = Mr / 2, ci = pos % h;
            uint32_t plen = logM0 - r;
            put64(&p, words[r][ci]);
            put64(&p, words[r][ci + h]);
            orc_merkle_path(trees[r], Mr, ci, p); p += (size_t)plen * 32;
            orc_merkle_path(trees[r], Mr, ci + h, p); p += (size_t)plen * 32;
            pos = ci;
        }
    }
    memcpy(p, z, (size_t)v * 8); p += (size_t)v * 8;
    put64(&p, y);
    for (uint32_t r = 0; r <= v; r++) { free(words[r]); free(trees[r]); }
    free(words); free(trees); free(cc); free(ww);
    return (size_t)(p - out);
}

/* zkllm-src/p3_basefold.cuh:499-535 + p3_fri.cuh:466-502 */
int orc_bf_verify_eval(const uint8_t* proof, size_t len, const char* seed) {
    if (len < 12) return 0;
    uint32_t v, R, Q;
    memcpy(&v, proof, 4); memcpy(&R, proof + 4, 4); memcpy(&Q, proof + 8, 4);
    if (v > 40 || R > 8 || len != orc_bf_proof_size(v, R, Q)) return 0;
    uint32_t logM0 = v + R;
    size_t M0 = (size_t)1 << logM0, fin = (size_t)1 << R;
    const uint8_t* roots = proof + 12;
    const uint8_t* msgs = roots + (size_t)v * 32;
    const uint8_t* fw = msgs + (size_t)v * 24;
    const uint8_t* qs = fw + fin * 8;
    const uint8_t* zp = proof + len - 8 - (size_t)v * 8;
    uint64_t y; memcpy(&y, proof + len - 8, 8);
    uint64_t* z = (uint64_t*)malloc(((size_t)v + 1) * 8);
    uint64_t* al = (uint64_t*)malloc(((size_t)v + 1) * 8);
    uint64_t* final_word = (uint64_t*)malloc(fin * 8);
    memcpy(z, zp, (size_t)v * 8);
    memcpy(final_word, fw, fin * 8);
    int ok = 1;
    uint8_t st[32];
    orc_tr_init(st, seed, strlen(seed));
    orc_tr_absorb(st, "z", z, (uint64_t)v * 8);
    orc_tr_absorb(st, "y", &y, 8);
    uint64_t claim = y;
    for (uint32_t r = 0; r < v && ok; r++) {
        orc_tr_absorb(st, "root", roots + (size_t)r * 32, 32);
        uint64_t m[3]; memcpy(m, msgs + (size_t)r * 24, 24);
        if (orc_gl_add(m[0], m[1]) != claim) ok = 0;
        orc_tr_absorb(st, "sc", m, 24);
        al[r] = orc_tr_chal(st);
        claim = orc_quad_eval(m[0], m[1], m[2], al[r]);
    }
    orc_tr_absorb(st, "final", final_word, fin * 8);
    for (size_t i = 1; i < fin; i++) if (final_word[i] != final_word[0]) ok = 0;
    if (claim != orc_gl_mul(final_word[0], orc_eq_point(al, z, v))) ok = 0;
    const uint8_t* p = qs;
    for (uint32_t q = 0; q < Q && ok; q++) {
        size_t pos = (size_t)orc_tr_idx(st, M0 / 2);
        uint64_t prev_folded = 0;
        for (uint32_t r = 0; r < v; r++) {
            size_t Mr = M0 >> r, h = Mr / 2, ci = pos % h;
            uint32_t plen = logM0 - r;
            uint64_t a, b; memcpy(&a, p, 8); memcpy(&b, p + 8, 8); p += 16;
            const uint8_t* pa = p; p += (size_t)plen * 32;
            const uint8_t* pb = p; p += (size_t)plen * 32;
            uint8_t lh[32];
            orc_leaf_hash(a, lh);
            if (!orc_merkle_verify_path(lh, ci, pa, plen, roots + (size_t)r * 32)) ok = 0;
            orc_leaf_hash(b, lh);
            if (!orc_merkle_verify_path(lh, ci + h, pb, plen, roots + (size_t)r * 32)) ok = 0;
            if (r > 0) {
                /* the previous round folded to position `pos` of this round's word */
                uint64_t val = pos < h ? a : b;
                if (val != prev_folded) ok = 0;
            }
            uint64_t x = orc_gl_pow(orc_gl_root_of_unity(plen), ci);
            prev_folded = orc_fold_pair(a, b, orc_gl_inv(x), al[r], 1);
            if (r + 1 == v && final_word[ci] != prev_folded) ok = 0;
            pos = ci;
        }
    }
    free(z); free(al); free(final_word);
    return ok;
}

/* ======================= GKR fractional-sum tree ======================= */
size_t orc_gkr_proof_size(uint32_t L) {
    size_t s = 16;
    for (uint32_t h = L; h >= 1; h--) s += 4 + (size_t)(L - h) * 32 + 32;
    return s;
}
/* zkllm-src/p3_gkr.cuh:200-364, A.6 schedule */
size_t orc_gkr_prove(uint8_t st[32], const char* tag, const uint64_t* pl, const uint64_t* ql,
                     uint32_t L, int combine_last, uint64_t* rfin, uint64_t cpq[2], uint8_t* out,
                     size_t cap) {
    size_t need = orc_gkr_proof_size(L);
    if (!out) return need;
    if (cap < need || L < 1) return 0;
    /* levels h=0 (leaves) .. L (root); level h has 2^(L-h) nodes; node y <- children 2y,2y+1 */
    uint64_t** lp = (uint64_t**)calloc(L + 1, sizeof(uint64_t*));
    uint64_t** lq = (uint64_t**)calloc(L + 1, sizeof(uint64_t*));
    size_t N0 = (size_t)1 << L;
    lp[0] = (uint64_t*)malloc(N0 * 8); memcpy(lp[0], pl, N0 * 8);
    lq[0] = (uint64_t*)malloc(N0 * 8); memcpy(lq[0], ql, N0 * 8);
    for (uint32_t h = 1; h <= L; h++) {
        size_t n = (size_t)1 << (L - h);
        lp[h] = (uint64_t*)malloc(n * 8);
        lq[h] = (uint64_t*)malloc(n * 8);
        for (size_t yv = 0; yv < n; yv++) {
            uint64_t p1 = lp[h - 1][2 * yv], p2 = lp[h - 1][2 * yv + 1];
            uint64_t q1 = lq[h - 1][2 * yv], q2 = lq[h - 1][2 * yv + 1];
            lp[h][yv] = orc_gl_add(orc_gl_mul(p1, q2), orc_gl_mul(p2, q1));
            lq[h][yv] = orc_gl_mul(q1, q2);
        }
    }
    uint8_t* p = out;
    uint64_t rt[2] = {lp[L][0], lq[L][0]};
    size_t ret = 0;
    if (rt[1] == 0) goto done;               /* zero denominator: reference throws */
    put64(&p, rt[0]); put64(&p, rt[1]);
    orc_tr_absorb(st, tag, rt, 16);
    {
        uint64_t* zpt = (uint64_t*)calloc(L + 1, 8);
        uint64_t* r = (uint64_t*)calloc(L + 1, 8);
        uint32_t zlen = 0;
        for (uint32_t h = L; h >= 1; h--) {
            const uint64_t* cp = lp[h - 1];
            const uint64_t* cq = lq[h - 1];
            uint64_t term[4];
            uint32_t nr = 0;
            if (h == L) {
                term[0] = cp[0]; term[1] = cp[1]; term[2] = cq[0]; term[3] = cq[1];
                put32(&p, 0);
            } else {
                uint64_t lam = orc_tr_chal(st);
                size_t n = (size_t)1 << (L - h);
                uint64_t* colsbuf = (uint64_t*)malloc(5 * n * 8);
                uint64_t* cols[5];
                for (int k = 0; k < 5; k++) cols[k] = colsbuf + (size_t)k * n;
                orc_build_eq(zpt, zlen, cols[0]);
                for (size_t yv = 0; yv < n; yv++) {
                    cols[1][yv] = cp[2 * yv]; cols[2][yv] = cp[2 * yv + 1];
                    cols[3][yv] = cq[2 * yv]; cols[4][yv] = cq[2 * yv + 1];
                }
                nr = L - h;
                put32(&p, nr);
                uint64_t fin[5];
                orc_sumcheck(st, tag, ORC_F_GKR, 4, cols, 5, nr, &lam, (uint64_t*)(void*)p, r, fin, 1);
                p += (size_t)nr * 32;
                term[0] = fin[1]; term[1] = fin[2]; term[2] = fin[3]; term[3] = fin[4];
                free(colsbuf);
            }
            memcpy(p, term, 32); p += 32;
            orc_tr_absorb(st, tag, term, 32);
            if (h > 1 || combine_last) {
                uint64_t mu = orc_tr_chal(st);
                zpt[0] = mu;
                memcpy(zpt + 1, r, (size_t)nr * 8);
                zlen = nr + 1;
                if (h == 1) {
                    memcpy(rfin, zpt, (size_t)zlen * 8);
                    if (cpq) {
                        cpq[0] = orc_gl_add(term[0], orc_gl_mul(mu, orc_gl_sub(term[1], term[0])));
                        cpq[1] = orc_gl_add(term[2], orc_gl_mul(mu, orc_gl_sub(term[3], term[2])));
                    }
                }
            } else {
                memcpy(rfin, r, (size_t)nr * 8);
            }
        }
        free(zpt); free(r);
    }
    ret = (size_t)(p - out);
done:
    for (uint32_t h = 0; h <= L; h++) { free(lp[h]); free(lq[h]); }
    free(lp); free(lq);
    return ret;
}

/* zkllm-src/p3_gkr.cuh:370-421 */
int orc_gkr_verify(uint8_t st[32], const char* tag, uint32_t L, const uint8_t* proof, size_t len,
                   int combine_last, uint64_t* rfin, uint64_t out4[4]) {
    if (L < 1 || len != orc_gkr_proof_size(L)) return 0;
    const uint8_t* p = proof;
    uint64_t rt[2]; memcpy(rt, p, 16); p += 16;
    if (rt[1] == 0) return 0;
    orc_tr_absorb(st, tag, rt, 16);
    uint64_t* zpt = (uint64_t*)calloc(L + 1, 8);
    uint64_t* r = (uint64_t*)calloc(L + 1, 8);
    uint32_t zlen = 0;
    uint64_t cp = 0, cq = 0;
    int ok = 1;
    for (uint32_t h = L; h >= 1 && ok; h--) {
        uint32_t nm; memcpy(&nm, p, 4); p += 4;
        if (nm != L - h) { ok = 0; break; }
        const uint8_t* mp = p; p += (size_t)nm * 32;
        uint64_t t[4]; memcpy(t, p, 32); p += 32;
        uint64_t cross = orc_gl_add(orc_gl_mul(t[0], t[3]), orc_gl_mul(t[1], t[2]));
        uint64_t qq = orc_gl_mul(t[2], t[3]);
        if (h == L) {
            if (cross != rt[0] || qq != rt[1]) ok = 0;
        } else {
            uint64_t lam = orc_tr_chal(st);
            uint64_t claim = orc_gl_add(cp, orc_gl_mul(lam, cq));
            for (uint32_t rd = 0; rd < nm; rd++) {
                uint64_t m[4]; memcpy(m, mp + (size_t)rd * 32, 32);
                if (orc_gl_add(m[0], m[1]) != claim) ok = 0;
                orc_tr_absorb(st, tag, m, 32);
                r[rd] = orc_tr_chal(st);
                claim = orc_cubic_eval(m[0], m[1], m[2], m[3], r[rd]);
            }
            uint64_t end = orc_gl_mul(orc_eq_point(zpt, r, nm), orc_gl_add(cross, orc_gl_mul(lam, qq)));
            if (claim != end) ok = 0;
        }
        orc_tr_absorb(st, tag, t, 32);
        if (h > 1 || combine_last) {
            uint64_t mu = orc_tr_chal(st);
            cp = orc_gl_add(t[0], orc_gl_mul(mu, orc_gl_sub(t[1], t[0])));
            cq = orc_gl_add(t[2], orc_gl_mul(mu, orc_gl_sub(t[3], t[2])));
            zpt[0] = mu;
            memcpy(zpt + 1, r, (size_t)nm * 8);
            zlen = nm + 1;
            if (h == 1) {
                memcpy(rfin, zpt, (size_t)zlen * 8);
                out4[0] = cp; out4[1] = 0; out4[2] = cq; out4[3] = 0;
            }
        } else {
            memcpy(rfin, r, (size_t)nm * 8);
            memcpy(out4, t, 32);
        }
    }
    (void)zlen;
    free(zpt); free(r);
    return ok;
}

/* ======================= logUp primitives ======================= */
/* zkllm-src/p3_logup.cuh:149-172 (device) / :1412-1475 (host loop): cnt[idx[i]]++ */
int orc_histogram(const uint32_t* idx, size_t n, uint32_t M, uint64_t* cnt) {
    memset(cnt, 0, (size_t)M * 8);
    for (size_t i = 0; i < n; i++) {
        if (idx[i] >= M) return -1;
        cnt[idx[i]]++;
    }
    return 0;
}
/* zkllm-src/p3_logup.cuh:636-660 -- out[i] = 1/(A[i]+beta); the blocking of the
 * reference's batch inversion does not change any value, so one block is used. */
int orc_inv_all_add(const uint64_t* A, size_t n, uint64_t beta, uint64_t* out) {
    if (!n) return 0;
    uint64_t* d = (uint64_t*)malloc(n * 8);
    uint64_t acc = 1;
    int zero = 0;
    for (size_t i = 0; i < n; i++) {
        uint64_t di = orc_gl_add(A[i], beta);
        if (di == 0) { zero = 1; di = 1; }
        d[i] = di;
        out[i] = acc;              /* prefix product of d[0..i) */
        acc = orc_gl_mul(acc, di);
    }
    uint64_t inv = orc_gl_inv(acc);
    for (size_t i = n; i-- > 0;) {
        out[i] = orc_gl_mul(out[i], inv);
        inv = orc_gl_mul(inv, d[i]);
    }
    free(d);
    return zero ? -1 : 0;
}
/* zkllm-src/p3_logup.cuh:663-672 -- out[i] = sum_k g^k cols[k][i] */
void orc_combine(const uint64_t* const* cols, int c, size_t n, uint64_t g, uint64_t* out) {
    memset(out, 0, n * 8);
    uint64_t gk = 1;
    for (int k = 0; k < c; k++) {
        for (size_t i = 0; i < n; i++) out[i] = orc_gl_add(out[i], orc_gl_mul(gk, cols[k][i]));
        gk = orc_gl_mul(gk, g);
    }
}

/* zkllm-src/p3_basefold_selftest.cu:12-13 -- s = s*6364136223846793005 + 1442695040888963407;
 * output z = s ^ (s >> 31), reduced mod p by the caller there; here reduced directly */
void orc_lcg_fill(uint64_t* out, size_t n, uint64_t* state) {
    uint64_t s = *state;
    for (size_t i = 0; i < n; i++) {
        s = s * 6364136223846793005ULL + 1442695040888963407ULL;
        uint64_t zz = s ^ (s >> 31);
        out[i] = zz % P;
    }
    *state = s;
}

/* randomness of the hiding mode (zkllm-src/p3_zkc.cuh:100-118): the sequential chain and the random-access stream */
void orc_zprng_fill(uint64_t s, uint64_t* out, size_t n) {
    for (size_t i = 0; i < n; i++) {
        s = s * 6364136223846793005ULL + 1442695040888963407ULL;
        uint64_t z = s ^ (s >> 31);
        out[i] = z % P;
    }
}
uint64_t orc_zprng_at(uint64_t seed, uint64_t i) {
    uint64_t z = seed + 0x9E3779B97F4A7C15ULL * (i + 1);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    z ^= z >> 31;
    return z % P;
}

/* ======================= batched opening (one size class, non-zk) ======================= */
/* Serialized BatchProof (fields of p3bo::BatchProof in declaration order, zk fields omitted):
 *   u32 v, R, Q, nc | ystar nc*8 | rmsgs v*24 | roots (v-1)*32 | omsgs v*24 | final 2^R*8 |
 *   per query q, per round r = 1..v-1: a(8) b(8) pa((v+R-r)*32) pb((v+R-r)*32) |
 *   per distinct column: u32 nvals, vals nvals*8, u32 nnodes, nodes nnodes*32 */
static int cmp_u32(const void* a, const void* b) {
    uint32_t x = *(const uint32_t*)a, y = *(const uint32_t*)b;
    return x < y ? -1 : x > y;
}
size_t orc_bo_proof_bound(uint32_t v, uint32_t R, uint32_t Q, uint32_t nc) {
    size_t s = 16 + (size_t)nc * 8 + (size_t)v * 48 + (size_t)(v ? v - 1 : 0) * 32 + ((size_t)8 << R);
    for (uint32_t r = 1; r < v; r++) s += (size_t)Q * (16 + 2 * (size_t)(v + R - r) * 32);
    s += (size_t)nc * (8 + (size_t)2 * Q * 8 + (size_t)2 * Q * (v + R) * 32);
    return s;
}
/* distinct columns by root, first appearance: zkllm-src/p3_batchopen.cuh:393-403 */
static uint32_t dedupe_roots(const uint8_t* roots, uint32_t k, uint32_t* colidx, uint32_t* first) {
    uint32_t nc = 0;
    for (uint32_t j = 0; j < k; j++) {
        uint32_t c = 0;
        while (c < nc && memcmp(roots + (size_t)first[c] * 32, roots + (size_t)j * 32, 32)) c++;
        if (c == nc) first[nc++] = j;
        colidx[j] = c;
    }
    return nc;
}
/* pruned multi-path node stream: zkllm-src/p3_batchopen.cuh:75-106 (subset_prove).  The emitted
 * siblings do not depend on the recomputed hashes, so only the index walk is needed. */
static size_t subset_nodes(uint32_t logM, const uint32_t* upos, uint32_t nu, const uint8_t* tree, size_t M,
                           uint8_t* out) {
    uint32_t* fr = (uint32_t*)malloc((size_t)nu * 4);
    memcpy(fr, upos, (size_t)nu * 4);
    uint32_t nf = nu;
    size_t nn = 0;
    const uint8_t* lvl = tree;
    size_t cnt = M;
    for (uint32_t l = 0; l < logM; l++) {
        uint32_t w = 0, i = 0;
        while (i < nf) {
            uint32_t idx = fr[i];
            if (!(idx & 1) && i + 1 < nf && fr[i + 1] == (idx | 1)) i += 2;
            else { memcpy(out + nn * 32, lvl + (size_t)(idx ^ 1) * 32, 32); nn++; i += 1; }
            fr[w++] = idx >> 1;
        }
        nf = w;
        lvl += cnt * 32;
        cnt /= 2;
    }
    free(fr);
    return nn;
}
/* zkllm-src/p3_batchopen.cuh:307-1147 (prove_class), A.8 schedule; sseeds != NULL: the hiding mode's salted
 * round-0 openings (:1028-1131), the class blinder having been appended to the ledger by the caller */
static size_t bo_prove_class_impl(uint8_t st[32], uint32_t v, const uint64_t* pts, uint32_t T,
                          const uint64_t* const* cols, const uint8_t* roots, const uint32_t* zid, uint32_t k,
                          uint32_t R, uint32_t Q, const char* label, uint8_t* out, size_t cap, const uint64_t* sseeds) {
    const size_t N = (size_t)1 << v;
    const uint32_t logM0 = v + R;
    const size_t M0 = (size_t)1 << logM0;
    uint32_t* colidx = (uint32_t*)malloc((size_t)k * 4);
    uint32_t* first = (uint32_t*)malloc((size_t)k * 4);
    const uint32_t nc = dedupe_roots(roots, k, colidx, first);
    if (cap < orc_bo_proof_bound(v, R, Q, nc) + (sseeds ? (size_t)nc * 2 * Q * 32 : 0)) { free(colidx); free(first); return 0; }
    uint8_t* p = out;
    put32(&p, v); put32(&p, R); put32(&p, Q); put32(&p, nc);
    uint8_t* p_ystar = p;            p += (size_t)nc * 8;
    uint8_t* p_rmsgs = p;            p += (size_t)v * 24;
    uint8_t* p_roots = p;            p += (size_t)(v ? v - 1 : 0) * 32;
    uint8_t* p_omsgs = p;            p += (size_t)v * 24;
    uint8_t* p_final = p;            p += (size_t)8 << R;

    uint64_t mu = orc_tr_chal(st);
    /* G_t = sum_{j at point t} mu^j col_j ; E_t = eq(z_t, .) */
    uint64_t* G = (uint64_t*)calloc((size_t)T * N, 8);
    uint64_t* E = (uint64_t*)malloc((size_t)T * N * 8);
    uint64_t wj = 1;
    for (uint32_t j = 0; j < k; j++) {
        uint64_t* g = G + (size_t)zid[j] * N;
        for (size_t i = 0; i < N; i++) g[i] = orc_gl_add(g[i], orc_gl_mul(wj, cols[j][i]));
        wj = orc_gl_mul(wj, mu);
    }
    for (uint32_t t = 0; t < T; t++) orc_build_eq(pts + (size_t)t * v, v, E + (size_t)t * N);
    /* reduction sumcheck over all points at once */
    uint64_t* rstar = (uint64_t*)malloc(((size_t)v + 1) * 8);
    for (uint32_t rd = 0; rd < v; rd++) {
        size_t L = N >> rd, half = L / 2;
        uint64_t s0 = 0, s1 = 0, s2 = 0;
        for (uint32_t t = 0; t < T; t++) {
            const uint64_t* c = G + (size_t)t * L;   /* bound arrays stay packed per point */
            const uint64_t* w = E + (size_t)t * L;
            for (size_t i = 0; i < half; i++) {
                uint64_t cl = c[2 * i], ch = c[2 * i + 1], wl = w[2 * i], wh = w[2 * i + 1];
                s0 = orc_gl_add(s0, orc_gl_mul(cl, wl));
                s1 = orc_gl_add(s1, orc_gl_mul(ch, wh));
                s2 = orc_gl_add(s2, orc_gl_mul(orc_gl_sub(orc_gl_add(ch, ch), cl),
                                               orc_gl_sub(orc_gl_add(wh, wh), wl)));
            }
        }
        uint64_t m[3] = {s0, s1, s2};
        memcpy(p_rmsgs + (size_t)rd * 24, m, 24);
        orc_tr_absorb(st, "bo-rm", m, 24);
        uint64_t a = orc_tr_chal(st);
        rstar[rd] = a;
        /* the stacked arrays bind as one array: pairs never cross a point (L is even) */
        orc_bind_lsb(G, (size_t)T * L, a);
        orc_bind_lsb(E, (size_t)T * L, a);
    }
    free(G); free(E);
    /* per-column terminal evaluations */
    uint64_t* eqr = (uint64_t*)malloc(N * 8);
    orc_build_eq(rstar, v, eqr);
    uint64_t* ystar = (uint64_t*)malloc(((size_t)nc + 1) * 8);
    for (uint32_t c = 0; c < nc; c++) ystar[c] = orc_eval_h(cols[first[c]], eqr, N);
    memcpy(p_ystar, ystar, (size_t)nc * 8);
    orc_tr_absorb(st, "bo-ys", ystar, (uint64_t)nc * 8);
    uint64_t rho = orc_tr_chal(st);
    uint64_t* U = (uint64_t*)calloc(N, 8);
    uint64_t yU = 0, w = 1;
    for (uint32_t c = 0; c < nc; c++) {
        const uint64_t* col = cols[first[c]];
        for (size_t i = 0; i < N; i++) U[i] = orc_gl_add(U[i], orc_gl_mul(w, col[i]));
        yU = orc_gl_add(yU, orc_gl_mul(w, ystar[c]));
        w = orc_gl_mul(w, rho);
    }
    /* opening of U at r* on its own transcript; round 0 carries no root */
    uint8_t ot[32];
    orc_tr_init(ot, label, strlen(label));
    orc_tr_absorb(ot, "z", rstar, (uint64_t)v * 8);
    orc_tr_absorb(ot, "y", &yU, 8);
    uint64_t** words = (uint64_t**)calloc(v + 1, sizeof(uint64_t*));
    uint8_t** trees = (uint8_t**)calloc(v + 1, sizeof(uint8_t*));
    words[0] = (uint64_t*)malloc(M0 * 8);
    orc_rs_encode(U, v, R, words[0]);
    for (uint32_t r = 0; r < v; r++) {
        size_t Mr = M0 >> r, n = N >> r, half = n / 2;
        if (r > 0) {
            trees[r] = (uint8_t*)malloc((2 * Mr - 1) * 32);
            orc_merkle_build(words[r], Mr, trees[r]);
            const uint8_t* root = trees[r] + (2 * Mr - 2) * 32;
            memcpy(p_roots + (size_t)(r - 1) * 32, root, 32);
            orc_tr_absorb(ot, "root", root, 32);
        }
        uint64_t s0 = 0, s1 = 0, s2 = 0;
        for (size_t b = 0; b < half; b++) {
            uint64_t cl = U[2 * b], ch = U[2 * b + 1], wl = eqr[2 * b], wh = eqr[2 * b + 1];
            s0 = orc_gl_add(s0, orc_gl_mul(cl, wl));
            s1 = orc_gl_add(s1, orc_gl_mul(ch, wh));
            s2 = orc_gl_add(s2, orc_gl_mul(orc_gl_sub(orc_gl_add(ch, ch), cl), orc_gl_sub(orc_gl_add(wh, wh), wl)));
        }
        uint64_t m[3] = {s0, s1, s2};
        memcpy(p_omsgs + (size_t)r * 24, m, 24);
        orc_tr_absorb(ot, "sc", m, 24);
        uint64_t a = orc_tr_chal(ot);
        orc_bind_lsb(U, n, a);
        orc_bind_lsb(eqr, n, a);
        words[r + 1] = (uint64_t*)malloc((Mr / 2) * 8);
        orc_fold(words[r], Mr, orc_gl_root_of_unity(logM0 - r), a, 1, words[r + 1]);
    }
    size_t fin = (size_t)1 << R;
    memcpy(p_final, words[v], fin * 8);
    orc_tr_absorb(ot, "final", words[v], fin * 8);
    uint32_t* pos0 = (uint32_t*)malloc(((size_t)Q + 1) * 4);
    for (uint32_t q = 0; q < Q; q++) {
        size_t pos = (size_t)orc_tr_idx(ot, M0 / 2);
        for (uint32_t r = 0; r < v; r++) {
            size_t Mr = M0 >> r, h = Mr / 2, ci = pos % h;
            if (r == 0) pos0[q] = (uint32_t)ci;
            else {
                uint32_t plen = logM0 - r;
                put64(&p, words[r][ci]);
                put64(&p, words[r][ci + h]);
                orc_merkle_path(trees[r], Mr, ci, p); p += (size_t)plen * 32;
                orc_merkle_path(trees[r], Mr, ci + h, p); p += (size_t)plen * 32;
            }
            pos = ci;
        }
    }
    /* round-0 openings per distinct column against its own commitment */
    uint32_t* upos = (uint32_t*)malloc(((size_t)2 * Q + 1) * 4);
    uint32_t nu = 0;
    for (uint32_t q = 0; q < Q; q++) { upos[nu++] = pos0[q]; upos[nu++] = pos0[q] + (uint32_t)(M0 / 2); }
    qsort(upos, nu, 4, cmp_u32);
    { uint32_t w2 = 0; for (uint32_t i = 0; i < nu; i++) if (!i || upos[i] != upos[i - 1]) upos[w2++] = upos[i]; nu = w2; }
    uint64_t* cwc = (uint64_t*)malloc(M0 * 8);
    uint8_t* treec = (uint8_t*)malloc((2 * M0 - 1) * 32);
    for (uint32_t c = 0; c < nc; c++) {
        orc_rs_encode(cols[first[c]], v, R, cwc);
        if (sseeds) orc_merkle_build_salted(cwc, M0, sseeds[first[c]], treec);
        else orc_merkle_build(cwc, M0, treec);
        put32(&p, nu);
        for (uint32_t i = 0; i < nu; i++) put64(&p, cwc[upos[i]]);
        if (sseeds)
            for (uint32_t i = 0; i < nu; i++) { orc_salt_of(sseeds[first[c]], upos[i], p); p += 32; }
        uint8_t* p_cnt = p; p += 4;
        uint32_t nn = (uint32_t)subset_nodes(logM0, upos, nu, treec, M0, p);
        memcpy(p_cnt, &nn, 4);
        p += (size_t)nn * 32;
    }
    free(cwc); free(treec); free(upos); free(pos0);
    for (uint32_t r = 0; r <= v; r++) { free(words[r]); free(trees[r]); }
    free(words); free(trees); free(U); free(eqr); free(ystar); free(rstar); free(colidx); free(first);
    return (size_t)(p - out);
}
size_t orc_bo_prove_class(uint8_t st[32], uint32_t v, const uint64_t* pts, uint32_t T,
                          const uint64_t* const* cols, const uint8_t* roots, const uint32_t* zid, uint32_t k,
                          uint32_t R, uint32_t Q, const char* label, uint8_t* out, size_t cap) {
    return bo_prove_class_impl(st, v, pts, T, cols, roots, zid, k, R, Q, label, out, cap, NULL);
}
size_t orc_bo_prove_class_salted(uint8_t st[32], uint32_t v, const uint64_t* pts, uint32_t T,
                                 const uint64_t* const* cols, const uint8_t* roots, const uint32_t* zid,
                                 const uint64_t* sseeds, uint32_t k, uint32_t R, uint32_t Q, const char* label,
                                 uint8_t* out, size_t cap) {
    return bo_prove_class_impl(st, v, pts, T, cols, roots, zid, k, R, Q, label, out, cap, sseeds);
}

/* subset_verify: zkllm-src/p3_batchopen.cuh:108-135 */
static int subset_verify(uint32_t logM, const uint32_t* upos, uint32_t nu, const uint8_t* leaves,
                         const uint8_t* nodes, uint32_t nnodes, const uint8_t root[32]) {
    uint32_t* fi = (uint32_t*)malloc((size_t)nu * 4);
    uint8_t* fh = (uint8_t*)malloc((size_t)nu * 32);
    memcpy(fi, upos, (size_t)nu * 4);
    memcpy(fh, leaves, (size_t)nu * 32);
    uint32_t nf = nu, ni = 0;
    int ok = 1;
    for (uint32_t l = 0; l < logM && ok; l++) {
        uint32_t w = 0, i = 0;
        while (i < nf) {
            uint32_t idx = fi[i];
            uint8_t h[32];
            if (!(idx & 1) && i + 1 < nf && fi[i + 1] == (idx | 1)) {
                orc_node_hash(fh + (size_t)i * 32, fh + (size_t)(i + 1) * 32, h);
                i += 2;
            } else {
                if (ni >= nnodes) { ok = 0; break; }
                const uint8_t* sib = nodes + (size_t)ni++ * 32;
                if (idx & 1) orc_node_hash(sib, fh + (size_t)i * 32, h);
                else orc_node_hash(fh + (size_t)i * 32, sib, h);
                i += 1;
            }
            fi[w] = idx >> 1;
            memcpy(fh + (size_t)w * 32, h, 32);
            w++;
        }
        nf = w;
    }
    ok = ok && ni == nnodes && nf == 1 && !memcmp(fh, root, 32);
    free(fi); free(fh);
    return ok;
}
/* zkllm-src/p3_batchopen.cuh:1149-1302 (verify_class), non-zk.  1 = accept */
int orc_bo_verify_class(uint8_t st[32], uint32_t v, const uint64_t* pts, uint32_t T, const uint8_t* roots,
                        const uint32_t* zid, const uint64_t* y, uint32_t k, uint32_t R, uint32_t Q,
                        const char* label, const uint8_t* proof, size_t len) {
    const uint32_t logM0 = v + R;
    const size_t M0 = (size_t)1 << logM0, fin = (size_t)1 << R;
    if (len < 16) return 0;
    uint32_t hv, hR, hQ, hnc;
    memcpy(&hv, proof, 4); memcpy(&hR, proof + 4, 4); memcpy(&hQ, proof + 8, 4); memcpy(&hnc, proof + 12, 4);
    if (hv != v || hR != R || hQ != Q) return 0;
    uint32_t* colidx = (uint32_t*)malloc((size_t)k * 4);
    uint32_t* first = (uint32_t*)malloc((size_t)k * 4);
    const uint32_t nc = dedupe_roots(roots, k, colidx, first);
    int ok = hnc == nc;
    size_t fixed = 16 + (size_t)nc * 8 + (size_t)v * 48 + (size_t)(v ? v - 1 : 0) * 32 + fin * 8;
    for (uint32_t r = 1; r < v; r++) fixed += (size_t)Q * (16 + 2 * (size_t)(logM0 - r) * 32);
    if (!ok || len < fixed) { free(colidx); free(first); return 0; }
    const uint8_t* p = proof + 16;
    const uint64_t* ystar = (const uint64_t*)(const void*)p;  p += (size_t)nc * 8;
    const uint8_t* rmsgs = p;  p += (size_t)v * 24;
    const uint8_t* proots = p; p += (size_t)(v ? v - 1 : 0) * 32;
    const uint8_t* omsgs = p;  p += (size_t)v * 24;
    const uint8_t* fw = p;     p += fin * 8;
    const uint8_t* qsec = p;
    uint64_t* ys = (uint64_t*)malloc(((size_t)nc + 1) * 8);
    memcpy(ys, ystar, (size_t)nc * 8);
    uint64_t* final_word = (uint64_t*)malloc(fin * 8);
    memcpy(final_word, fw, fin * 8);

    uint64_t mu = orc_tr_chal(st);
    uint64_t claim = 0, wj = 1;
    for (uint32_t j = 0; j < k; j++) { claim = orc_gl_add(claim, orc_gl_mul(wj, y[j])); wj = orc_gl_mul(wj, mu); }
    uint64_t* rstar = (uint64_t*)malloc(((size_t)v + 1) * 8);
    uint64_t* al = (uint64_t*)malloc(((size_t)v + 1) * 8);
    for (uint32_t rd = 0; rd < v; rd++) {
        uint64_t m[3]; memcpy(m, rmsgs + (size_t)rd * 24, 24);
        if (orc_gl_add(m[0], m[1]) != claim) ok = 0;
        orc_tr_absorb(st, "bo-rm", m, 24);
        rstar[rd] = orc_tr_chal(st);
        claim = orc_quad_eval(m[0], m[1], m[2], rstar[rd]);
    }
    orc_tr_absorb(st, "bo-ys", ys, (uint64_t)nc * 8);
    {
        uint64_t* gt = (uint64_t*)calloc(T, 8);
        wj = 1;
        for (uint32_t j = 0; j < k; j++) {
            gt[zid[j]] = orc_gl_add(gt[zid[j]], orc_gl_mul(wj, ys[colidx[j]]));
            wj = orc_gl_mul(wj, mu);
        }
        uint64_t end = 0;
        for (uint32_t t = 0; t < T; t++)
            end = orc_gl_add(end, orc_gl_mul(orc_eq_point(rstar, pts + (size_t)t * v, v), gt[t]));
        if (end != claim) ok = 0;
        free(gt);
    }
    uint64_t rho = orc_tr_chal(st);
    uint64_t* rhop = (uint64_t*)malloc(((size_t)nc + 1) * 8);
    uint64_t yU = 0, wc = 1;
    for (uint32_t c = 0; c < nc; c++) { rhop[c] = wc; yU = orc_gl_add(yU, orc_gl_mul(wc, ys[c])); wc = orc_gl_mul(wc, rho); }
    uint8_t ot[32];
    orc_tr_init(ot, label, strlen(label));
    orc_tr_absorb(ot, "z", rstar, (uint64_t)v * 8);
    orc_tr_absorb(ot, "y", &yU, 8);
    uint64_t oclaim = yU;
    for (uint32_t r = 0; r < v; r++) {
        if (r > 0) orc_tr_absorb(ot, "root", proots + (size_t)(r - 1) * 32, 32);
        uint64_t m[3]; memcpy(m, omsgs + (size_t)r * 24, 24);
        if (orc_gl_add(m[0], m[1]) != oclaim) ok = 0;
        orc_tr_absorb(ot, "sc", m, 24);
        al[r] = orc_tr_chal(ot);
        oclaim = orc_quad_eval(m[0], m[1], m[2], al[r]);
    }
    orc_tr_absorb(ot, "final", final_word, fin * 8);
    for (size_t i = 1; i < fin; i++) if (final_word[i] != final_word[0]) ok = 0;
    if (oclaim != orc_gl_mul(final_word[0], orc_eq_point(al, rstar, v))) ok = 0;
    uint32_t* c0q = (uint32_t*)malloc(((size_t)Q + 1) * 4);
    uint32_t* upos = (uint32_t*)malloc(((size_t)2 * Q + 1) * 4);
    uint32_t nu = 0;
    for (uint32_t q = 0; q < Q; q++) {
        c0q[q] = (uint32_t)orc_tr_idx(ot, M0 / 2);
        upos[nu++] = c0q[q]; upos[nu++] = c0q[q] + (uint32_t)(M0 / 2);
    }
    qsort(upos, nu, 4, cmp_u32);
    { uint32_t w2 = 0; for (uint32_t i = 0; i < nu; i++) if (!i || upos[i] != upos[i - 1]) upos[w2++] = upos[i]; nu = w2; }
    /* locate the per-column sections */
    const uint8_t* q0 = qsec;
    for (uint32_t r = 1; r < v; r++) q0 += (size_t)Q * (16 + 2 * (size_t)(logM0 - r) * 32);
    const uint8_t** cvals = (const uint8_t**)calloc(nc + 1, sizeof(uint8_t*));
    const uint8_t* cp = q0;
    uint8_t* leaves = (uint8_t*)malloc(((size_t)nu + 1) * 32);
    for (uint32_t c = 0; c < nc && ok; c++) {
        if ((size_t)(cp - proof) + 4 > len) { ok = 0; break; }
        uint32_t nv; memcpy(&nv, cp, 4); cp += 4;
        if (nv != nu || (size_t)(cp - proof) + (size_t)nv * 8 + 4 > len) { ok = 0; break; }
        cvals[c] = cp; cp += (size_t)nv * 8;
        uint32_t nn; memcpy(&nn, cp, 4); cp += 4;
        if ((size_t)(cp - proof) + (size_t)nn * 32 > len) { ok = 0; break; }
        for (uint32_t i = 0; i < nu; i++) { uint64_t x; memcpy(&x, cvals[c] + (size_t)i * 8, 8); orc_leaf_hash(x, leaves + (size_t)i * 32); }
        if (!subset_verify(logM0, upos, nu, leaves, cp, nn, roots + (size_t)first[c] * 32)) ok = 0;
        cp += (size_t)nn * 32;
    }
    if (ok && (size_t)(cp - proof) != len) ok = 0;
    const uint8_t* qp = qsec;
    for (uint32_t q = 0; q < Q && ok; q++) {
        size_t pos = c0q[q];
        uint64_t prev = 0;
        for (uint32_t r = 0; r < v; r++) {
            size_t Mr = M0 >> r, h = Mr / 2, ci = pos % h;
            uint32_t plen = logM0 - r;
            uint64_t a = 0, b = 0;
            if (r == 0) {
                uint32_t key = (uint32_t)ci, sa, sb;
                sa = (uint32_t)((uint32_t*)bsearch(&key, upos, nu, 4, cmp_u32) - upos);
                key = (uint32_t)(ci + h);
                sb = (uint32_t)((uint32_t*)bsearch(&key, upos, nu, 4, cmp_u32) - upos);
                for (uint32_t c = 0; c < nc; c++) {
                    uint64_t va, vb;
                    memcpy(&va, cvals[c] + (size_t)sa * 8, 8); memcpy(&vb, cvals[c] + (size_t)sb * 8, 8);
                    a = orc_gl_add(a, orc_gl_mul(rhop[c], va));
                    b = orc_gl_add(b, orc_gl_mul(rhop[c], vb));
                }
            } else {
                memcpy(&a, qp, 8); memcpy(&b, qp + 8, 8); qp += 16;
                const uint8_t* pa = qp; qp += (size_t)plen * 32;
                const uint8_t* pb = qp; qp += (size_t)plen * 32;
                uint8_t lh[32];
                orc_leaf_hash(a, lh);
                if (!orc_merkle_verify_path(lh, ci, pa, plen, proots + (size_t)(r - 1) * 32)) ok = 0;
                orc_leaf_hash(b, lh);
                if (!orc_merkle_verify_path(lh, ci + h, pb, plen, proots + (size_t)(r - 1) * 32)) ok = 0;
                uint64_t val = pos < h ? a : b;
                if (val != prev) ok = 0;
            }
            uint64_t x = orc_gl_pow(orc_gl_root_of_unity(plen), ci);
            prev = orc_fold_pair(a, b, orc_gl_inv(x), al[r], 1);
            if (r + 1 == v && final_word[ci] != prev) ok = 0;
            pos = ci;
        }
    }
    free(colidx); free(first); free(ys); free(final_word); free(rstar); free(al); free(rhop); free(c0q); free(upos);
    free(cvals); free(leaves);
    return ok;
}
