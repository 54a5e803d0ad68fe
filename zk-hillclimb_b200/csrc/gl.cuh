// Goldilocks field p = 2^64 - 2^32 + 1 for sm_100a kernels.
//
// Value semantics follow the reference exactly (zkllm-src/p3_goldilocks.cuh:16-73):
// an element is its canonical integer in [0, p); no Montgomery form.  How a value
// is computed is free -- every function here returns the unique canonical
// representative, so results are bit-identical to the reference's.
//
// Two layers:
//   * gl_add / gl_sub / gl_mul ...   canonical in, canonical out
//   * Acc192                         lazy accumulator for sums of products: 128-bit
//                                    products are added into 160 bits and reduced
//                                    once (2^64 = 2^32-1, 2^96 = -1, 2^128 = -2^32)
#pragma once
#include <cstdint>

#define GL_P 0xFFFFFFFF00000001ULL
#define GL_EPS 0x00000000FFFFFFFFULL

#if defined(__CUDACC__)
#define GL_HD __host__ __device__ __forceinline__
#else
#define GL_HD inline
#endif

typedef uint64_t gl_t;

GL_HD gl_t gl_add(gl_t a, gl_t b) {
    uint64_t s = a + b;
    if (s < a) s += GL_EPS;  // wrapped past 2^64 == EPS (mod p); cannot wrap twice
    if (s >= GL_P) s -= GL_P;
    return s;
}
GL_HD gl_t gl_sub(gl_t a, gl_t b) {
    uint64_t d = a - b;
    if (a < b) d -= GL_EPS;  // borrow of 2^64 == EPS
    return d;
}
GL_HD gl_t gl_neg(gl_t a) { return a ? GL_P - a : 0; }
GL_HD gl_t gl_dbl(gl_t a) { return gl_add(a, a); }

// hi:lo (< 2^128) -> canonical.  hi = hh*2^32 + hl:  lo - hh + hl*(2^32-1)
GL_HD gl_t gl_reduce128(uint64_t lo, uint64_t hi) {
    uint32_t hh = (uint32_t)(hi >> 32), hl = (uint32_t)hi;
    uint64_t t0 = lo - hh;
    if (lo < hh) t0 -= GL_EPS;
    uint64_t t1 = ((uint64_t)hl << 32) - hl;
    uint64_t t2 = t0 + t1;
    if (t2 < t0) t2 += GL_EPS;
    if (t2 >= GL_P) t2 -= GL_P;
    return t2;
}
GL_HD void gl_mul_wide(gl_t a, gl_t b, uint64_t& lo, uint64_t& hi) {
#ifdef __CUDA_ARCH__
    lo = a * b;
    hi = __umul64hi(a, b);
#else
    unsigned __int128 p = (unsigned __int128)a * b;
    lo = (uint64_t)p;
    hi = (uint64_t)(p >> 64);
#endif
}
GL_HD gl_t gl_mul(gl_t a, gl_t b) {
    uint64_t lo, hi;
    gl_mul_wide(a, b, lo, hi);
    return gl_reduce128(lo, hi);
}
GL_HD gl_t gl_pow(gl_t a, uint64_t e) {
    gl_t r = 1, base = a;
    while (e) {
        if (e & 1) r = gl_mul(r, base);
        base = gl_mul(base, base);
        e >>= 1;
    }
    return r;
}
GL_HD gl_t gl_inv(gl_t a) { return gl_pow(a, GL_P - 2); }
// primitive 2^logn-th root of unity: 7 generates F_p^*, 7^(2^32-1) has order 2^32
GL_HD gl_t gl_root_of_unity(uint32_t logn) {
    return gl_pow(gl_pow(7ULL, GL_EPS), 1ULL << (32 - logn));
}
// a + t*(b-a): the multilinear bind of one pair
GL_HD gl_t gl_lerp(gl_t a, gl_t b, gl_t t) { return gl_add(a, gl_mul(t, gl_sub(b, a))); }

// Lazy sum of 128-bit products.  Holds up to 2^32 products without overflow.
struct Acc192 {
    uint64_t lo, mid;
    uint32_t top;
    GL_HD void clear() { lo = 0; mid = 0; top = 0; }
    GL_HD void add_prod(gl_t a, gl_t b) {
        uint64_t pl, ph;
        gl_mul_wide(a, b, pl, ph);
        lo += pl;
        uint64_t c = lo < pl;
        uint64_t m = mid + ph;
        uint32_t c2 = m < ph;
        m += c;
        c2 += m < c;
        mid = m;
        top += c2;
    }
    GL_HD void add_val(gl_t a) {
        lo += a;
        uint64_t c = lo < a;
        mid += c;
        top += (uint32_t)(mid < c);
    }
    // canonical value of lo + mid*2^64 + top*2^128
    GL_HD gl_t reduce() const {
        gl_t r = gl_reduce128(lo, mid);
        // 2^128 == -2^32 (mod p); top < 2^32 so top*2^32 < 2^64; bring below p first
        uint64_t t = (uint64_t)top << 32;
        if (t >= GL_P) t -= GL_P;
        return gl_sub(r, t);
    }
};
