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

#ifdef __CUDA_ARCH__
// ---- carry-chain forms for the device: the canonical add / sub / reduce are the bulk of the
// integer-ALU work of every kernel, and the compiler's compare+select sequences for the
// 64-bit carries are about twice as long as these.
__device__ __forceinline__ void gl_split(uint64_t x, uint32_t& lo, uint32_t& hi) {
    asm("mov.b64 {%0,%1}, %2;" : "=r"(lo), "=r"(hi) : "l"(x));
}
__device__ __forceinline__ uint64_t gl_join(uint32_t lo, uint32_t hi) {
    uint64_t x;
    asm("mov.b64 %0, {%1,%2};" : "=l"(x) : "r"(lo), "r"(hi));
    return x;
}
// a, b canonical -> canonical a+b.  s = a+b (65 bits); s >= p  <=>  s + (2^32-1) >= 2^64.
__device__ __forceinline__ gl_t gl_add(gl_t a, gl_t b) {
    uint32_t al, ah, bl, bh, tl, th, ul, uh, c;
    gl_split(a, al, ah);
    gl_split(b, bl, bh);
    asm("{\n\t"
        "add.cc.u32 %0, %5, %7;\n\t"
        "addc.cc.u32 %1, %6, %8;\n\t"
        "addc.u32 %4, 0, 0;\n\t"
        "add.cc.u32 %2, %0, 0xffffffff;\n\t"
        "addc.cc.u32 %3, %1, 0;\n\t"
        "addc.u32 %4, %4, 0;\n\t"
        "}"
        : "=&r"(tl), "=&r"(th), "=&r"(ul), "=&r"(uh), "=&r"(c)
        : "r"(al), "r"(ah), "r"(bl), "r"(bh));
    return c ? gl_join(ul, uh) : gl_join(tl, th);
}
// a, b canonical -> canonical a-b: on borrow add p, i.e. subtract 2^32-1 from the wrapped value
__device__ __forceinline__ gl_t gl_sub(gl_t a, gl_t b) {
    uint32_t al, ah, bl, bh, dl, dh;
    gl_split(a, al, ah);
    gl_split(b, bl, bh);
    asm("{\n\t"
        ".reg .u32 m;\n\t"
        "sub.cc.u32 %0, %2, %4;\n\t"
        "subc.cc.u32 %1, %3, %5;\n\t"
        "subc.u32 m, 0, 0;\n\t"
        "sub.cc.u32 %0, %0, m;\n\t"
        "subc.u32 %1, %1, 0;\n\t"
        "}"
        : "=&r"(dl), "=&r"(dh)
        : "r"(al), "r"(ah), "r"(bl), "r"(bh));
    return gl_join(dl, dh);
}
// hi:lo (any 128-bit value) -> canonical.  hi = hh*2^32 + hl:  lo - hh + hl*(2^32-1)
__device__ __forceinline__ gl_t gl_reduce128(uint64_t lo, uint64_t hi) {
    uint32_t ll, lh, hl, hh, rl, rh, ul, uh, c;
    gl_split(lo, ll, lh);
    gl_split(hi, hl, hh);
    asm("{\n\t"
        ".reg .u32 m, t1l, t1h, k;\n\t"
        "sub.cc.u32 %0, %5, %8;\n\t"      // t0 = lo - hh
        "subc.cc.u32 %1, %6, 0;\n\t"
        "subc.u32 m, 0, 0;\n\t"
        "sub.cc.u32 %0, %0, m;\n\t"       // borrow: -(2^32-1)
        "subc.u32 %1, %1, 0;\n\t"
        "sub.cc.u32 t1l, 0, %7;\n\t"      // t1 = (hl<<32) - hl
        "subc.u32 t1h, %7, 0;\n\t"
        "add.cc.u32 %0, %0, t1l;\n\t"     // t2 = t0 + t1
        "addc.cc.u32 %1, %1, t1h;\n\t"
        "addc.u32 k, 0, 0;\n\t"
        "sub.u32 k, 0, k;\n\t"            // carry: +(2^32-1)
        "add.cc.u32 %0, %0, k;\n\t"
        "addc.u32 %1, %1, 0;\n\t"
        "add.cc.u32 %2, %0, 0xffffffff;\n\t"  // >= p  <=>  + (2^32-1) carries
        "addc.cc.u32 %3, %1, 0;\n\t"
        "addc.u32 %4, 0, 0;\n\t"
        "}"
        : "=&r"(rl), "=&r"(rh), "=&r"(ul), "=&r"(uh), "=&r"(c)
        : "r"(ll), "r"(lh), "r"(hl), "r"(hh));
    return c ? gl_join(ul, uh) : gl_join(rl, rh);
}
#else
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
#endif
GL_HD gl_t gl_neg(gl_t a) { return a ? GL_P - a : 0; }
GL_HD gl_t gl_dbl(gl_t a) { return gl_add(a, a); }

#ifndef __CUDA_ARCH__
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
#endif
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
// a + t*(b-a): the multilinear bind of one pair.  The addend joins the 128-bit product before the
// single reduction ((p-1)^2 + p-1 < 2^128).
GL_HD gl_t gl_lerp(gl_t a, gl_t b, gl_t t) {
    uint64_t lo, hi;
    gl_mul_wide(t, gl_sub(b, a), lo, hi);
    lo += a;
    hi += (lo < a);
    return gl_reduce128(lo, hi);
}

// Lazy sum of 128-bit products.  Holds up to 2^32 products without overflow.
struct Acc192 {
    uint64_t lo, mid;
    uint32_t top;
    GL_HD void clear() { lo = 0; mid = 0; top = 0; }
    GL_HD void add_prod(gl_t a, gl_t b) {
        uint64_t pl, ph;
        gl_mul_wide(a, b, pl, ph);
#ifdef __CUDA_ARCH__
        asm("{\n\t"
            ".reg .u32 a0, a1, a2, a3, b0, b1, b2, b3;\n\t"
            "mov.b64 {a0,a1}, %0;\n\t"
            "mov.b64 {a2,a3}, %1;\n\t"
            "mov.b64 {b0,b1}, %3;\n\t"
            "mov.b64 {b2,b3}, %4;\n\t"
            "add.cc.u32 a0, a0, b0;\n\t"
            "addc.cc.u32 a1, a1, b1;\n\t"
            "addc.cc.u32 a2, a2, b2;\n\t"
            "addc.cc.u32 a3, a3, b3;\n\t"
            "addc.u32 %2, %2, 0;\n\t"
            "mov.b64 %0, {a0,a1};\n\t"
            "mov.b64 %1, {a2,a3};\n\t"
            "}"
            : "+l"(lo), "+l"(mid), "+r"(top)
            : "l"(pl), "l"(ph));
        return;
#endif
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
