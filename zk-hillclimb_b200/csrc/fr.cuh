// BLS12-381 scalar field for sm_100a.
//   p = 0x73eda753299d7d483339d80809a1d80553bda402fffe5bfeffffffff00000001  (255 bits)
// Elements are eight 32-bit limbs, little endian, 32 bytes: the reference's Fr_t
// (zkllm-src/bls12-381.cuh:116-120).  The reference keeps tensors as PLAIN integers and multiplies
// with a Montgomery routine, converting around each product (e.g. zkllm-src/zkfc.cu:94-112); every
// quantity that reaches a proof or a transcript is a plain canonical value.  The kernels here follow
// the same convention at their boundaries and track the power of R = 2^256 a product chain carries
// internally, correcting once per reduced sum instead of once per element.
//
// Montgomery multiplication is operand scanning with two carry chains per row (even and odd limbs of
// the multiplicand, each product's low half directly followed by its high half: mad.lo.cc / madc.hi.cc),
// then the same pair of chains for m*p with m = t[0] * (-1/p mod 2^32) = -t[0] (p = 1 mod 2^32).
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace zkh {

struct __align__(16) Fr { uint32_t v[8]; };

#define ZKH_FR_LIMBS(a, b, c, d, e, f, g, h) {{a, b, c, d, e, f, g, h}}
#define ZKH_FR_P_INIT  ZKH_FR_LIMBS(0x00000001u, 0xffffffffu, 0xfffe5bfeu, 0x53bda402u, 0x09a1d805u, 0x3339d808u, 0x299d7d48u, 0x73eda753u)
#define ZKH_FR_R1_INIT ZKH_FR_LIMBS(0xfffffffeu, 0x00000001u, 0x00034802u, 0x5884b7fau, 0xecbc4ff5u, 0x998c4fefu, 0xacc5056fu, 0x1824b159u)
#define ZKH_FR_R2_INIT ZKH_FR_LIMBS(0xf3f29c6du, 0xc999e990u, 0x87925c23u, 0x2b6cedcbu, 0x7254398fu, 0x05d31496u, 0x9f59ff11u, 0x0748d9d9u)
#define ZKH_FR_R3_INIT ZKH_FR_LIMBS(0x439b73afu, 0xc62c1807u, 0x8cf06990u, 0x1b3e0d18u, 0xc7b5f418u, 0x73d13c71u, 0xc8db33e9u, 0x6e2a5bb9u)
#define ZKH_FR_R4_INIT ZKH_FR_LIMBS(0xd0831ad3u, 0x1b9c9191u, 0x6f830a6cu, 0x08fd47d3u, 0xb364c750u, 0xf948ab00u, 0x916f202cu, 0x08a63526u)

#ifdef __CUDACC__
static __device__ __constant__ Fr FR_P = ZKH_FR_P_INIT;
// R^k mod p, k = 1..4: multiplying a value that carries R^-(k-1) by R^k (Montgomery) makes it plain
static __device__ __constant__ Fr FR_RPOW[4] = {ZKH_FR_R1_INIT, ZKH_FR_R2_INIT, ZKH_FR_R3_INIT, ZKH_FR_R4_INIT};

__device__ __forceinline__ Fr fr_zero() {
    Fr r;
#pragma unroll
    for (int i = 0; i < 8; i++) r.v[i] = 0;
    return r;
}
__device__ __forceinline__ Fr fr_load(const Fr* p) {
    const uint4* q = reinterpret_cast<const uint4*>(p);
    uint4 a = __ldg(q), b = __ldg(q + 1);
    Fr r;
    r.v[0] = a.x; r.v[1] = a.y; r.v[2] = a.z; r.v[3] = a.w;
    r.v[4] = b.x; r.v[5] = b.y; r.v[6] = b.z; r.v[7] = b.w;
    return r;
}
__device__ __forceinline__ void fr_store(Fr* p, const Fr& x) {
    uint4* q = reinterpret_cast<uint4*>(p);
    q[0] = make_uint4(x.v[0], x.v[1], x.v[2], x.v[3]);
    q[1] = make_uint4(x.v[4], x.v[5], x.v[6], x.v[7]);
}

// r = a - p if a >= p else a   (a < 2p)
__device__ __forceinline__ Fr fr_csub_p(const Fr& a) {
    Fr d;
    uint32_t borrow;
    asm("sub.cc.u32 %0, %9, %17;\n\t"
        "subc.cc.u32 %1, %10, %18;\n\t"
        "subc.cc.u32 %2, %11, %19;\n\t"
        "subc.cc.u32 %3, %12, %20;\n\t"
        "subc.cc.u32 %4, %13, %21;\n\t"
        "subc.cc.u32 %5, %14, %22;\n\t"
        "subc.cc.u32 %6, %15, %23;\n\t"
        "subc.cc.u32 %7, %16, %24;\n\t"
        "subc.u32 %8, 0, 0;"
        : "=r"(d.v[0]), "=r"(d.v[1]), "=r"(d.v[2]), "=r"(d.v[3]), "=r"(d.v[4]), "=r"(d.v[5]), "=r"(d.v[6]),
          "=r"(d.v[7]), "=r"(borrow)
        : "r"(a.v[0]), "r"(a.v[1]), "r"(a.v[2]), "r"(a.v[3]), "r"(a.v[4]), "r"(a.v[5]), "r"(a.v[6]), "r"(a.v[7]),
          "r"(FR_P.v[0]), "r"(FR_P.v[1]), "r"(FR_P.v[2]), "r"(FR_P.v[3]), "r"(FR_P.v[4]), "r"(FR_P.v[5]),
          "r"(FR_P.v[6]), "r"(FR_P.v[7]));
    Fr r;
#pragma unroll
    for (int i = 0; i < 8; i++) r.v[i] = borrow ? a.v[i] : d.v[i];
    return r;
}
// a + b mod p  (a, b < p; the sum stays below 2^256)
__device__ __forceinline__ Fr fr_add(const Fr& a, const Fr& b) {
    Fr s;
    asm("add.cc.u32 %0, %8, %16;\n\t"
        "addc.cc.u32 %1, %9, %17;\n\t"
        "addc.cc.u32 %2, %10, %18;\n\t"
        "addc.cc.u32 %3, %11, %19;\n\t"
        "addc.cc.u32 %4, %12, %20;\n\t"
        "addc.cc.u32 %5, %13, %21;\n\t"
        "addc.cc.u32 %6, %14, %22;\n\t"
        "addc.u32 %7, %15, %23;"
        : "=r"(s.v[0]), "=r"(s.v[1]), "=r"(s.v[2]), "=r"(s.v[3]), "=r"(s.v[4]), "=r"(s.v[5]), "=r"(s.v[6]),
          "=r"(s.v[7])
        : "r"(a.v[0]), "r"(a.v[1]), "r"(a.v[2]), "r"(a.v[3]), "r"(a.v[4]), "r"(a.v[5]), "r"(a.v[6]), "r"(a.v[7]),
          "r"(b.v[0]), "r"(b.v[1]), "r"(b.v[2]), "r"(b.v[3]), "r"(b.v[4]), "r"(b.v[5]), "r"(b.v[6]), "r"(b.v[7]));
    return fr_csub_p(s);
}
// a - b mod p
__device__ __forceinline__ Fr fr_sub(const Fr& a, const Fr& b) {
    Fr d;
    uint32_t borrow;
    asm("sub.cc.u32 %0, %9, %17;\n\t"
        "subc.cc.u32 %1, %10, %18;\n\t"
        "subc.cc.u32 %2, %11, %19;\n\t"
        "subc.cc.u32 %3, %12, %20;\n\t"
        "subc.cc.u32 %4, %13, %21;\n\t"
        "subc.cc.u32 %5, %14, %22;\n\t"
        "subc.cc.u32 %6, %15, %23;\n\t"
        "subc.cc.u32 %7, %16, %24;\n\t"
        "subc.u32 %8, 0, 0;"
        : "=r"(d.v[0]), "=r"(d.v[1]), "=r"(d.v[2]), "=r"(d.v[3]), "=r"(d.v[4]), "=r"(d.v[5]), "=r"(d.v[6]),
          "=r"(d.v[7]), "=r"(borrow)
        : "r"(a.v[0]), "r"(a.v[1]), "r"(a.v[2]), "r"(a.v[3]), "r"(a.v[4]), "r"(a.v[5]), "r"(a.v[6]), "r"(a.v[7]),
          "r"(b.v[0]), "r"(b.v[1]), "r"(b.v[2]), "r"(b.v[3]), "r"(b.v[4]), "r"(b.v[5]), "r"(b.v[6]), "r"(b.v[7]));
    // borrow is 0xffffffff when a < b: add p back under that mask
    Fr r;
    asm("add.cc.u32 %0, %8, %16;\n\t"
        "addc.cc.u32 %1, %9, %17;\n\t"
        "addc.cc.u32 %2, %10, %18;\n\t"
        "addc.cc.u32 %3, %11, %19;\n\t"
        "addc.cc.u32 %4, %12, %20;\n\t"
        "addc.cc.u32 %5, %13, %21;\n\t"
        "addc.cc.u32 %6, %14, %22;\n\t"
        "addc.u32 %7, %15, %23;"
        : "=r"(r.v[0]), "=r"(r.v[1]), "=r"(r.v[2]), "=r"(r.v[3]), "=r"(r.v[4]), "=r"(r.v[5]), "=r"(r.v[6]),
          "=r"(r.v[7])
        : "r"(d.v[0]), "r"(d.v[1]), "r"(d.v[2]), "r"(d.v[3]), "r"(d.v[4]), "r"(d.v[5]), "r"(d.v[6]), "r"(d.v[7]),
          "r"(FR_P.v[0] & borrow), "r"(FR_P.v[1] & borrow), "r"(FR_P.v[2] & borrow), "r"(FR_P.v[3] & borrow),
          "r"(FR_P.v[4] & borrow), "r"(FR_P.v[5] & borrow), "r"(FR_P.v[6] & borrow), "r"(FR_P.v[7] & borrow));
    return r;
}

// t[0..9] += x[0..7] * y.  Two carry-propagating additions: the products of the even limbs occupy limb pairs
// (0,1) (2,3) (4,5) (6,7), those of the odd limbs (1,2) (3,4) (5,6) (7,8); inside a chain every low half is
// followed by the high half of the same product, the shape that maps to one wide multiply-add with carry.
__device__ __forceinline__ void fr_row_mad(uint32_t (&t)[10], const uint32_t (&x)[8], uint32_t y) {
    asm("mad.lo.cc.u32 %0, %10, %18, %0;\n\t"
        "madc.hi.cc.u32 %1, %10, %18, %1;\n\t"
        "madc.lo.cc.u32 %2, %12, %18, %2;\n\t"
        "madc.hi.cc.u32 %3, %12, %18, %3;\n\t"
        "madc.lo.cc.u32 %4, %14, %18, %4;\n\t"
        "madc.hi.cc.u32 %5, %14, %18, %5;\n\t"
        "madc.lo.cc.u32 %6, %16, %18, %6;\n\t"
        "madc.hi.cc.u32 %7, %16, %18, %7;\n\t"
        "addc.cc.u32 %8, %8, 0;\n\t"
        "addc.u32 %9, %9, 0;\n\t"
        "mad.lo.cc.u32 %1, %11, %18, %1;\n\t"
        "madc.hi.cc.u32 %2, %11, %18, %2;\n\t"
        "madc.lo.cc.u32 %3, %13, %18, %3;\n\t"
        "madc.hi.cc.u32 %4, %13, %18, %4;\n\t"
        "madc.lo.cc.u32 %5, %15, %18, %5;\n\t"
        "madc.hi.cc.u32 %6, %15, %18, %6;\n\t"
        "madc.lo.cc.u32 %7, %17, %18, %7;\n\t"
        "madc.hi.cc.u32 %8, %17, %18, %8;\n\t"
        "addc.u32 %9, %9, 0;"
        : "+r"(t[0]), "+r"(t[1]), "+r"(t[2]), "+r"(t[3]), "+r"(t[4]), "+r"(t[5]), "+r"(t[6]), "+r"(t[7]),
          "+r"(t[8]), "+r"(t[9])
        : "r"(x[0]), "r"(x[1]), "r"(x[2]), "r"(x[3]), "r"(x[4]), "r"(x[5]), "r"(x[6]), "r"(x[7]), "r"(y));
}

// Montgomery product a*b/R mod p, canonical result (a, b < p)
__device__ __forceinline__ Fr fr_mmul(const Fr& a, const Fr& b) {
    uint32_t t[10];
#pragma unroll
    for (int i = 0; i < 10; i++) t[i] = 0;
    uint32_t pl[8];
#pragma unroll
    for (int i = 0; i < 8; i++) pl[i] = FR_P.v[i];
#pragma unroll
    for (int i = 0; i < 8; i++) {
        fr_row_mad(t, a.v, b.v[i]);
        const uint32_t m = 0u - t[0];  // t[0] * 0xffffffff mod 2^32
        fr_row_mad(t, pl, m);          // now t[0] == 0
#pragma unroll
        for (int j = 0; j < 9; j++) t[j] = t[j + 1];
        t[9] = 0;
    }
    Fr r;
#pragma unroll
    for (int i = 0; i < 8; i++) r.v[i] = t[i];
    return fr_csub_p(r);  // t < 2p and 2p < 2^256, so t[8] == 0 here
}
// plain x -> x*R (Montgomery form) and back
__device__ __forceinline__ Fr fr_to_mont(const Fr& x) { return fr_mmul(x, FR_RPOW[1]); }
__device__ __forceinline__ Fr fr_from_mont(const Fr& x) {
    Fr one = fr_zero();
    one.v[0] = 1;
    return fr_mmul(x, one);
}
// a + x*(b - a) with x in Montgomery form, a and b plain: plain result
__device__ __forceinline__ Fr fr_lerp(const Fr& a, const Fr& b, const Fr& x_mont) {
    return fr_add(a, fr_mmul(x_mont, fr_sub(b, a)));
}
__device__ __forceinline__ Fr fr_shfl_down(const Fr& x, int d) {
    Fr r;
#pragma unroll
    for (int i = 0; i < 8; i++) r.v[i] = __shfl_down_sync(0xffffffffu, x.v[i], d);
    return r;
}
__device__ __forceinline__ bool fr_is_zero(const Fr& x) {
    uint32_t o = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) o |= x.v[i];
    return o == 0;
}
// Montgomery-form inverse by Fermat: x^(p-2)
static __device__ __noinline__ Fr fr_inv_mont(const Fr& x) {
    // p - 2, little-endian limbs
    const uint32_t e[8] = {0xffffffffu, 0xfffffffeu, 0xfffe5bfeu, 0x53bda402u, 0x09a1d805u, 0x3339d808u, 0x299d7d48u, 0x73eda753u};
    Fr r = FR_RPOW[0];   // 1 in Montgomery form
    for (int limb = 7; limb >= 0; limb--)
        for (int b = 31; b >= 0; b--) {
            r = fr_mmul(r, r);
            if ((e[limb] >> b) & 1u) r = fr_mmul(r, x);
        }
    return r;
}
#endif  // __CUDACC__

}  // namespace zkh
