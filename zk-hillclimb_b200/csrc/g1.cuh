// BLS12-381 base field and G1 points for sm_100a, in the reference's representation (zkllm-src/bls12-381.cuh:222-225, :424-433):
// an Fp element is twelve 32-bit limbs, little endian, holding a * 2^384 mod p (Montgomery form, always fully reduced); a G1 point
// is Jacobian (X, Y, Z), 144 bytes, the point at infinity (0, 1, 0).  Because every result is the canonical residue, any correct
// arithmetic gives the reference's bytes; what has to match the reference is the FORMULA of each group operation (a Jacobian
// triple is one of many representatives of its point): add-2007-bl with its early returns, dbl-2009-l
// (zkllm-src/bls12-381.cu:1361-1386, :1429-1464).
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace zkh {

struct __align__(16) Fp { uint32_t v[12]; };
struct __align__(16) G1 { Fp x, y, z; };

#define ZKH_FP_P_INIT  {{4294945451u, 3120496639u, 2975072255u, 514588670u, 4138792484u, 1731252896u, 4085584575u, 1685539716u, 1129032919u, 1260103606u, 964683418u, 436277738u}}
#define ZKH_FP_ONE_INIT {{196605u, 1980301312u, 3289120770u, 3958636555u, 1405573306u, 1598593111u, 1884444485u, 2010011731u, 2723605613u, 1543969431u, 4202751123u, 368467651u}}
constexpr uint32_t ZKH_FP_INV = 4294770685u;      // -1 / p mod 2^32

#ifdef __CUDACC__
static __device__ __constant__ Fp FP_P = ZKH_FP_P_INIT;
static __device__ __constant__ Fp FP_ONE = ZKH_FP_ONE_INIT;      // 2^384 mod p

__device__ __forceinline__ bool fp_is_zero(const Fp& a) {
    uint32_t o = 0;
#pragma unroll
    for (int i = 0; i < 12; i++) o |= a.v[i];
    return o == 0;
}
__device__ __forceinline__ bool fp_eq(const Fp& a, const Fp& b) {
    uint32_t o = 0;
#pragma unroll
    for (int i = 0; i < 12; i++) o |= a.v[i] ^ b.v[i];
    return o == 0;
}
__device__ __forceinline__ bool fp_gte_p(const Fp& a) {
#pragma unroll
    for (int i = 11; i >= 0; i--) {
        if (a.v[i] > FP_P.v[i]) return true;
        if (a.v[i] < FP_P.v[i]) return false;
    }
    return true;
}
__device__ __forceinline__ Fp fp_sub_p(const Fp& a) {
    Fp r;
    uint64_t br = 0;
#pragma unroll
    for (int i = 0; i < 12; i++) {
        const uint64_t d = (uint64_t)a.v[i] - FP_P.v[i] - br;
        r.v[i] = (uint32_t)d;
        br = (d >> 32) & 1;
    }
    return r;
}
__device__ __forceinline__ Fp fp_add(const Fp& a, const Fp& b) {
    Fp r;
    uint64_t c = 0;
#pragma unroll
    for (int i = 0; i < 12; i++) {
        c += (uint64_t)a.v[i] + b.v[i];
        r.v[i] = (uint32_t)c;
        c >>= 32;
    }
    return fp_gte_p(r) ? fp_sub_p(r) : r;          // p < 2^382: the sum of two residues fits 384 bits
}
__device__ __forceinline__ Fp fp_double(const Fp& a) { return fp_add(a, a); }
__device__ __forceinline__ Fp fp_sub(const Fp& a, const Fp& b) {
    Fp r;
    uint64_t br = 0;
#pragma unroll
    for (int i = 0; i < 12; i++) {
        const uint64_t d = (uint64_t)a.v[i] - b.v[i] - br;
        r.v[i] = (uint32_t)d;
        br = (d >> 32) & 1;
    }
    if (br) {
        uint64_t c = 0;
#pragma unroll
        for (int i = 0; i < 12; i++) {
            c += (uint64_t)r.v[i] + FP_P.v[i];
            r.v[i] = (uint32_t)c;
            c >>= 32;
        }
    }
    return r;
}
// t[0..13] += x[0..11] * y.  Two carry chains: the products of the even limbs occupy limb pairs (0,1) .. (10,11), those of the odd
// limbs (1,2) .. (11,12); inside a chain every low half is followed by the high half of the same product.
__device__ __forceinline__ void fp_row_mad(uint32_t (&t)[14], const uint32_t (&x)[12], uint32_t y) {
    asm(
        "mad.lo.cc.u32 %0, %14, %26, %0;\n\t"
        "madc.hi.cc.u32 %1, %14, %26, %1;\n\t"
        "madc.lo.cc.u32 %2, %16, %26, %2;\n\t"
        "madc.hi.cc.u32 %3, %16, %26, %3;\n\t"
        "madc.lo.cc.u32 %4, %18, %26, %4;\n\t"
        "madc.hi.cc.u32 %5, %18, %26, %5;\n\t"
        "madc.lo.cc.u32 %6, %20, %26, %6;\n\t"
        "madc.hi.cc.u32 %7, %20, %26, %7;\n\t"
        "madc.lo.cc.u32 %8, %22, %26, %8;\n\t"
        "madc.hi.cc.u32 %9, %22, %26, %9;\n\t"
        "madc.lo.cc.u32 %10, %24, %26, %10;\n\t"
        "madc.hi.cc.u32 %11, %24, %26, %11;\n\t"
        "addc.cc.u32 %12, %12, 0;\n\t"
        "addc.u32 %13, %13, 0;\n\t"
        "mad.lo.cc.u32 %1, %15, %26, %1;\n\t"
        "madc.hi.cc.u32 %2, %15, %26, %2;\n\t"
        "madc.lo.cc.u32 %3, %17, %26, %3;\n\t"
        "madc.hi.cc.u32 %4, %17, %26, %4;\n\t"
        "madc.lo.cc.u32 %5, %19, %26, %5;\n\t"
        "madc.hi.cc.u32 %6, %19, %26, %6;\n\t"
        "madc.lo.cc.u32 %7, %21, %26, %7;\n\t"
        "madc.hi.cc.u32 %8, %21, %26, %8;\n\t"
        "madc.lo.cc.u32 %9, %23, %26, %9;\n\t"
        "madc.hi.cc.u32 %10, %23, %26, %10;\n\t"
        "madc.lo.cc.u32 %11, %25, %26, %11;\n\t"
        "madc.hi.cc.u32 %12, %25, %26, %12;\n\t"
        "addc.u32 %13, %13, 0;"
        : "+r"(t[0]), "+r"(t[1]), "+r"(t[2]), "+r"(t[3]), "+r"(t[4]), "+r"(t[5]), "+r"(t[6]), "+r"(t[7]), "+r"(t[8]), "+r"(t[9]), "+r"(t[10]), "+r"(t[11]), "+r"(t[12]), "+r"(t[13])
        : "r"(x[0]), "r"(x[1]), "r"(x[2]), "r"(x[3]), "r"(x[4]), "r"(x[5]), "r"(x[6]), "r"(x[7]), "r"(x[8]), "r"(x[9]), "r"(x[10]), "r"(x[11]), "r"(y));
}
// Montgomery product a * b / 2^384 mod p, operand scanning with the reduction interleaved
static __device__ __noinline__ Fp fp_mul(const Fp& a, const Fp& b) {
    uint32_t t[14];
#pragma unroll
    for (int i = 0; i < 14; i++) t[i] = 0;
    uint32_t pl[12], av[12];
#pragma unroll
    for (int i = 0; i < 12; i++) { pl[i] = FP_P.v[i]; av[i] = a.v[i]; }
#pragma unroll
    for (int i = 0; i < 12; i++) {
        fp_row_mad(t, av, b.v[i]);
        const uint32_t m = t[0] * ZKH_FP_INV;
        fp_row_mad(t, pl, m);              // now t[0] == 0
#pragma unroll
        for (int j = 0; j < 13; j++) t[j] = t[j + 1];
        t[13] = 0;
    }
    Fp r;
#pragma unroll
    for (int i = 0; i < 12; i++) r.v[i] = t[i];
    return fp_gte_p(r) ? fp_sub_p(r) : r;  // t < 2p < 2^383: t[12] == 0 here
}
__device__ __forceinline__ Fp fp_sqr(const Fp& a) { return fp_mul(a, a); }
// two independent products in one pass: r0 = a0 * b0, r1 = a1 * b1.  A Montgomery product is one long dependent chain of
// multiply-adds (each waits for the carry of the one before); two of them side by side give the scheduler a second chain
// to issue from while the first waits.
#ifdef ZKH_FP_PAIR_AS_SINGLE
// (a translation unit whose kernels run at high occupancy does better with two plain products: fewer live registers)
__device__ __forceinline__ void fp_mul2(Fp& r0, Fp& r1, const Fp& a0, const Fp& b0, const Fp& a1, const Fp& b1) {
    const Fp x = fp_mul(a0, b0), y = fp_mul(a1, b1);
    r0 = x;
    r1 = y;
}
#else
static __device__ __noinline__ void fp_mul2(Fp& r0, Fp& r1, const Fp& a0, const Fp& b0, const Fp& a1, const Fp& b1) {
    uint32_t t[14], u[14];
#pragma unroll
    for (int i = 0; i < 14; i++) { t[i] = 0; u[i] = 0; }
    uint32_t pl[12], av[12], cv[12];
#pragma unroll
    for (int i = 0; i < 12; i++) { pl[i] = FP_P.v[i]; av[i] = a0.v[i]; cv[i] = a1.v[i]; }
#pragma unroll
    for (int i = 0; i < 12; i++) {
        fp_row_mad(t, av, b0.v[i]);
        fp_row_mad(u, cv, b1.v[i]);
        const uint32_t m = t[0] * ZKH_FP_INV, k = u[0] * ZKH_FP_INV;
        fp_row_mad(t, pl, m);
        fp_row_mad(u, pl, k);
#pragma unroll
        for (int j = 0; j < 13; j++) { t[j] = t[j + 1]; u[j] = u[j + 1]; }
        t[13] = 0;
        u[13] = 0;
    }
    Fp x, y;
#pragma unroll
    for (int i = 0; i < 12; i++) { x.v[i] = t[i]; y.v[i] = u[i]; }
    r0 = fp_gte_p(x) ? fp_sub_p(x) : x;
    r1 = fp_gte_p(y) ? fp_sub_p(y) : y;
}
#endif

__device__ __forceinline__ G1 g1_zero() {
    G1 r;
#pragma unroll
    for (int i = 0; i < 12; i++) { r.x.v[i] = 0; r.z.v[i] = 0; }
    r.y = FP_ONE;
    return r;
}
// dbl-2009-l (zkllm-src/bls12-381.cu:1361-1386).  Operands by reference, the result built in a local of its own.
static __device__ __noinline__ G1 g1_double(const G1& p) {
    G1 r;
    if (fp_is_zero(p.z)) {
        r = p;
        return r;
    }
    Fp a, b, c, d, f, yz, t;
    fp_mul2(a, b, p.x, p.x, p.y, p.y);                 // A = X1^2, B = Y1^2
    const Fp xb = fp_add(p.x, b);
    fp_mul2(c, d, b, b, xb, xb);                       // C = B^2, (X1 + B)^2
    d = fp_double(fp_sub(fp_sub(d, a), c));            // D = 2 ((X1 + B)^2 - A - C)
    const Fp e = fp_add(fp_double(a), a);              // E = 3 A
    fp_mul2(f, yz, e, e, p.y, p.z);                    // F = E^2, Y1 Z1
    r.z = fp_double(yz);
    r.x = fp_sub(fp_sub(f, d), d);
    c = fp_double(fp_double(fp_double(c)));
    t = fp_mul(fp_sub(d, r.x), e);
    r.y = fp_sub(t, c);
    return r;
}
// add-2007-bl with the reference's early returns (zkllm-src/bls12-381.cu:1429-1464)
static __device__ __noinline__ G1 g1_add(const G1& a, const G1& b) {
    G1 r;
    if (fp_is_zero(a.z)) {
        r = b;
        return r;
    }
    if (fp_is_zero(b.z)) {
        r = a;
        return r;
    }
    Fp z1z1, z2z2, u1, u2, s1, s2, ii, zz, jj, v, r2, sj, t1, t2;
    fp_mul2(z1z1, z2z2, a.z, a.z, b.z, b.z);
    fp_mul2(u1, u2, a.x, z2z2, b.x, z1z1);             // U1 = X1 Z2Z2, U2 = X2 Z1Z1
    fp_mul2(t1, t2, a.y, b.z, b.y, a.z);
    fp_mul2(s1, s2, t1, z2z2, t2, z1z1);               // S1 = Y1 Z2 Z2Z2, S2 = Y2 Z1 Z1Z1
    if (fp_eq(u1, u2) && fp_eq(s1, s2)) return g1_double(a);
    const Fp h = fp_sub(u2, u1), h2 = fp_double(h), zs = fp_add(a.z, b.z);
    fp_mul2(ii, zz, h2, h2, zs, zs);                   // I = (2H)^2, (Z1 + Z2)^2
    fp_mul2(jj, v, h, ii, u1, ii);                     // J = H I, V = U1 I
    const Fp rr = fp_double(fp_sub(s2, s1));           // r = 2 (S2 - S1)
    fp_mul2(r2, sj, rr, rr, s1, jj);
    r.x = fp_sub(fp_sub(fp_sub(r2, jj), v), v);        // X3 = r^2 - J - 2 V
    fp_mul2(t1, t2, fp_sub(v, r.x), rr, fp_sub(fp_sub(zz, z1z1), z2z2), h);
    r.y = fp_sub(t1, fp_double(sj));                   // Y3 = r (V - X3) - 2 S1 J
    r.z = t2;                                          // Z3 = ((Z1 + Z2)^2 - Z1Z1 - Z2Z2) H
    return r;
}
__device__ __forceinline__ void fp_load(Fp& c, const uint4* q) {
#pragma unroll
    for (int j = 0; j < 3; j++) {
        const uint4 t = __ldg(q + j);
        c.v[4 * j] = t.x; c.v[4 * j + 1] = t.y; c.v[4 * j + 2] = t.z; c.v[4 * j + 3] = t.w;
    }
}
__device__ __forceinline__ G1 g1_load(const G1* p) {
    G1 r;
    const uint4* q = reinterpret_cast<const uint4*>(p);
    fp_load(r.x, q);
    fp_load(r.y, q + 3);
    fp_load(r.z, q + 6);
    return r;
}
__device__ __forceinline__ void g1_store(G1* p, const G1& v) {
    uint4* q = reinterpret_cast<uint4*>(p);
    const uint32_t* w = v.x.v;                  // x, y, z are contiguous: 36 limbs
#pragma unroll
    for (int j = 0; j < 9; j++) q[j] = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
}
// -P: (X, 0 - Y, Z), the reference's G1Jacobian_minus (zkllm-src/g1-tensor.cu:11-21)
__device__ __forceinline__ G1 g1_neg(const G1& p) {
    G1 r = p;
    Fp z;
#pragma unroll
    for (int i = 0; i < 12; i++) z.v[i] = 0;
    r.y = fp_sub(z, p.y);
    return r;
}

// ------------------------------------------------------------------ group law on four lanes
// The kernels that walk one long chain of additions or doublings per point are bound by the latency of a single thread's
// 384-bit products, with most of the GPU idle.  Here a point operation runs on four neighbouring lanes (a quad): every
// lane holds the same operands and ends with the same result; in between the independent products of the formula run one
// per lane and are passed round with shuffles.  An addition is five products deep instead of sixteen, a doubling three
// instead of seven.  Field results are canonical residues, so the triples equal those of g1_add / g1_double bit for bit.
// All four lanes of a quad must call together; qmask names them.
__device__ __forceinline__ uint32_t g1q_mask() { return 0xFu << ((threadIdx.x & 31u) & ~3u); }
__device__ __forceinline__ Fp fpq_from(const Fp& v, int src, uint32_t qmask) {
    Fp r;
#pragma unroll
    for (int i = 0; i < 12; i++) r.v[i] = __shfl_sync(qmask, v.v[i], src, 4);
    return r;
}
static __device__ __noinline__ G1 g1q_double(const G1& p, uint32_t qmask) {
    G1 r;
    if (fp_is_zero(p.z)) {
        r = p;
        return r;
    }
    const int ql = threadIdx.x & 3;
    // X^2 | Y^2 | Y Z
    Fp m = fp_mul(ql == 0 ? p.x : p.y, ql == 0 ? p.x : ql == 1 ? p.y : p.z);
    const Fp a = fpq_from(m, 0, qmask), b = fpq_from(m, 1, qmask), yz = fpq_from(m, 2, qmask);
    const Fp e = fp_add(fp_double(a), a), xb = fp_add(p.x, b);
    // B^2 | (X + B)^2 | E^2
    const Fp& o2 = ql == 0 ? b : ql == 1 ? xb : e;
    m = fp_mul(o2, o2);
    Fp c = fpq_from(m, 0, qmask);
    const Fp t = fpq_from(m, 1, qmask), f = fpq_from(m, 2, qmask);
    const Fp d = fp_double(fp_sub(fp_sub(t, a), c));
    r.z = fp_double(yz);
    r.x = fp_sub(fp_sub(f, d), d);
    c = fp_double(fp_double(fp_double(c)));
    r.y = fp_sub(fp_mul(fp_sub(d, r.x), e), c);      // every lane: the last product has no sibling
    return r;
}
static __device__ __noinline__ G1 g1q_add(const G1& a, const G1& b, uint32_t qmask) {
    G1 r;
    if (fp_is_zero(a.z)) {
        r = b;
        return r;
    }
    if (fp_is_zero(b.z)) {
        r = a;
        return r;
    }
    const int ql = threadIdx.x & 3;
    // Z1^2 | Z2^2 | Y1 Z2 | Y2 Z1
    Fp m = fp_mul(ql == 0 ? a.z : ql == 1 ? b.z : ql == 2 ? a.y : b.y, (ql == 0 || ql == 3) ? a.z : b.z);
    const Fp z1z1 = fpq_from(m, 0, qmask), z2z2 = fpq_from(m, 1, qmask);
    // U1 = X1 Z2Z2 | U2 = X2 Z1Z1 | S1 = Y1 Z2 Z2Z2 | S2 = Y2 Z1 Z1Z1
    m = fp_mul(ql == 0 ? a.x : ql == 1 ? b.x : m, (ql == 0 || ql == 2) ? z2z2 : z1z1);
    const Fp u1 = fpq_from(m, 0, qmask), u2 = fpq_from(m, 1, qmask), s1 = fpq_from(m, 2, qmask), s2 = fpq_from(m, 3, qmask);
    if (fp_eq(u1, u2) && fp_eq(s1, s2)) return g1q_double(a, qmask);
    const Fp h = fp_sub(u2, u1), h2 = fp_double(h), zs = fp_add(a.z, b.z), rr = fp_double(fp_sub(s2, s1));
    // I = (2H)^2 | r^2 | (Z1 + Z2)^2
    const Fp& o3 = ql == 0 ? h2 : ql == 1 ? rr : zs;
    m = fp_mul(o3, o3);
    const Fp ii = fpq_from(m, 0, qmask), r2 = fpq_from(m, 1, qmask);
    // J = H I | V = U1 I | Z3 = ((Z1 + Z2)^2 - Z1Z1 - Z2Z2) H
    const Fp zz = fp_sub(fp_sub(m, z1z1), z2z2);      // meaningful on lane 2
    m = fp_mul(ql == 0 ? h : ql == 1 ? u1 : zz, ql == 2 ? h : ii);
    const Fp jj = fpq_from(m, 0, qmask), v = fpq_from(m, 1, qmask);
    r.z = fpq_from(m, 2, qmask);
    r.x = fp_sub(fp_sub(fp_sub(r2, jj), v), v);        // X3 = r^2 - J - 2 V
    // S1 J | r (V - X3)
    const Fp vx = fp_sub(v, r.x);
    m = fp_mul(ql == 0 ? s1 : vx, ql == 0 ? jj : rr);
    const Fp sj = fpq_from(m, 0, qmask), t1 = fpq_from(m, 1, qmask);
    r.y = fp_sub(t1, fp_double(sj));                   // Y3 = r (V - X3) - 2 S1 J
    return r;
}
#endif  // __CUDACC__

}  // namespace zkh
