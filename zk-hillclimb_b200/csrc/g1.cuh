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
// Montgomery product a * b / 2^384 mod p, operand scanning with the reduction interleaved (CIOS)
__device__ __noinline__ Fp fp_mul(const Fp& a, const Fp& b) {
    uint32_t t[14];
#pragma unroll
    for (int i = 0; i < 14; i++) t[i] = 0;
#pragma unroll
    for (int i = 0; i < 12; i++) {
        uint64_t c = 0;
#pragma unroll
        for (int j = 0; j < 12; j++) {
            c += (uint64_t)a.v[j] * b.v[i] + t[j];
            t[j] = (uint32_t)c;
            c >>= 32;
        }
        c += t[12];
        t[12] = (uint32_t)c;
        t[13] = (uint32_t)(c >> 32);
        const uint32_t m = t[0] * ZKH_FP_INV;
        c = (uint64_t)m * FP_P.v[0] + t[0];
        c >>= 32;
#pragma unroll
        for (int j = 1; j < 12; j++) {
            c += (uint64_t)m * FP_P.v[j] + t[j];
            t[j - 1] = (uint32_t)c;
            c >>= 32;
        }
        c += t[12];
        t[11] = (uint32_t)c;
        t[12] = t[13] + (uint32_t)(c >> 32);
    }
    Fp r;
#pragma unroll
    for (int i = 0; i < 12; i++) r.v[i] = t[i];
    return fp_gte_p(r) ? fp_sub_p(r) : r;
}
__device__ __forceinline__ Fp fp_sqr(const Fp& a) { return fp_mul(a, a); }

__device__ __forceinline__ G1 g1_zero() {
    G1 r;
#pragma unroll
    for (int i = 0; i < 12; i++) { r.x.v[i] = 0; r.z.v[i] = 0; }
    r.y = FP_ONE;
    return r;
}
// dbl-2009-l (zkllm-src/bls12-381.cu:1361-1386).  Operands by reference, the result built in a local of its own.
__device__ __noinline__ G1 g1_double(const G1& p) {
    G1 r;
    if (fp_is_zero(p.z)) {
        r = p;
        return r;
    }
    const Fp a = fp_sqr(p.x), b = fp_sqr(p.y);
    Fp c = fp_sqr(b);
    Fp d = fp_sqr(fp_add(p.x, b));
    d = fp_double(fp_sub(fp_sub(d, a), c));
    const Fp e = fp_add(fp_double(a), a), f = fp_sqr(e);
    r.z = fp_double(fp_mul(p.y, p.z));
    r.x = fp_sub(fp_sub(f, d), d);
    c = fp_double(fp_double(fp_double(c)));
    r.y = fp_sub(fp_mul(fp_sub(d, r.x), e), c);
    return r;
}
// add-2007-bl with the reference's early returns (zkllm-src/bls12-381.cu:1429-1464)
__device__ __noinline__ G1 g1_add(const G1& a, const G1& b) {
    G1 r;
    if (fp_is_zero(a.z)) {
        r = b;
        return r;
    }
    if (fp_is_zero(b.z)) {
        r = a;
        return r;
    }
    const Fp z1z1 = fp_sqr(a.z), z2z2 = fp_sqr(b.z);
    const Fp u1 = fp_mul(a.x, z2z2), u2 = fp_mul(b.x, z1z1);
    Fp s1 = fp_mul(fp_mul(a.y, b.z), z2z2);
    const Fp s2 = fp_mul(fp_mul(b.y, a.z), z1z1);
    if (fp_eq(u1, u2) && fp_eq(s1, s2)) return g1_double(a);
    const Fp h = fp_sub(u2, u1);
    const Fp i = fp_sqr(fp_double(h));
    const Fp j = fp_mul(h, i);
    const Fp rr = fp_double(fp_sub(s2, s1));
    const Fp v = fp_mul(u1, i);
    r.x = fp_sub(fp_sub(fp_sub(fp_sqr(rr), j), v), v);
    r.y = fp_mul(fp_sub(v, r.x), rr);
    s1 = fp_double(fp_mul(s1, j));
    r.y = fp_sub(r.y, s1);
    r.z = fp_sqr(fp_add(a.z, b.z));
    r.z = fp_mul(fp_sub(fp_sub(r.z, z1z1), z2z2), h);
    return r;
}
#endif  // __CUDACC__

}  // namespace zkh
