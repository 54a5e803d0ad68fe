// Constraint summands of the fp8 ("Hawkeye") matmul gadget, as device functors for the wide
// sumcheck engine.  Each is an eq-weighted random linear combination of per-row constraints
// (degree <= 4 in the round variable); the column order and the constraint order are the
// reference's (zkllm-src/p3_hawkeye.cuh:87-101 column enums, :850-1010 constraint functions),
// because both are part of the proof statement.
//
// A functor exposes NC (columns), NLAM (random coefficients) and
//   eval(v, lam) = F(v[0..NC), lam[0..NLAM))   as a canonical field element.
// The weighted sum over constraints is accumulated lazily (one reduction per evaluation).
#pragma once
#include "gl.cuh"

namespace zkh {

// sum_j lam[j] * r_j with one modular reduction at the end.  PART / NP: only the constraints j = PART (mod NP) are
// accumulated (j is a compile-time value in the straight-line constraint lists below, so the others, and the column
// reads only they need, disappear from the code): the summand is linear in the weighted sum, which lets NP warps share
// one row, each evaluating its own share of the constraints.
template <int PART = 0, int NP = 1>
struct RlcT {
    Acc192 a;
    const gl_t* lam;
    int j;
    __device__ __forceinline__ explicit RlcT(const gl_t* l) : lam(l), j(0) { a.clear(); }
    __device__ __forceinline__ void push(gl_t r) {
        if (j % NP == PART) a.add_prod(lam[j], r);
        j++;
    }
    __device__ __forceinline__ gl_t weighted(gl_t e) { return gl_mul(e, a.reduce()); }
};
using Rlc = RlcT<0, 1>;
__device__ __forceinline__ gl_t hw_bool(gl_t x) { return gl_sub(gl_mul(x, x), x); }          // x^2 - x
__device__ __forceinline__ gl_t hw_or(gl_t a, gl_t b) { return gl_sub(gl_add(a, b), gl_mul(a, b)); }
__device__ __forceinline__ gl_t hw_xor(gl_t a, gl_t b) { return gl_sub(gl_add(a, b), gl_mul(gl_dbl(a), b)); }
__device__ __forceinline__ gl_t hw_sgn(gl_t s) { return gl_sub(1, gl_dbl(s)); }              // 1 - 2s
__device__ __forceinline__ gl_t hw_not(gl_t z) { return gl_sub(1, z); }

template <int F> struct WFn;

// ---- per-product alignment: [E | eb mag sg pr sh pw q r al sel | gmax]
template <> struct WFn<ZKH_F_HW_DP> {
    static constexpr int NC = 12, NLAM = 6;
    enum { EB = 1, MAG, SG, PR, SH, PW, Q, R, AL, SEL, GMAX };
    static __device__ __forceinline__ gl_t eval(const gl_t* v, const gl_t* lam) {
        Rlc c(lam);
        c.push(gl_sub(gl_add(gl_mul(v[Q], v[PW]), v[R]), v[MAG]));                  // q*pw + r = mag
        c.push(gl_sub(v[AL], gl_mul(gl_mul(v[PR], v[Q]), hw_sgn(v[SG]))));          // al = pr*q*(+-1)
        c.push(gl_mul(v[PR], gl_sub(gl_add(v[SH], gl_add(v[EB], 127)), v[GMAX])));  // shift = gmax - eb - 127
        c.push(gl_mul(v[SEL], v[SH]));                                              // selected => shift 0
        c.push(hw_bool(v[SEL]));
        c.push(gl_mul(v[SEL], hw_not(v[PR])));                                      // selected => present
        return c.weighted(v[0]);
    }
};

// ---- per-group accumulate / normalise: [E | 29 group columns]
template <> struct WFn<ZKH_F_HW_DG> {
    static constexpr int NC = 30, NLAM = 18;
    enum { ASIG = 1, BEXP, ASGN, AZ, AINV, ABASE, ALO, ASH, APW, AQ, AR, MAX, ASEL, CSUM, TSGN, TMAG, TZ, TINV,
           WD, PLO, PHI, PDN, PUP, NR, S14, U1H, U1L, U2H, U2L };
    template <int PART = 0, int NP = 1, class V = const gl_t*>
    static __device__ __forceinline__ gl_t eval(const V& v, const gl_t* lam) {
        RlcT<PART, NP> c(lam);
        c.push(gl_mul(v[AZ], v[ASIG]));                                                            // 0
        c.push(gl_sub(gl_mul(v[ASIG], v[AINV]), hw_not(v[AZ])));                                   // 1
        c.push(gl_sub(v[ASIG], gl_add(gl_mul(v[ABASE], 1024), v[ALO])));                           // 2
        c.push(gl_add(gl_sub(v[ASH], v[MAX]), gl_mul(hw_not(v[AZ]), v[BEXP])));                    // 3
        c.push(gl_sub(gl_add(gl_mul(v[AQ], v[APW]), v[AR]), v[ABASE]));                            // 4
        c.push(gl_mul(v[ASEL], v[ASH]));                                                           // 5
        c.push(gl_sub(gl_sub(gl_mul(hw_sgn(v[TSGN]), v[TMAG]), v[CSUM]),
                      gl_mul(hw_sgn(v[ASGN]), v[AQ])));                                            // 6
        c.push(gl_mul(v[TZ], v[TMAG]));                                                            // 7
        c.push(gl_sub(gl_mul(v[TMAG], v[TINV]), hw_not(v[TZ])));                                   // 8
        c.push(gl_mul(v[TZ], v[TSGN]));                                                            // 9
        c.push(gl_sub(gl_sub(v[TMAG], v[PLO]), gl_add(gl_mul(v[U1H], 1024), v[U1L])));             // 10
        c.push(gl_sub(gl_sub(gl_sub(v[PHI], 1), v[TMAG]), gl_add(gl_mul(v[U2H], 1024), v[U2L])));  // 11
        c.push(gl_sub(gl_add(gl_mul(v[S14], v[PDN]), v[NR]), gl_mul(v[TMAG], v[PUP])));            // 12
        c.push(hw_bool(v[AZ]));
        c.push(hw_bool(v[ASEL]));
        c.push(hw_bool(v[TSGN]));
        c.push(hw_bool(v[TZ]));
        c.push(hw_bool(v[ASGN]));
        return c.weighted(v[0]);
    }
};

// ---- state chain between groups: [U V U0 | asig bexp asgn tz s14 gmax wd tsgn]
template <> struct WFn<ZKH_F_HW_CH> {
    static constexpr int NC = 11, NLAM = 6;
    static __device__ __forceinline__ gl_t eval(const gl_t* v, const gl_t* lam) {
        const gl_t live = hw_not(v[6]);
        const gl_t sig_out = gl_mul(gl_mul(live, v[7]), 1024);
        const gl_t exp_out = gl_mul(live, gl_sub(gl_add(v[8], v[9]), 14));
        Acc192 in, out, bnd;
        in.clear(); out.clear(); bnd.clear();
        in.add_prod(lam[0], v[3]);  in.add_prod(lam[1], v[4]);  in.add_prod(lam[2], v[5]);
        out.add_prod(lam[0], sig_out); out.add_prod(lam[1], exp_out); out.add_prod(lam[2], v[10]);
        bnd.add_prod(lam[3], v[3]); bnd.add_prod(lam[4], v[4]); bnd.add_prod(lam[5], v[5]);
        return gl_add(gl_sub(gl_mul(v[0], in.reduce()), gl_mul(v[1], out.reduce())), gl_mul(v[2], bnd.reduce()));
    }
};

// ---- group sum and attainment: [EQg al sel]
template <> struct WFn<ZKH_F_HW_GS> {
    static constexpr int NC = 3, NLAM = 2;
    static __device__ __forceinline__ gl_t eval(const gl_t* v, const gl_t* lam) {
        Rlc c(lam);
        c.push(v[1]);
        c.push(v[2]);
        return c.weighted(v[0]);
    }
};

// ---- per-row scale decomposition: [E | sbits ss se sei zs smh sml]
template <> struct WFn<ZKH_F_HW_DS> {
    static constexpr int NC = 8, NLAM = 6;
    static __device__ __forceinline__ gl_t eval(const gl_t* v, const gl_t* lam) {
        const gl_t sm = gl_add(gl_mul(v[6], 4096), v[7]);
        Rlc c(lam);
        c.push(gl_sub(v[1], gl_add(gl_add(gl_mul(v[2], 1ull << 31), gl_mul(v[3], 1ull << 23)), sm)));
        c.push(hw_bool(v[2]));
        c.push(hw_bool(v[5]));
        c.push(gl_mul(v[5], v[3]));
        c.push(gl_sub(gl_mul(v[3], v[4]), hw_not(v[5])));
        c.push(gl_mul(v[5], sm));
        return c.weighted(v[0]);
    }
};

// ---- per-output float pipeline (two fp32 multiplies, bf16 cast): [E | 46 output columns | 10 scale columns]
template <> struct WFn<ZKH_F_HW_DO> {
    static constexpr int NC = 57, NLAM = 49;
    enum { S14F = 1, BEXP, SGN, FZ, FINV,
           C1, REM1, RB1, RT1, RTI1, ZRT1, FH1, FL1, FLH1, L01, RUP1, C21, M1, E1, S1, Z1,
           C2, RB2, TH2, TL2, RTI2, ZRT2, FH2, FL2, FLH2, L02, RUP2, C22, M2, E2, S2, Z2,
           Q16, Q16H, L03, RB3, RT3, RTI3, ZRT3, RUP3, YB,
           XSS, XSE, XZS, XSMH, XSML, WSS, WSE, WZS, WSMH, WSML };
    template <int PART = 0, int NP = 1, class V = const gl_t*>
    static __device__ __forceinline__ gl_t eval(const V& v, const gl_t* lam) {
        constexpr gl_t B23 = 1ull << 23, B24 = 1ull << 24, B31 = 1ull << 31;
        const gl_t live1 = hw_not(v[Z1]), live2 = hw_not(v[Z2]);
        const gl_t manx = gl_add(B23, gl_add(gl_mul(v[XSMH], 4096), v[XSML]));
        const gl_t manw = gl_add(B23, gl_add(gl_mul(v[WSMH], 4096), v[WSML]));
        const gl_t up1 = gl_add(1, v[C1]), up2 = gl_add(1, v[C2]);
        const gl_t fr1 = gl_add(gl_mul(v[FH1], 4096), v[FL1]);
        const gl_t fr2 = gl_add(gl_mul(v[FH2], 4096), v[FL2]);
        const gl_t t2 = gl_add(gl_mul(v[TH2], 4096), v[TL2]);
        RlcT<PART, NP> c(lam);
        // accumulator value entering the output stage
        c.push(gl_mul(v[FZ], v[S14F]));                                                             // 0
        c.push(gl_sub(gl_mul(v[S14F], v[FINV]), hw_not(v[FZ])));                                    // 1
        c.push(hw_bool(v[FZ]));                                                                     // 2
        c.push(hw_bool(v[SGN]));                                                                    // 3
        c.push(gl_sub(v[Z1], hw_or(v[FZ], v[XZS])));                                                // 4
        c.push(gl_sub(v[Z2], hw_or(v[Z1], v[WZS])));                                                // 5
        // first multiply (by the activation scale)
        c.push(gl_mul(live1, gl_sub(gl_mul(v[S14F], manx),
                                    gl_add(gl_mul(gl_mul(fr1, 8192), up1), v[REM1]))));             // 6
        c.push(gl_sub(v[REM1], gl_add(gl_mul(gl_mul(v[RB1], 4096), up1), v[RT1])));                 // 7
        c.push(hw_bool(v[C1]));                                                                     // 8
        c.push(hw_bool(v[RB1]));                                                                    // 9
        c.push(hw_bool(v[C21]));                                                                    // 10
        c.push(hw_bool(v[L01]));                                                                    // 11
        c.push(hw_bool(v[ZRT1]));                                                                   // 12
        c.push(gl_sub(v[FL1], gl_add(gl_dbl(v[FLH1]), v[L01])));                                    // 13
        c.push(gl_mul(v[ZRT1], v[RT1]));                                                            // 14
        c.push(gl_sub(gl_mul(v[RT1], v[RTI1]), hw_not(v[ZRT1])));                                   // 15
        c.push(gl_sub(v[RUP1], gl_mul(v[RB1], gl_add(hw_not(v[ZRT1]), gl_mul(v[ZRT1], v[L01])))));  // 16
        c.push(gl_mul(v[C21], gl_sub(gl_add(fr1, v[RUP1]), B24)));                                  // 17
        c.push(gl_mul(live1, gl_add(gl_sub(gl_sub(v[M1], fr1), v[RUP1]), gl_mul(v[C21], B23))));    // 18
        c.push(gl_mul(v[Z1], gl_sub(v[M1], B23)));                                                  // 19
        c.push(gl_mul(live1, gl_sub(v[E1], gl_add(gl_sub(gl_add(v[BEXP], v[XSE]), 139),
                                                  gl_add(v[C1], v[C21])))));                        // 20
        c.push(gl_mul(v[Z1], gl_sub(v[E1], 1)));                                                    // 21
        c.push(gl_sub(v[S1], hw_xor(v[SGN], v[XSS])));                                              // 22
        // second multiply (by the weight scale)
        c.push(gl_mul(live2, gl_sub(gl_mul(v[M1], manw),
                                    gl_add(gl_add(gl_mul(gl_mul(fr2, B23), up2),
                                                  gl_mul(gl_mul(v[RB2], 1ull << 22), up2)), t2)))); // 23
        c.push(hw_bool(v[C2]));                                                                     // 24
        c.push(hw_bool(v[RB2]));                                                                    // 25
        c.push(hw_bool(v[C22]));                                                                    // 26
        c.push(hw_bool(v[L02]));                                                                    // 27
        c.push(hw_bool(v[ZRT2]));                                                                   // 28
        c.push(gl_sub(v[FL2], gl_add(gl_dbl(v[FLH2]), v[L02])));                                    // 29
        c.push(gl_mul(v[ZRT2], v[TH2]));                                                            // 30
        c.push(gl_mul(v[ZRT2], v[TL2]));                                                            // 31
        c.push(gl_sub(gl_mul(t2, v[RTI2]), hw_not(v[ZRT2])));                                       // 32
        c.push(gl_sub(v[RUP2], gl_mul(v[RB2], gl_add(hw_not(v[ZRT2]), gl_mul(v[ZRT2], v[L02])))));  // 33
        c.push(gl_mul(v[C22], gl_sub(gl_add(fr2, v[RUP2]), B24)));                                  // 34
        c.push(gl_mul(live2, gl_add(gl_sub(gl_sub(v[M2], fr2), v[RUP2]), gl_mul(v[C22], B23))));    // 35
        c.push(gl_mul(v[Z2], gl_sub(v[M2], B23)));                                                  // 36
        c.push(gl_mul(live2, gl_sub(v[E2], gl_add(gl_sub(gl_add(v[E1], v[WSE]), 127),
                                                  gl_add(v[C2], v[C22])))));                        // 37
        c.push(gl_mul(v[Z2], gl_sub(v[E2], 1)));                                                    // 38
        c.push(gl_sub(v[S2], hw_xor(v[S1], v[WSS])));                                               // 39
        // cast of the fp32 bit pattern to bf16 (round to nearest even)
        c.push(gl_sub(gl_add(gl_add(gl_mul(v[Q16], 65536), gl_mul(v[RB3], 32768)), v[RT3]),
                      gl_add(gl_mul(v[S2], B31),
                             gl_mul(live2, gl_sub(gl_add(gl_mul(v[E2], B23), v[M2]), B23)))));      // 40
        c.push(gl_sub(v[Q16], gl_add(gl_dbl(v[Q16H]), v[L03])));                                    // 41
        c.push(hw_bool(v[RB3]));                                                                    // 42
        c.push(hw_bool(v[L03]));                                                                    // 43
        c.push(hw_bool(v[ZRT3]));                                                                   // 44
        c.push(gl_mul(v[ZRT3], v[RT3]));                                                            // 45
        c.push(gl_sub(gl_mul(v[RT3], v[RTI3]), hw_not(v[ZRT3])));                                   // 46
        c.push(gl_sub(v[RUP3], gl_mul(v[RB3], gl_add(hw_not(v[ZRT3]), gl_mul(v[ZRT3], v[L03])))));  // 47
        c.push(gl_sub(v[YB], gl_add(v[Q16], v[RUP3])));                                             // 48
        return c.weighted(v[0]);
    }
};

}  // namespace zkh
