// Witness of the fp8 (Hawkeye) matmul gadget on the GPU: the exact replay of the fp8 forward pass
// (p3hwl::gen_witness, zkllm-src/p3_hawkeye.cuh:342-637, a host loop in the reference) written as one kernel.
//
// One warp per output (b, n): lane kk owns product kk of the current group of 32, so the group maximum, the first
// attaining product and the aligned sum are warp reductions, and every per-product column is written as one 256-byte
// line per warp.  The warp walks the K/32 groups in order carrying the accumulator state (sign, biased exponent,
// significand) in registers; the per-group and per-output columns are written by lane 0.  Columns that hold a field
// inverse (1/x or 0) receive x here and are inverted in place afterwards, 16 elements per Fermat inversion.
// The kernel is write-bound: 10 + 2 field columns and 4 index columns per product = 112 bytes per product.
#include "common.cuh"

namespace {

enum { NDP = 10, NDG = 29, NDO = 46, NDS = 6, NLU = 38 };
enum { C_DP = 0, C_DG = NDP, C_DO = NDP + NDG, C_DB = NDP + NDG + NDO, C_DN = C_DB + NDS, C_VA = C_DN + NDS, C_VB = C_VA + 1,
       NC64 = C_VB + 1 };
// column ids inside their domains (zkllm-src/p3_hawkeye.cuh:86-112)
enum { P_EB = 0, P_MAG, P_SG, P_PR, P_SH, P_PW, P_Q, P_R, P_AL, P_SEL };
enum { G_ASIG = 0, G_BEXP, G_ASGN, G_AZ, G_AINV, G_ABASE, G_ALO, G_ASH, G_APW, G_AQ, G_AR, G_MAX, G_ASEL, G_CSUM, G_TSGN, G_TMAG,
       G_TZ, G_TINV, G_WD, G_PLO, G_PHI, G_PDN, G_PUP, G_NR, G_S14, G_U1H, G_U1L, G_U2H, G_U2L };
enum { O_S14F = 0, O_BEXP, O_SGN, O_FZ, O_FINV, O_C1, O_REM1, O_RB1, O_RT1, O_RTI1, O_ZRT1, O_FH1, O_FL1, O_FLH1, O_L01, O_RUP1,
       O_C21, O_M1, O_E1, O_S1, O_Z1, O_C2, O_RB2, O_TH2, O_TL2, O_RTI2, O_ZRT2, O_FH2, O_FL2, O_FLH2, O_L02, O_RUP2, O_C22, O_M2,
       O_E2, O_S2, O_Z2, O_Q16, O_Q16H, O_L03, O_RB3, O_RT3, O_RTI3, O_ZRT3, O_RUP3, O_YB };
enum { S_SS = 0, S_SE, S_SEI, S_ZS, S_SMH, S_SML };
enum { LU_DM = 0, LU_SH, LU_RM, LU_Q15, LU_ASH, LU_ARM, LU_AQ, LU_ABASE, LU_ALO, LU_WD, LU_U1H, LU_U1L, LU_U2H, LU_U2L, LU_NR, LU_S14,
       LU_M1REM, LU_M1RT, LU_M1FH, LU_M1FL, LU_M1FLH, LU_M1E, LU_M2TH, LU_M2TL, LU_M2FH, LU_M2FL, LU_M2FLH, LU_M2E, LU_Q16,
       LU_Q16H, LU_RT3, LU_S14F, LU_XSE, LU_XSMH, LU_XSML, LU_WSE, LU_WSMH, LU_WSML };
// error bits: the conditions under which the reference's replay throws
enum { E_X_INF = 1, E_X_SUB = 2, E_W_INF = 4, E_W_SUB = 8, E_SHIFT = 16, E_ASHIFT = 32, E_WIDTH = 64, E_S14 = 128, E_FSIG = 256,
       E_MUL1 = 512, E_MUL2 = 1024 };

struct HwlPtrs {
    const gl_t *xc, *wc, *xsb, *wsb;
    gl_t* c[NC64];
    uint32_t* li[NLU];
};

__device__ __forceinline__ gl_t enc(long long x) { return x >= 0 ? (gl_t)x : GL_P - (gl_t)(-x); }
__device__ __forceinline__ void decode_e4m3(uint32_t raw, int& exp_eff, int& sig_abs, int& sign) {
    sign = (raw >> 7) & 1;
    const int eb = (raw >> 3) & 15, mant = raw & 7;
    sig_abs = eb ? (mant | 8) : mant;
    exp_eff = eb ? eb : 1;
}

// per-row scale decomposition (Db / Dn): rows of the x scales first, then the w scales
__global__ void __launch_bounds__(256) hwl_scale_kernel(HwlPtrs P, uint32_t Bpad, uint32_t Npad, unsigned int* err) {
    const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= Bpad + Npad) return;
    const bool isx = t < Bpad;
    const uint32_t i = isx ? t : t - Bpad;
    const uint32_t v = (uint32_t)(isx ? P.xsb[i] : P.wsb[i]);
    const uint32_t ss = v >> 31, se = (v >> 23) & 255, sm = v & 0x7FFFFF;
    unsigned e = 0;
    if (se == 255) e |= isx ? E_X_INF : E_W_INF;
    if (se == 0 && sm != 0) e |= isx ? E_X_SUB : E_W_SUB;
    if (e) atomicOr(err, e);
    const int sb = isx ? C_DB : C_DN;
    P.c[sb + S_SS][i] = ss; P.c[sb + S_SE][i] = se; P.c[sb + S_SEI][i] = se; P.c[sb + S_ZS][i] = se == 0;
    P.c[sb + S_SMH][i] = sm >> 12; P.c[sb + S_SML][i] = sm & 4095;
    const int l0 = isx ? LU_XSE : LU_WSE;
    P.li[l0][i] = se; P.li[l0 + 1][i] = sm >> 12; P.li[l0 + 2][i] = sm & 4095;
}

__global__ void __launch_bounds__(256) hwl_replay_kernel(HwlPtrs P, uint32_t lb, uint32_t ln, uint32_t lg, unsigned int* err) {
    const unsigned FULL = 0xFFFFFFFFu;
    const uint32_t lane = threadIdx.x & 31;
    const size_t o = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const size_t Opad = (size_t)1 << (lb + ln);
    if (o >= Opad) return;
    const uint32_t b = (uint32_t)(o >> ln), n = (uint32_t)(o & (((size_t)1 << ln) - 1));
    const uint32_t Gpad = 1u << lg;
    const size_t Kpad = (size_t)32 << lg;
    const gl_t* xrow = P.xc + (size_t)b * Kpad + lane;
    const gl_t* wrow = P.wc + (size_t)n * Kpad + lane;
    long long sgn = 0, bexp = 0, sig = 0;
    unsigned e = 0;
    for (uint32_t g = 0; g < Gpad; g++) {
        const size_t gi = (size_t)g * Opad + o, p = gi * 32 + lane;
        const uint32_t ca = (uint32_t)xrow[(size_t)g * 32], cb = (uint32_t)wrow[(size_t)g * 32];
        int ea, siga, sna, eb2, sigb, snb;
        decode_e4m3(ca, ea, siga, sna);
        decode_e4m3(cb, eb2, sigb, snb);
        const int pr = (siga && sigb) ? 1 : 0;
        const int eb = ea + eb2 - 2, bpe = eb + 127;
        const int mag = (siga * sigb) << 7;
        const int sg = (pr && (sna ^ snb)) ? 1 : 0;
        const int az = sig == 0;
        const int baee = az ? 0 : (int)bexp;
        const int bgmax = max(baee, __reduce_max_sync(FULL, pr ? bpe : -1));
        const int asel = baee == bgmax;
        const unsigned att = __ballot_sync(FULL, pr && bpe == bgmax);
        const int sel_kk = (!asel && att) ? (__ffs(att) - 1) : -1;
        const int sh = pr ? bgmax - bpe : 0;
        if (sh > 63) e |= E_SHIFT;
        const int shc = min(sh, 15), pw = 1 << shc;
        const int q = mag >> shc, r = mag - (q << shc);
        const int al = pr ? (sg ? -q : q) : 0;
        const int csum = __reduce_add_sync(FULL, al);
        P.c[C_DP + P_EB][p] = (gl_t)eb; P.c[C_DP + P_MAG][p] = (gl_t)mag; P.c[C_DP + P_SG][p] = (gl_t)sg;
        P.c[C_DP + P_PR][p] = (gl_t)pr; P.c[C_DP + P_SH][p] = (gl_t)sh; P.c[C_DP + P_PW][p] = (gl_t)pw;
        P.c[C_DP + P_Q][p] = (gl_t)q; P.c[C_DP + P_R][p] = (gl_t)r; P.c[C_DP + P_AL][p] = enc(al);
        P.c[C_DP + P_SEL][p] = (gl_t)(sel_kk == (int)lane);
        P.c[C_VA][p] = ca; P.c[C_VB][p] = cb;
        P.li[LU_DM][p] = ca * 256 + cb; P.li[LU_SH][p] = (uint32_t)sh;
        P.li[LU_RM][p] = (uint32_t)(pw - 1 + r); P.li[LU_Q15][p] = (uint32_t)q;
        // accumulator realign and normalisation: the same values on every lane
        const long long abase = sig >> 10, alo = sig & 1023;
        const int ash = bgmax - baee;
        if (ash < 0 || ash > 255) e |= E_ASHIFT;
        const int ashc = min(max(ash, 0), 15);
        const long long apw = 1LL << ashc;
        const long long aq = abase >> ashc, ar = abase - (aq << ashc);
        const long long total = (long long)csum + (sgn ? -aq : aq);
        const long long tsgn = total < 0, tmag = total < 0 ? -total : total;
        const int tz = tmag == 0;
        int wd = 64 - __clzll(tmag);
        if (wd > 20) { e |= E_WIDTH; wd = 20; }
        const long long plo = wd ? 1LL << (wd - 1) : 0, phi = 1LL << wd;
        const int dns = wd > 14 ? wd - 14 : 0, ups = wd < 14 ? 14 - wd : 0;
        const long long pdn = 1LL << dns, pup = 1LL << ups;
        const long long u1 = tmag - plo, u2 = phi - 1 - tmag;
        const long long nr = wd > 14 ? (tmag & (pdn - 1)) : 0;
        const long long s14 = wd > 14 ? (tmag >> dns) : (tmag << ups);
        if (s14 * pdn + nr != tmag * pup) e |= E_S14;
        if (lane == 0) {
            P.c[C_DG + G_ASIG][gi] = (gl_t)sig; P.c[C_DG + G_BEXP][gi] = (gl_t)bexp; P.c[C_DG + G_ASGN][gi] = (gl_t)sgn; P.c[C_DG + G_AZ][gi] = (gl_t)az;
            P.c[C_DG + G_AINV][gi] = (gl_t)sig; P.c[C_DG + G_ABASE][gi] = (gl_t)abase; P.c[C_DG + G_ALO][gi] = (gl_t)alo; P.c[C_DG + G_ASH][gi] = (gl_t)ash;
            P.c[C_DG + G_APW][gi] = (gl_t)apw; P.c[C_DG + G_AQ][gi] = (gl_t)aq; P.c[C_DG + G_AR][gi] = enc(ar); P.c[C_DG + G_MAX][gi] = (gl_t)bgmax;
            P.c[C_DG + G_ASEL][gi] = (gl_t)asel; P.c[C_DG + G_CSUM][gi] = enc(csum); P.c[C_DG + G_TSGN][gi] = (gl_t)tsgn; P.c[C_DG + G_TMAG][gi] = (gl_t)tmag;
            P.c[C_DG + G_TZ][gi] = (gl_t)tz; P.c[C_DG + G_TINV][gi] = (gl_t)tmag; P.c[C_DG + G_WD][gi] = (gl_t)wd; P.c[C_DG + G_PLO][gi] = (gl_t)plo;
            P.c[C_DG + G_PHI][gi] = (gl_t)phi; P.c[C_DG + G_PDN][gi] = (gl_t)pdn; P.c[C_DG + G_PUP][gi] = (gl_t)pup; P.c[C_DG + G_NR][gi] = (gl_t)nr;
            P.c[C_DG + G_S14][gi] = (gl_t)s14; P.c[C_DG + G_U1H][gi] = (gl_t)(u1 >> 10); P.c[C_DG + G_U1L][gi] = (gl_t)(u1 & 1023);
            P.c[C_DG + G_U2H][gi] = (gl_t)(u2 >> 10); P.c[C_DG + G_U2L][gi] = (gl_t)(u2 & 1023);
            P.li[LU_ASH][gi] = (uint32_t)ash; P.li[LU_ARM][gi] = (uint32_t)(apw - 1 + ar); P.li[LU_AQ][gi] = (uint32_t)aq;
            P.li[LU_ABASE][gi] = (uint32_t)abase; P.li[LU_ALO][gi] = (uint32_t)alo; P.li[LU_WD][gi] = (uint32_t)wd;
            P.li[LU_U1H][gi] = (uint32_t)(u1 >> 10); P.li[LU_U1L][gi] = (uint32_t)(u1 & 1023);
            P.li[LU_U2H][gi] = (uint32_t)(u2 >> 10); P.li[LU_U2L][gi] = (uint32_t)(u2 & 1023);
            P.li[LU_NR][gi] = (uint32_t)(pdn - 1 + nr); P.li[LU_S14][gi] = (uint32_t)s14;
        }
        if (!tz) { sgn = tsgn; bexp = bgmax + wd - 14; sig = s14 << 10; }
        else { sgn = 0; bexp = 0; sig = 0; }
    }
    if (lane == 0) {
        // output stage: accumulator -> fp32, two round-to-nearest-even multiplies by the scales, bf16 downcast
        const long long s14f = sig >> 10;
        if ((s14f << 10) != sig) e |= E_FSIG;
        const int fz = sig == 0;
        const uint32_t xb = (uint32_t)P.xsb[b], wb = (uint32_t)P.wsb[n];
        const uint32_t ssx = xb >> 31, sex = (xb >> 23) & 255, smx = xb & 0x7FFFFF;
        const uint32_t ssw = wb >> 31, sew = (wb >> 23) & 255, smw = wb & 0x7FFFFF;
        const int z1 = fz || sex == 0, z2 = z1 || sew == 0;
        const long long s1o = sgn ^ (long long)ssx, s2o = s1o ^ (long long)ssw;
        long long c1 = 0, rem1 = 0, rb1 = 0, rt1 = 0, rup1 = 0, c21 = 0, fh1 = 2048, fl1 = 0, m1o = 1 << 23, e1o = 1;
        if (!z1) {
            const unsigned long long mm1 = (unsigned long long)s14f * ((1u << 23) | smx);
            c1 = mm1 >= (1ULL << 37);
            const unsigned long long mfl1 = mm1 >> (13 + c1);
            rem1 = (long long)(mm1 & ((1ULL << (13 + c1)) - 1));
            fh1 = (long long)(mfl1 >> 12); fl1 = (long long)(mfl1 & 4095);
            rb1 = rem1 >> (12 + c1); rt1 = rem1 & ((1LL << (12 + c1)) - 1);
            rup1 = (rb1 && (rt1 != 0 || (fl1 & 1))) ? 1 : 0;
            const long long mr1 = (long long)mfl1 + rup1;
            c21 = mr1 == (1 << 24);
            m1o = mr1 - (c21 << 23);
            e1o = (bexp - 12) + (long long)sex - 127 + c1 + c21;
            if (e1o < 1 || e1o > 254) e |= E_MUL1;
        }
        P.c[C_DO + O_S14F][o] = (gl_t)s14f; P.c[C_DO + O_BEXP][o] = (gl_t)bexp; P.c[C_DO + O_SGN][o] = (gl_t)sgn; P.c[C_DO + O_FZ][o] = (gl_t)fz;
        P.c[C_DO + O_FINV][o] = (gl_t)s14f; P.c[C_DO + O_C1][o] = (gl_t)c1; P.c[C_DO + O_REM1][o] = (gl_t)rem1; P.c[C_DO + O_RB1][o] = (gl_t)rb1;
        P.c[C_DO + O_RT1][o] = (gl_t)rt1; P.c[C_DO + O_RTI1][o] = (gl_t)rt1; P.c[C_DO + O_ZRT1][o] = (gl_t)(rt1 == 0); P.c[C_DO + O_FH1][o] = (gl_t)fh1;
        P.c[C_DO + O_FL1][o] = (gl_t)fl1; P.c[C_DO + O_FLH1][o] = (gl_t)(fl1 >> 1); P.c[C_DO + O_L01][o] = (gl_t)(fl1 & 1); P.c[C_DO + O_RUP1][o] = (gl_t)rup1;
        P.c[C_DO + O_C21][o] = (gl_t)c21; P.c[C_DO + O_M1][o] = (gl_t)m1o; P.c[C_DO + O_E1][o] = (gl_t)e1o; P.c[C_DO + O_S1][o] = (gl_t)s1o; P.c[C_DO + O_Z1][o] = (gl_t)z1;
        P.li[LU_S14F][o] = (uint32_t)s14f;
        P.li[LU_M1REM][o] = (uint32_t)(c1 ? 8192 + rem1 : rem1); P.li[LU_M1RT][o] = (uint32_t)(c1 ? 4096 + rt1 : rt1);
        P.li[LU_M1FH][o] = (uint32_t)(fh1 - 2048); P.li[LU_M1FL][o] = (uint32_t)fl1; P.li[LU_M1FLH][o] = (uint32_t)(fl1 >> 1);
        P.li[LU_M1E][o] = (uint32_t)e1o;
        long long c2 = 0, rb2 = 0, th2 = 0, tl2 = 0, rup2 = 0, c22 = 0, fh2 = 2048, fl2 = 0, m2o = 1 << 23, e2o = 1;
        if (!z2) {
            const unsigned long long mm2 = (unsigned long long)m1o * ((1u << 23) | smw);
            c2 = mm2 >= (1ULL << 47);
            const unsigned long long mfl2 = mm2 >> (23 + c2);
            const unsigned long long rem2 = mm2 & ((1ULL << (23 + c2)) - 1);
            fh2 = (long long)(mfl2 >> 12); fl2 = (long long)(mfl2 & 4095);
            rb2 = (long long)(rem2 >> (22 + c2));
            const unsigned long long rt2 = rem2 & ((1ULL << (22 + c2)) - 1);
            th2 = (long long)(rt2 >> 12); tl2 = (long long)(rt2 & 4095);
            rup2 = (rb2 && (rt2 != 0 || (fl2 & 1))) ? 1 : 0;
            const long long mr2 = (long long)mfl2 + rup2;
            c22 = mr2 == (1 << 24);
            m2o = mr2 - (c22 << 23);
            e2o = e1o + (long long)sew - 127 + c2 + c22;
            if (e2o < 1 || e2o > 254) e |= E_MUL2;
        }
        const long long rt2v = th2 * 4096 + tl2;
        P.c[C_DO + O_C2][o] = (gl_t)c2; P.c[C_DO + O_RB2][o] = (gl_t)rb2; P.c[C_DO + O_TH2][o] = (gl_t)th2; P.c[C_DO + O_TL2][o] = (gl_t)tl2;
        P.c[C_DO + O_RTI2][o] = (gl_t)rt2v; P.c[C_DO + O_ZRT2][o] = (gl_t)(rt2v == 0); P.c[C_DO + O_FH2][o] = (gl_t)fh2; P.c[C_DO + O_FL2][o] = (gl_t)fl2;
        P.c[C_DO + O_FLH2][o] = (gl_t)(fl2 >> 1); P.c[C_DO + O_L02][o] = (gl_t)(fl2 & 1); P.c[C_DO + O_RUP2][o] = (gl_t)rup2; P.c[C_DO + O_C22][o] = (gl_t)c22;
        P.c[C_DO + O_M2][o] = (gl_t)m2o; P.c[C_DO + O_E2][o] = (gl_t)e2o; P.c[C_DO + O_S2][o] = (gl_t)s2o; P.c[C_DO + O_Z2][o] = (gl_t)z2;
        P.li[LU_M2TH][o] = (uint32_t)(c2 ? 1024 + th2 : th2); P.li[LU_M2TL][o] = (uint32_t)tl2;
        P.li[LU_M2FH][o] = (uint32_t)(fh2 - 2048); P.li[LU_M2FL][o] = (uint32_t)fl2; P.li[LU_M2FLH][o] = (uint32_t)(fl2 >> 1);
        P.li[LU_M2E][o] = (uint32_t)e2o;
        const unsigned long long b32 = ((unsigned long long)s2o << 31) |
                                       (z2 ? 0ULL : (((unsigned long long)e2o << 23) | (unsigned long long)(m2o - (1 << 23))));
        const long long q16 = (long long)(b32 >> 16), rem3 = (long long)(b32 & 0xFFFF);
        const long long rb3 = rem3 >> 15, rt3 = rem3 & 0x7FFF;
        const long long rup3 = (rb3 && (rt3 != 0 || (q16 & 1))) ? 1 : 0;
        P.c[C_DO + O_Q16][o] = (gl_t)q16; P.c[C_DO + O_Q16H][o] = (gl_t)(q16 >> 1); P.c[C_DO + O_L03][o] = (gl_t)(q16 & 1); P.c[C_DO + O_RB3][o] = (gl_t)rb3;
        P.c[C_DO + O_RT3][o] = (gl_t)rt3; P.c[C_DO + O_RTI3][o] = (gl_t)rt3; P.c[C_DO + O_ZRT3][o] = (gl_t)(rt3 == 0); P.c[C_DO + O_RUP3][o] = (gl_t)rup3;
        P.c[C_DO + O_YB][o] = (gl_t)(q16 + rup3);
        P.li[LU_Q16][o] = (uint32_t)q16; P.li[LU_Q16H][o] = (uint32_t)(q16 >> 1); P.li[LU_RT3][o] = (uint32_t)rt3;
    }
    if (e) atomicOr(err, e);
}

// a[i] <- 1/a[i], or 0 where a[i] == 0; 16 strided elements share one Fermat inversion
#define HWL_INV_K 16
__global__ void __launch_bounds__(256) hwl_inv_or0_kernel(gl_t* __restrict__ a, size_t n) {
    const size_t nthreads = (size_t)gridDim.x * blockDim.x, t = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    gl_t d[HWL_INV_K], pre[HWL_INV_K];
    gl_t acc = 1;
#pragma unroll
    for (int k = 0; k < HWL_INV_K; k++) {
        const size_t i = t + (size_t)k * nthreads;
        const gl_t v = i < n ? a[i] : 0;
        d[k] = v;
        pre[k] = acc;
        acc = gl_mul(acc, v ? v : 1);
    }
    gl_t inv = gl_inv(acc);
#pragma unroll
    for (int k = HWL_INV_K - 1; k >= 0; k--) {
        const size_t i = t + (size_t)k * nthreads;
        if (i < n) a[i] = d[k] ? gl_mul(pre[k], inv) : 0;
        inv = gl_mul(inv, d[k] ? d[k] : 1);
    }
}

const char* hwl_err_text(unsigned e) {
    if (e & E_X_INF) return "hwl: inf/nan x-scale unsupported";
    if (e & E_X_SUB) return "hwl: subnormal x-scale unsupported";
    if (e & E_W_INF) return "hwl: inf/nan w-scale unsupported";
    if (e & E_W_SUB) return "hwl: subnormal w-scale unsupported";
    if (e & E_SHIFT) return "hwl: product shift > 63";
    if (e & E_ASHIFT) return "hwl: acc shift out of [0,255]";
    if (e & E_WIDTH) return "hwl: total width > 20";
    if (e & E_S14) return "hwl: s14 identity";
    if (e & E_FSIG) return "hwl: fsig low bits";
    if (e & E_MUL1) return "hwl: mul1 out of normal fp32 range";
    return "hwl: mul2 out of normal fp32 range";
}
}  // namespace

extern "C" int zkh_hwl_witness(zkh_ctx* c, uint32_t lb, uint32_t ln, uint32_t lg, const uint64_t* xcodes_dev,
                               const uint64_t* wcodes_dev, const uint64_t* xsb_dev, const uint64_t* wsb_dev,
                               uint64_t* const* cols_dev, uint32_t* const* lidx_dev) {
    if (!c) return ZKH_ERR_ARG;
    if (!xcodes_dev || !wcodes_dev || !xsb_dev || !wsb_dev || !cols_dev || !lidx_dev)
        return zkh_fail(c, ZKH_ERR_ARG, "hwl_witness: null pointer");
    if (lb < 1 || ln < 1 || lg < 1 || lb + ln + lg + 5 > 34) return zkh_fail(c, ZKH_ERR_ARG, "hwl_witness: dims out of range");
    HwlPtrs P;
    P.xc = xcodes_dev; P.wc = wcodes_dev; P.xsb = xsb_dev; P.wsb = wsb_dev;
    for (int i = 0; i < NC64; i++) {
        if (!cols_dev[i]) return zkh_fail(c, ZKH_ERR_ARG, "hwl_witness: null column");
        P.c[i] = cols_dev[i];
    }
    for (int i = 0; i < NLU; i++) {
        if (!lidx_dev[i]) return zkh_fail(c, ZKH_ERR_ARG, "hwl_witness: null index column");
        P.li[i] = lidx_dev[i];
    }
    ZKH_CUDA(c, cudaSetDevice(c->device));
    unsigned int* err = &c->d_ctl->err;
    ZKH_CUDA(c, cudaMemsetAsync(err, 0, 4, c->stream));
    const uint32_t Bpad = 1u << lb, Npad = 1u << ln;
    const size_t Opad = (size_t)Bpad * Npad, G = Opad << lg;
    hwl_scale_kernel<<<(Bpad + Npad + 255) / 256, 256, 0, c->stream>>>(P, Bpad, Npad, err);
    hwl_replay_kernel<<<(unsigned)((Opad * 32 + 255) / 256), 256, 0, c->stream>>>(P, lb, ln, lg, err);
    ZKH_CUDA(c, cudaGetLastError());
    auto inv = [&](gl_t* a, size_t n) {
        const size_t threads = (n + HWL_INV_K - 1) / HWL_INV_K;
        hwl_inv_or0_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, c->stream>>>(a, n);
    };
    inv(P.c[C_DG + G_AINV], G); inv(P.c[C_DG + G_TINV], G);
    inv(P.c[C_DO + O_FINV], Opad); inv(P.c[C_DO + O_RTI1], Opad); inv(P.c[C_DO + O_RTI2], Opad); inv(P.c[C_DO + O_RTI3], Opad);
    inv(P.c[C_DB + S_SEI], Bpad); inv(P.c[C_DN + S_SEI], Npad);
    ZKH_CUDA(c, cudaGetLastError());
    ZKH_CUDA(c, cudaMemcpyAsync(&c->h_ctl->err, err, 4, cudaMemcpyDeviceToHost, c->stream));
    ZKH_CUDA(c, cudaStreamSynchronize(c->stream));
    if (c->h_ctl->err) return zkh_fail(c, ZKH_ERR_DOMAIN, hwl_err_text(c->h_ctl->err));
    return ZKH_OK;
}
