// BLS12-381 G1 openings of the first proof stack for sm_100a: the Fiat-Shamir inner-product argument (ipa_prove / ipa_verify,
// zkllm-src/vrf_common.cuh:302-371), the multi-scalar product in the reference's summation order (dev_msm, :165-184) and
// the pair-fold chains of commitments and generators (fold_chain with k_com_me / k_gen_fold, :52-66 and :144-163).
//
// The proof files hold Jacobian triples, so every group element has to come out of the same sequence of additions and
// doublings as in the reference.  Its scalar multiple (G1Jacobian_mul, zkllm-src/g1-tensor.cu:445-453) runs two chains
// side by side, from the lowest bit up: the doublings 2^k P, which do not depend on the scalar, and the sum of those
// selected by the scalar's bits.  Here the two are separate steps:
//   * a table kernel writes 2^k P for k < 256 once per point (k-major, so that a warp reads neighbouring records);
//   * a chain kernel adds the selected entries in bit order.
// One table serves every product of a point: in a round of the argument the halves of g are multiplied by the halves of a
// (for L and R) and then by the challenge and its inverse (for the fold), three products from one table where the
// reference doubles three times.  A round is a fixed sequence of launches on the context's stream with the transcript on
// the device; the host reads L, R, the final scalar and the transcript state once at the end.  Every kernel here is bound by
// the latency of one chain of dependent group operations with most of the GPU idle, so each point operation is spread over
// four lanes (g1q_add / g1q_double: the independent 384-bit products of a formula run one per lane) and blocks are single
// warps of eight points spread over all SMs.
#include "common.cuh"
#include "fr_dev.cuh"
#include "g1.cuh"
#include "sha256.cuh"

namespace zkh {

constexpr uint32_t G1_BITS = 256;               // table depth: bit k of the scalar's eight raw limbs selects 2^k P
constexpr int G1_WARP = 32;
constexpr int G1_QPB = G1_WARP / 4;             // points per block: each point operation runs on four lanes (g1q_add / g1q_double)

// index of this thread's quad in the grid
__device__ __forceinline__ uint32_t quad_index() { return blockIdx.x * G1_QPB + (threadIdx.x >> 2); }
// the four lanes of a quad hold the same point and store a quarter each
__device__ __forceinline__ void g1q_store(G1* p, const G1& v) {
    uint4* q = reinterpret_cast<uint4*>(p);
    const uint32_t* w = v.x.v;                  // x, y, z are contiguous: 36 limbs, nine 16-byte pieces
    const int ql = threadIdx.x & 3;
#pragma unroll
    for (int j = 0; j < 9; j++)
        if ((j & 3) == ql) q[j] = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
}

// tab[k * n + i] = 2^k g[i]
__global__ void __launch_bounds__(G1_WARP) g1_table_kernel(const G1* __restrict__ g, uint32_t n, G1* __restrict__ tab) {
    const uint32_t i = quad_index();
    if (i >= n) return;
    const uint32_t qm = g1q_mask();
    G1 a = g1_load(g + i);
    for (uint32_t k = 0; k < G1_BITS; k++) {
        g1q_store(tab + (size_t)k * n + i, a);
        if (k + 1 < G1_BITS) a = g1q_double(a, qm);
    }
}
// sum over the set bits of s, lowest first, of 2^k P: the accumulator of G1Jacobian_mul, which starts at infinity and
// therefore takes the first selected entry unchanged.  The loop visits set bits only, so that the quads of a warp, whose
// scalars differ, all add in every iteration.
__device__ __forceinline__ G1 g1q_chain(const G1* __restrict__ tab, size_t n, size_t i, const Fr& s, uint32_t qm) {
    G1 out = g1_zero();
    uint32_t w = 0, cur = s.v[0];
    for (;;) {
        while (cur == 0 && w < 7) cur = s.v[++w];
        if (cur == 0) break;
        const uint32_t k = 32 * w + (uint32_t)__ffs((int)cur) - 1;
        cur &= cur - 1;
        out = g1q_add(out, g1_load(tab + (size_t)k * n + i), qm);
    }
    return out;
}
// One batch of scalar multiples: out[idx] = s(idx) * point((idx ^ pxor) & pmask) for idx < count.
// mode 0: s = sc[idx]; mode 1: s = sc[0]; mode 2: s = sc[1] for idx < count / 2, sc[0] above.
struct ChainSeg {
    const G1* tab;
    const Fr* sc;
    G1* out;
    uint32_t n, count, pxor, pmask, mode;
};
__global__ void __launch_bounds__(G1_WARP) g1_chain_kernel(ChainSeg A, ChainSeg B) {
    uint32_t idx = quad_index();
    const bool second = idx >= A.count;
    if (second) idx -= A.count;
    const ChainSeg& S = second ? B : A;
    if (idx >= S.count) return;
    const Fr s = fr_load(S.sc + (S.mode == 0 ? idx : S.mode == 1 ? 0u : (idx < S.count / 2 ? 1u : 0u)));
    g1q_store(S.out + idx, g1q_chain(S.tab, S.n, (idx ^ S.pxor) & S.pmask, s, g1q_mask()));
}
// one level of the pairwise sums of dev_msm: p[i] += p[i + half], for each of gridDim.y arrays `stride` apart
__global__ void __launch_bounds__(G1_WARP) g1_tree_kernel(G1* T, uint32_t stride, uint32_t half) {
    const uint32_t i = quad_index();
    if (i >= half) return;
    G1* p = T + (size_t)blockIdx.y * stride;
    g1q_store(p + i, g1q_add(g1_load(p + i), g1_load(p + i + half), g1q_mask()));
}

// ------------------------------------------------------------------ the argument's rounds
// sc[0] = <a_lo, b_hi>, sc[1] = <a_hi, b_lo> as plain integers (dev_ip); block 0 / block 1
__global__ void __launch_bounds__(FR_THREADS) ipa_dot_kernel(const Fr* __restrict__ a, const Fr* __restrict__ b, uint32_t h, Fr* sc) {
    __shared__ __align__(16) Fr sh[32];
    const Fr* x = blockIdx.x ? a + h : a;
    const Fr* y = blockIdx.x ? b : b + h;
    Fr acc[1] = {fr_zero()};
    for (uint32_t i = threadIdx.x; i < h; i += blockDim.x) acc[0] = fr_add(acc[0], fr_mmul(fr_load(x + i), fr_load(y + i)));
    fr_block_sum<1>(acc, sh);
    if (threadIdx.x == 0) fr_store(sc + blockIdx.x, fr_mmul(acc[0], FR_RPOW[1]));   // the products carried 1/R
}
// L = T[0] + c_L Q, R = T[h] + c_R Q; absorb "L", "R"; x = challenge, 1/x.  One warp.  sc[2] = x, sc[3] = 1/x.
__global__ void __launch_bounds__(G1_WARP) ipa_round_end_kernel(const G1* T, uint32_t h, const G1* QT, ZkhCtl* ctl, G1* Lout, G1* Rout,
                                                              Fr* sc, ZkhTag tagL, ZkhTag tagR) {
    __shared__ __align__(16) G1 lr[2];
    __shared__ __align__(16) uint32_t trbuf[ZKH_TRBUF_WORDS];
    const uint32_t lane = threadIdx.x, q = lane >> 2;
    if (q < 2) {                                              // quad 0: L, quad 1: R
        const G1 v = g1q_add(g1_load(T + (size_t)q * h), g1_load(QT + q), g1q_mask());
        if ((lane & 3) == 0) lr[q] = v;
        g1q_store(q ? Rout : Lout, v);
    }
    __syncwarp();
    uint32_t st[8];
#pragma unroll
    for (int i = 0; i < 8; i++) st[i] = ctl->st[i];
    tr_warp_absorb(st, tagL.s, tagL.len, reinterpret_cast<const uint64_t*>(&lr[0]), sizeof(G1) / 8, trbuf);
    tr_warp_absorb(st, tagR.s, tagR.len, reinterpret_cast<const uint64_t*>(&lr[1]), sizeof(G1) / 8, trbuf);
    Fr x;
    bool ok = false;
    for (int tries = 0; tries < 8 && !ok; tries++) {        // the reference redraws while the challenge is zero
        tr_warp_challenge_limbs(st, x.v);
        x.v[7] %= 0x73eda753u;
        ok = !fr_is_zero(x);
    }
    if (lane == 0) {
        if (!ok) atomicOr(&ctl->err, 2u);
#pragma unroll
        for (int i = 0; i < 8; i++) ctl->st[i] = st[i];
        fr_store(sc + 2, x);
        fr_store(sc + 3, fr_from_mont(fr_inv_mont(fr_to_mont(x))));
    }
}
// a' = x a_lo + x^-1 a_hi, b' = x^-1 b_lo + x b_hi, g' = W_lo + W_hi (W = the halves of g times x^-1 and x), and the
// doubling table of g' for the next round
__global__ void __launch_bounds__(G1_WARP) ipa_fold_kernel(const Fr* __restrict__ a, const Fr* __restrict__ b, const G1* __restrict__ W,
                                                         const Fr* __restrict__ sc, uint32_t h, Fr* a2, Fr* b2, G1* g2, G1* tab) {
    const uint32_t i = quad_index();
    if (i >= h) return;
    const uint32_t qm = g1q_mask();
    const int ql = threadIdx.x & 3;
    if (ql < 2) {                                             // lane 0 folds a, lane 1 folds b
        const Fr xm = fr_to_mont(fr_load(sc + 2)), xim = fr_to_mont(fr_load(sc + 3));
        const Fr* v = ql ? b : a;
        fr_store((ql ? b2 : a2) + i, fr_add(fr_mmul(ql ? xim : xm, fr_load(v + i)), fr_mmul(ql ? xm : xim, fr_load(v + i + h))));
    }
    __syncwarp(qm);
    G1 p = g1q_add(g1_load(W + i), g1_load(W + i + h), qm);
    g1q_store(g2 + i, p);
    if (h < 2) return;
    for (uint32_t k = 0; k < G1_BITS; k++) {
        g1q_store(tab + (size_t)k * h + i, p);
        if (k + 1 < G1_BITS) p = g1q_double(p, qm);
    }
}

// ------------------------------------------------------------------ fold chains
// d[i] = c[2i+1] - c[2i] (orientation 0, k_com_me) or c[2i] - c[2i+1] (orientation 1, k_gen_fold); an odd level is padded with
// a record of zero bytes as the reference pads it (cudaMemset), which the addition treats as infinity
__device__ __forceinline__ G1 g1_zero_bytes() {
    G1 r;
#pragma unroll
    for (int i = 0; i < 12; i++) { r.x.v[i] = 0; r.y.v[i] = 0; r.z.v[i] = 0; }
    return r;
}
__global__ void __launch_bounds__(G1_WARP) g1_pair_diff_kernel(const G1* __restrict__ c, uint32_t sz, uint32_t nsz, int orientation, G1* d) {
    const uint32_t i = quad_index();
    if (i >= nsz) return;
    const uint32_t qm = g1q_mask();
    const G1 lo = g1_load(c + 2 * i), hi = (2 * i + 1 < sz) ? g1_load(c + 2 * i + 1) : g1_zero_bytes();
    g1q_store(d + i, orientation == 0 ? g1q_add(hi, g1_neg(lo), qm) : g1q_add(lo, g1_neg(hi), qm));
}
// out[i] = c[2i] + u d[i] (orientation 0) or c[2i+1] + u d[i] (orientation 1); M = u d
__global__ void __launch_bounds__(G1_WARP) g1_pair_join_kernel(const G1* __restrict__ c, uint32_t sz, uint32_t nsz, int orientation,
                                                             const G1* __restrict__ M, G1* out) {
    const uint32_t i = quad_index();
    if (i >= nsz) return;
    const uint32_t j = orientation == 0 ? 2 * i : 2 * i + 1;
    const G1 base = j < sz ? g1_load(c + j) : g1_zero_bytes();
    g1q_store(out + i, g1q_add(base, g1_load(M + i), g1q_mask()));
}

// ------------------------------------------------------------------ the argument's verifier
// One warp replays the transcript: absorb L_r, R_r, draw x_r.  Lane 0 then inverts all challenges with one Fermat inversion
// (prefix products) and writes xs[r], xis[r], sq[2r] = x_r^2, sq[2r+1] = x_r^-2, sq[2 rounds] = a_f b_f with
// b_f = prod_r (x_r^-1 (1 - u[v-1-r]) + x_r u[v-1-r]), the fold of the public weights (round r halves on the top
// remaining variable), and sq[2 rounds + 1] = a_f.  LR: L_0, R_0, L_1, R_1, ...
#define IPA_MAX_ROUNDS 20
__global__ void __launch_bounds__(G1_WARP) ipa_verify_transcript_kernel(const G1* LR, uint32_t rounds, const Fr* u, const Fr* a_f,
                                                                      ZkhCtl* ctl, Fr* xs, Fr* xis, Fr* sq, ZkhTag tagL, ZkhTag tagR) {
    __shared__ __align__(16) G1 pt;
    __shared__ __align__(16) uint32_t trbuf[ZKH_TRBUF_WORDS];
    const uint32_t lane = threadIdx.x;
    uint32_t st[8];
#pragma unroll
    for (int i = 0; i < 8; i++) st[i] = ctl->st[i];
    bool all_ok = true;
    for (uint32_t r = 0; r < rounds; r++) {
        for (uint32_t side = 0; side < 2; side++) {
            __syncwarp();
            if (lane == 0) pt = g1_load(LR + 2 * r + side);
            __syncwarp();
            const ZkhTag& tg = side ? tagR : tagL;
            tr_warp_absorb(st, tg.s, tg.len, reinterpret_cast<const uint64_t*>(&pt), sizeof(G1) / 8, trbuf);
        }
        Fr x;
        bool ok = false;
        for (int tries = 0; tries < 8 && !ok; tries++) {
            tr_warp_challenge_limbs(st, x.v);
            x.v[7] %= 0x73eda753u;
            ok = !fr_is_zero(x);
        }
        all_ok = all_ok && ok;
        if (lane == 0) fr_store(xs + r, x);
    }
    if (lane != 0) return;
    if (!all_ok) atomicOr(&ctl->err, 2u);
#pragma unroll
    for (int i = 0; i < 8; i++) ctl->st[i] = st[i];
    // prefix products in Montgomery form, one inversion, peel back
    Fr run = FR_RPOW[0];
    for (uint32_t r = 0; r < rounds; r++) {
        fr_store(xis + r, run);                                   // prefix before r
        run = fr_mmul(run, fr_to_mont(fr_load(xs + r)));
    }
    Fr inv = fr_inv_mont(run);
    for (int r = (int)rounds - 1; r >= 0; r--) {
        const Fr xm = fr_to_mont(fr_load(xs + r));
        const Fr xim = fr_mmul(inv, fr_load(xis + r));           // 1/x_r, Montgomery form
        inv = fr_mmul(inv, xm);
        fr_store(xis + r, fr_from_mont(xim));
    }
    Fr one = fr_zero();
    one.v[0] = 1;
    Fr bf = FR_RPOW[0];                                           // Montgomery form
    for (uint32_t r = 0; r < rounds; r++) {
        const Fr x = fr_load(xs + r), xi = fr_load(xis + r), xm = fr_to_mont(x), xim = fr_to_mont(xi);
        fr_store(sq + 2 * r, fr_mmul(xm, x));
        fr_store(sq + 2 * r + 1, fr_mmul(xim, xi));
        const Fr uu = fr_load(u + (rounds - 1 - r));
        const Fr term = fr_add(fr_mmul(xim, fr_sub(one, uu)), fr_mmul(xm, uu));     // plain
        bf = fr_mmul(bf, fr_to_mont(term));
    }
    const Fr af = fr_load(a_f);
    fr_store(sq + 2 * rounds, fr_mmul(bf, af));                   // (b_f R)(a_f)/R = a_f b_f, plain
    fr_store(sq + 2 * rounds + 1, af);
}
// s_i = prod_r (bit (rounds-1-r) of i ? x_r : 1/x_r)
__global__ void __launch_bounds__(FR_THREADS) ipa_svec_kernel(const Fr* __restrict__ xs, const Fr* __restrict__ xis, uint32_t rounds, uint32_t n,
                                                            Fr* s) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    Fr w = FR_RPOW[0];
    for (uint32_t r = 0; r < rounds; r++)
        w = fr_mmul(w, fr_to_mont(fr_load(((i >> (rounds - 1 - r)) & 1u) ? xs + r : xis + r)));
    fr_store(s + i, fr_from_mont(w));
}
// One quad: P = P0, then P = (x_r^2 L_r + P) + x_r^-2 R_r per round; accept iff P == a_f g_f + (a_f b_f) Q as group elements.
// M: the 2 rounds + 1 scaled points (L, R interleaved, then (a_f b_f) Q); gf = <g, s>.
__global__ void __launch_bounds__(4) ipa_verify_final_kernel(const G1* M, uint32_t rounds, const G1* P0, const G1* gf, const Fr* a_f,
                                                           int* accept) {
    const uint32_t qm = g1q_mask();
    G1 Pt = g1_load(P0);
    for (uint32_t r = 0; r < rounds; r++) Pt = g1q_add(g1q_add(g1_load(M + 2 * r), Pt, qm), g1_load(M + 2 * r + 1), qm);
    const Fr af = fr_load(a_f);
    G1 out = g1_zero(), a = g1_load(gf);
    for (uint32_t k = 0; k < G1_BITS; k++) {
        if ((af.v[k >> 5] >> (k & 31)) & 1u) out = g1q_add(out, a, qm);
        a = g1q_double(a, qm);
    }
    const G1 rhs = g1q_add(out, g1_load(M + 2 * rounds), qm);
    const G1 d = g1q_add(Pt, g1_neg(rhs), qm);
    if (threadIdx.x == 0) *accept = fp_is_zero(d.z) ? 1 : 0;
}

// ------------------------------------------------------------------ row-wise linear relation of commitments
// bad += 1 for every row j with lhs[j] != s a[j] + b[j] as group elements (the affine link of the rescaling obligation,
// zkllm-src/zkob_rescale.cu:226-241: com_X[j] == sf com_Xr[j] + com_rem[j]); one quad per row
__global__ void __launch_bounds__(G1_WARP) g1_rows_check_kernel(const G1* __restrict__ lhs, const G1* __restrict__ a, const G1* __restrict__ b, Fr s,
                                                              uint32_t rows, unsigned int* bad) {
    const uint32_t j = quad_index();
    if (j >= rows) return;
    const uint32_t qm = g1q_mask();
    G1 acc = g1_zero(), p = g1_load(a + j);
    int top = 255;
    while (top >= 0 && !((s.v[top >> 5] >> (top & 31)) & 1u)) top--;
    for (int k = 0; k <= top; k++) {
        if ((s.v[k >> 5] >> (k & 31)) & 1u) acc = g1q_add(acc, p, qm);
        if (k < top) p = g1q_double(p, qm);
    }
    const G1 rhs = g1q_add(acc, g1_load(b + j), qm);
    const G1 d = g1q_add(g1_load(lhs + j), g1_neg(rhs), qm);
    if ((threadIdx.x & 3) == 0 && !fp_is_zero(d.z)) atomicAdd(bad, 1u);
}

// out[j] = a[j] + b[j]: the homomorphic sum of two commitment vectors (hom_add of the skip-connection obligation,
// zkllm-src/zkob_skip.cu:39-48); one quad per row
__global__ void __launch_bounds__(G1_WARP) g1_rows_add_kernel(const G1* __restrict__ a, const G1* __restrict__ b, uint32_t rows, G1* __restrict__ out) {
    const uint32_t j = quad_index();
    if (j >= rows) return;
    g1q_store(out + j, g1q_add(g1_load(a + j), g1_load(b + j), g1q_mask()));
}

// out[j] = s a[j] + b[j] with the operand order of the reference's host helpers (hb_addmul, zkllm-src/zkob_fastg1.cuh:56-92):
// mul_first ? add(mul(a, s), b) : add(b, mul(a, s)); mul in the order of G1Jacobian_mul; one quad per row
__global__ void __launch_bounds__(G1_WARP) g1_rows_lincomb_kernel(const G1* __restrict__ a, Fr s, const G1* __restrict__ b, uint32_t rows, int mul_first,
                                                                G1* __restrict__ out) {
    const uint32_t j = quad_index();
    if (j >= rows) return;
    const uint32_t qm = g1q_mask();
    G1 acc = g1_zero(), p = g1_load(a + j);
    int top = 255;
    while (top >= 0 && !((s.v[top >> 5] >> (top & 31)) & 1u)) top--;
    for (int k = 0; k <= top; k++) {
        if ((s.v[k >> 5] >> (k & 31)) & 1u) acc = g1q_add(acc, p, qm);
        if (k < top) p = g1q_double(p, qm);
    }
    const G1 bj = g1_load(b + j);
    g1q_store(out + j, mul_first ? g1q_add(acc, bj, qm) : g1q_add(bj, acc, qm));
}

static inline unsigned warp_blocks(size_t items) { return (unsigned)((items + G1_QPB - 1) / G1_QPB); }   // a quad per item

// tab = tables of the n points at g, then out[i] = s(i) g[i]; stream-ordered
static int g1_mul_enqueue(zkh_ctx* c, const G1* g, uint32_t n, const Fr* sc, uint32_t mode, G1* tab, G1* out) {
    g1_table_kernel<<<warp_blocks(n), G1_WARP, 0, c->stream>>>(g, n, tab);
    ChainSeg A = {tab, sc, out, n, n, 0u, 0xffffffffu, mode}, B = {nullptr, nullptr, nullptr, 0u, 0u, 0u, 0u, 0u};
    g1_chain_kernel<<<warp_blocks(n), G1_WARP, 0, c->stream>>>(A, B);
    return cudaGetLastError() == cudaSuccess ? ZKH_OK : zkh_fail(c, ZKH_ERR_CUDA, "g1 scalar multiple launch");
}
static int g1_tree_enqueue(zkh_ctx* c, G1* T, uint32_t stride, uint32_t n, uint32_t arrays) {
    for (uint32_t half = n / 2; half >= 1; half /= 2)
        g1_tree_kernel<<<dim3(warp_blocks(half), arrays), G1_WARP, 0, c->stream>>>(T, stride, half);
    return cudaGetLastError() == cudaSuccess ? ZKH_OK : zkh_fail(c, ZKH_ERR_CUDA, "g1 tree launch");
}
static inline bool pow2(uint32_t n) { return n && !(n & (n - 1)); }

}  // namespace zkh

using namespace zkh;

static const uint32_t G1_MAX_N = 1u << 20;      // 2^20 points: a 38 GB table

extern "C" int zkh_g1_msm(zkh_ctx* c, const void* g_dev, const void* a_dev, uint32_t n, void* out144) {
    if (!c || !g_dev || !a_dev || !out144) return zkh_fail(c, ZKH_ERR_ARG, "g1_msm: null pointer");
    if (!pow2(n) || n > G1_MAX_N) return zkh_fail(c, ZKH_ERR_ARG, "g1_msm: n must be a power of two up to 2^20");
    if (((uintptr_t)g_dev | (uintptr_t)a_dev) & 15) return zkh_fail(c, ZKH_ERR_ARG, "g1_msm: buffers must be 16-byte aligned");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    const size_t szT = zkh_align((size_t)n * sizeof(G1)), szTab = zkh_align((size_t)n * G1_BITS * sizeof(G1));
    ZKH_TRY(zkh_ws_reserve(c, szT + szTab));
    G1* T = (G1*)c->ws;
    G1* tab = (G1*)((char*)c->ws + szT);
    ZKH_TRY(g1_mul_enqueue(c, (const G1*)g_dev, n, (const Fr*)a_dev, 0, tab, T));
    ZKH_TRY(g1_tree_enqueue(c, T, 0, n, 1));
    ZKH_CUDA(c, cudaMemcpyAsync(out144, T, sizeof(G1), cudaMemcpyDeviceToHost, c->stream));
    ZKH_CUDA(c, cudaStreamSynchronize(c->stream));
    return ZKH_OK;
}

extern "C" int zkh_g1_fold_chain(zkh_ctx* c, const void* src_dev, uint32_t size, const void* us, uint32_t nu, int orientation,
                                 void* out144) {
    if (!c || !src_dev || !out144 || (nu && !us)) return zkh_fail(c, ZKH_ERR_ARG, "g1_fold_chain: null pointer");
    if (!size || size > G1_MAX_N) return zkh_fail(c, ZKH_ERR_ARG, "g1_fold_chain: size must be 1..2^20");
    if (orientation != 0 && orientation != 1) return zkh_fail(c, ZKH_ERR_ARG, "g1_fold_chain: orientation is 0 or 1");
    if ((uintptr_t)src_dev & 15) return zkh_fail(c, ZKH_ERR_ARG, "g1_fold_chain: buffer must be 16-byte aligned");
    for (uint32_t r = 0; r < nu; r++)
        if (!fr_canonical((const uint32_t*)us + 8 * r)) return zkh_fail(c, ZKH_ERR_DOMAIN, "g1_fold_chain: challenge not below p");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    const uint32_t cap = (size + 1) / 2;
    const size_t szL = zkh_align((size_t)cap * sizeof(G1)), szTab = zkh_align((size_t)cap * G1_BITS * sizeof(G1));
    const size_t szU = zkh_align((size_t)(nu ? nu : 1) * sizeof(Fr));
    ZKH_TRY(zkh_ws_reserve(c, 4 * szL + szTab + szU));
    char* w = (char*)c->ws;
    G1* lvl[2] = {(G1*)w, (G1*)(w + szL)};
    G1* D = (G1*)(w + 2 * szL);
    G1* M = (G1*)(w + 3 * szL);
    G1* tab = (G1*)(w + 4 * szL);
    Fr* u_dev = (Fr*)(w + 4 * szL + szTab);
    if (nu) ZKH_CUDA(c, cudaMemcpyAsync(u_dev, us, (size_t)nu * sizeof(Fr), cudaMemcpyHostToDevice, c->stream));
    const G1* cur = (const G1*)src_dev;
    uint32_t sz = size;
    for (uint32_t r = 0; r < nu; r++) {
        const uint32_t nsz = (sz + 1) / 2;
        G1* nxt = lvl[r & 1];
        g1_pair_diff_kernel<<<warp_blocks(nsz), G1_WARP, 0, c->stream>>>(cur, sz, nsz, orientation, D);
        ZKH_TRY(g1_mul_enqueue(c, D, nsz, u_dev + r, 1, tab, M));
        g1_pair_join_kernel<<<warp_blocks(nsz), G1_WARP, 0, c->stream>>>(cur, sz, nsz, orientation, M, nxt);
        cur = nxt;
        sz = nsz;
    }
    ZKH_CUDA(c, cudaGetLastError());
    ZKH_CUDA(c, cudaMemcpyAsync(out144, cur, sizeof(G1), cudaMemcpyDeviceToHost, c->stream));
    ZKH_CUDA(c, cudaStreamSynchronize(c->stream));
    return ZKH_OK;
}

extern "C" int zkh_g1_ipa_prove(zkh_ctx* c, const void* a_dev, const void* b_dev, const void* g_dev, const void* Q144, uint32_t n,
                                uint8_t state[32], void* L_out, void* R_out, void* a_final32) {
    if (!c || !a_dev || !b_dev || !g_dev || !Q144 || !state || !a_final32)
        return zkh_fail(c, ZKH_ERR_ARG, "g1_ipa_prove: null pointer");
    if (!pow2(n) || n > G1_MAX_N) return zkh_fail(c, ZKH_ERR_ARG, "g1_ipa_prove: n must be a power of two up to 2^20");
    if (n > 1 && (!L_out || !R_out)) return zkh_fail(c, ZKH_ERR_ARG, "g1_ipa_prove: null proof buffer");
    if (((uintptr_t)a_dev | (uintptr_t)b_dev | (uintptr_t)g_dev) & 15)
        return zkh_fail(c, ZKH_ERR_ARG, "g1_ipa_prove: buffers must be 16-byte aligned");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    uint32_t rounds = 0;
    while ((1u << rounds) < n) rounds++;
    const uint32_t nh = n > 1 ? n / 2 : 1;
    const size_t szTab = zkh_align((size_t)n * G1_BITS * sizeof(G1)), szTQ = zkh_align((size_t)G1_BITS * sizeof(G1));
    const size_t szT = zkh_align((size_t)n * sizeof(G1)), szG = zkh_align((size_t)nh * sizeof(G1)), szF = zkh_align((size_t)nh * sizeof(Fr));
    const size_t szP = zkh_align((size_t)(rounds ? rounds : 1) * sizeof(G1)), szS = zkh_align(8 * sizeof(Fr) + 3 * sizeof(G1));
    ZKH_TRY(zkh_ws_reserve(c, szTab + szTQ + szT + 2 * szG + 4 * szF + 2 * szP + szS));
    char* w = (char*)c->ws;
    G1* tab = (G1*)w; w += szTab;
    G1* tabQ = (G1*)w; w += szTQ;
    G1* T = (G1*)w; w += szT;
    G1* gbuf[2]; gbuf[0] = (G1*)w; w += szG; gbuf[1] = (G1*)w; w += szG;
    Fr* abuf[2]; abuf[0] = (Fr*)w; w += szF; abuf[1] = (Fr*)w; w += szF;
    Fr* bbuf[2]; bbuf[0] = (Fr*)w; w += szF; bbuf[1] = (Fr*)w; w += szF;
    G1* Ld = (G1*)w; w += szP;
    G1* Rd = (G1*)w; w += szP;
    Fr* sc = (Fr*)w;                              // c_L, c_R, x, 1/x
    G1* QT = (G1*)(sc + 8);                       // c_L Q, c_R Q
    G1* Qd = QT + 2;
    ZkhCtl* hc = c->h_ctl;
    digest_from_bytes(state, hc->st);
    hc->counter = 0;
    hc->err = 0;
    ZKH_CUDA(c, cudaMemcpyAsync(c->d_ctl, hc, offsetof(ZkhCtl, local), cudaMemcpyHostToDevice, c->stream));
    const ZkhTag tagL = zkh_make_tag("L"), tagR = zkh_make_tag("R");
    const Fr* a = (const Fr*)a_dev;
    const Fr* b = (const Fr*)b_dev;
    const G1* g = (const G1*)g_dev;
    if (n > 1) {
        ZKH_CUDA(c, cudaMemcpyAsync(Qd, Q144, sizeof(G1), cudaMemcpyHostToDevice, c->stream));
        g1_table_kernel<<<1, G1_WARP, 0, c->stream>>>(Qd, 1, tabQ);
        g1_table_kernel<<<warp_blocks(n), G1_WARP, 0, c->stream>>>(g, n, tab);
    }
    uint32_t r = 0;
    for (uint32_t sz = n; sz > 1; sz /= 2, r++) {
        const uint32_t h = sz / 2;
        ipa_dot_kernel<<<2, FR_THREADS, 0, c->stream>>>(a, b, h, sc);
        // T[0..h) = a_lo[i] g_hi[i] (the terms of L), T[h..2h) = a_hi[i] g_lo[i] (of R); QT = c_L Q, c_R Q
        ChainSeg A = {tab, a, T, sz, sz, h, sz - 1, 0u}, B = {tabQ, sc, QT, 1u, 2u, 0u, 0u, 0u};
        g1_chain_kernel<<<warp_blocks((size_t)sz + 2), G1_WARP, 0, c->stream>>>(A, B);
        ZKH_TRY(g1_tree_enqueue(c, T, h, h, 2));
        ipa_round_end_kernel<<<1, G1_WARP, 0, c->stream>>>(T, h, QT, c->d_ctl, Ld + r, Rd + r, sc, tagL, tagR);
        // W[0..h) = x^-1 g_lo[i], W[h..2h) = x g_hi[i]
        ChainSeg F = {tab, sc + 2, T, sz, sz, 0u, sz - 1, 2u}, none = {nullptr, nullptr, nullptr, 0u, 0u, 0u, 0u, 0u};
        g1_chain_kernel<<<warp_blocks(sz), G1_WARP, 0, c->stream>>>(F, none);
        Fr* a2 = abuf[r & 1];
        Fr* b2 = bbuf[r & 1];
        G1* g2 = gbuf[r & 1];
        ipa_fold_kernel<<<warp_blocks(h), G1_WARP, 0, c->stream>>>(a, b, T, sc, h, a2, b2, g2, tab);
        a = a2; b = b2; g = g2;
    }
    ZKH_CUDA(c, cudaGetLastError());
    ZKH_CUDA(c, cudaMemcpyAsync(hc, c->d_ctl, offsetof(ZkhCtl, local), cudaMemcpyDeviceToHost, c->stream));
    if (rounds) {
        ZKH_CUDA(c, cudaMemcpyAsync(L_out, Ld, (size_t)rounds * sizeof(G1), cudaMemcpyDeviceToHost, c->stream));
        ZKH_CUDA(c, cudaMemcpyAsync(R_out, Rd, (size_t)rounds * sizeof(G1), cudaMemcpyDeviceToHost, c->stream));
    }
    ZKH_CUDA(c, cudaMemcpyAsync(a_final32, a, sizeof(Fr), cudaMemcpyDeviceToHost, c->stream));
    ZKH_CUDA(c, cudaStreamSynchronize(c->stream));
    if (hc->err) return zkh_fail(c, ZKH_ERR_DEVICE, "g1_ipa_prove: device error flag set");
    digest_to_bytes(hc->st, state);
    return ZKH_OK;
}

extern "C" int zkh_g1_ipa_verify(zkh_ctx* c, const void* g_dev, uint32_t n, const void* Q144, const void* P0_144, const void* u_b,
                                 const void* L, const void* R, const void* a_final32, uint8_t state[32], int* accept) {
    if (!c || !g_dev || !Q144 || !P0_144 || !a_final32 || !state || !accept)
        return zkh_fail(c, ZKH_ERR_ARG, "g1_ipa_verify: null pointer");
    if (!pow2(n) || n > G1_MAX_N) return zkh_fail(c, ZKH_ERR_ARG, "g1_ipa_verify: n must be a power of two up to 2^20");
    uint32_t rounds = 0;
    while ((1u << rounds) < n) rounds++;
    if (rounds && (!u_b || !L || !R)) return zkh_fail(c, ZKH_ERR_ARG, "g1_ipa_verify: null proof buffer");
    if ((uintptr_t)g_dev & 15) return zkh_fail(c, ZKH_ERR_ARG, "g1_ipa_verify: buffer must be 16-byte aligned");
    if (!fr_canonical((const uint32_t*)a_final32)) return zkh_fail(c, ZKH_ERR_DOMAIN, "g1_ipa_verify: final scalar not below p");
    for (uint32_t r = 0; r < rounds; r++)
        if (!fr_canonical((const uint32_t*)u_b + 8 * r)) return zkh_fail(c, ZKH_ERR_DOMAIN, "g1_ipa_verify: point not below p");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    const uint32_t nm = 2 * rounds + 1;                        // L_r, R_r interleaved, then Q
    const size_t szTab = zkh_align((size_t)n * G1_BITS * sizeof(G1)), szTM = zkh_align((size_t)nm * G1_BITS * sizeof(G1));
    const size_t szT = zkh_align((size_t)n * sizeof(G1)), szM = zkh_align((size_t)(nm + 1) * sizeof(G1));
    const size_t szS = zkh_align((size_t)n * sizeof(Fr)), szX = zkh_align((size_t)(5 * IPA_MAX_ROUNDS + 8) * sizeof(Fr));
    ZKH_TRY(zkh_ws_reserve(c, szTab + szTM + szT + 2 * szM + szS + szX + 256));
    char* w = (char*)c->ws;
    G1* tab = (G1*)w; w += szTab;
    G1* tabM = (G1*)w; w += szTM;
    G1* T = (G1*)w; w += szT;
    G1* pts = (G1*)w; w += szM;                               // nm points, then P0
    G1* M = (G1*)w; w += szM;
    Fr* s = (Fr*)w; w += szS;
    Fr* xs = (Fr*)w;
    Fr* xis = xs + IPA_MAX_ROUNDS;
    Fr* sq = xis + IPA_MAX_ROUNDS;                            // 2 rounds + 2
    Fr* ud = sq + 2 * IPA_MAX_ROUNDS + 2;
    Fr* afd = ud + IPA_MAX_ROUNDS;
    w += szX;
    int* acc_dev = (int*)w;
    ZkhCtl* hc = c->h_ctl;
    digest_from_bytes(state, hc->st);
    hc->counter = 0;
    hc->err = 0;
    ZKH_CUDA(c, cudaMemcpyAsync(c->d_ctl, hc, offsetof(ZkhCtl, local), cudaMemcpyHostToDevice, c->stream));
    for (uint32_t r = 0; r < rounds; r++) {
        ZKH_CUDA(c, cudaMemcpyAsync(pts + 2 * r, (const char*)L + (size_t)r * sizeof(G1), sizeof(G1), cudaMemcpyHostToDevice, c->stream));
        ZKH_CUDA(c, cudaMemcpyAsync(pts + 2 * r + 1, (const char*)R + (size_t)r * sizeof(G1), sizeof(G1), cudaMemcpyHostToDevice, c->stream));
    }
    ZKH_CUDA(c, cudaMemcpyAsync(pts + 2 * rounds, Q144, sizeof(G1), cudaMemcpyHostToDevice, c->stream));
    ZKH_CUDA(c, cudaMemcpyAsync(pts + nm, P0_144, sizeof(G1), cudaMemcpyHostToDevice, c->stream));
    if (rounds) ZKH_CUDA(c, cudaMemcpyAsync(ud, u_b, (size_t)rounds * sizeof(Fr), cudaMemcpyHostToDevice, c->stream));
    ZKH_CUDA(c, cudaMemcpyAsync(afd, a_final32, sizeof(Fr), cudaMemcpyHostToDevice, c->stream));
    ipa_verify_transcript_kernel<<<1, G1_WARP, 0, c->stream>>>(pts, rounds, ud, afd, c->d_ctl, xs, xis, sq, zkh_make_tag("L"),
                                                               zkh_make_tag("R"));
    ipa_svec_kernel<<<(n + FR_THREADS - 1) / FR_THREADS, FR_THREADS, 0, c->stream>>>(xs, xis, rounds, n, s);
    g1_table_kernel<<<warp_blocks(nm), G1_WARP, 0, c->stream>>>(pts, nm, tabM);
    g1_table_kernel<<<warp_blocks(n), G1_WARP, 0, c->stream>>>((const G1*)g_dev, n, tab);
    ChainSeg A = {tab, s, T, n, n, 0u, 0xffffffffu, 0u}, B = {tabM, sq, M, nm, nm, 0u, 0xffffffffu, 0u};
    g1_chain_kernel<<<warp_blocks((size_t)n + nm), G1_WARP, 0, c->stream>>>(A, B);
    ZKH_TRY(g1_tree_enqueue(c, T, 0, n, 1));
    ipa_verify_final_kernel<<<1, 4, 0, c->stream>>>(M, rounds, pts + nm, T, afd, acc_dev);
    ZKH_CUDA(c, cudaGetLastError());
    int acc = 0;
    ZKH_CUDA(c, cudaMemcpyAsync(hc, c->d_ctl, offsetof(ZkhCtl, local), cudaMemcpyDeviceToHost, c->stream));
    ZKH_CUDA(c, cudaMemcpyAsync(&acc, acc_dev, sizeof(int), cudaMemcpyDeviceToHost, c->stream));
    ZKH_CUDA(c, cudaStreamSynchronize(c->stream));
    if (hc->err) return zkh_fail(c, ZKH_ERR_DEVICE, "g1_ipa_verify: device error flag set");
    digest_to_bytes(hc->st, state);
    *accept = acc;
    return ZKH_OK;
}

extern "C" int zkh_g1_rows_check(zkh_ctx* c, const void* lhs_dev, const void* a_dev, const void* s32, const void* b_dev, uint32_t rows,
                                 uint32_t* n_bad) {
    if (!c || !lhs_dev || !a_dev || !s32 || !b_dev || !n_bad) return zkh_fail(c, ZKH_ERR_ARG, "g1_rows_check: null pointer");
    if (!rows) return zkh_fail(c, ZKH_ERR_ARG, "g1_rows_check: no rows");
    if (((uintptr_t)lhs_dev | (uintptr_t)a_dev | (uintptr_t)b_dev) & 15) return zkh_fail(c, ZKH_ERR_ARG, "g1_rows_check: buffers must be 16-byte aligned");
    if (!fr_canonical((const uint32_t*)s32)) return zkh_fail(c, ZKH_ERR_DOMAIN, "g1_rows_check: scalar not below p");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    ZKH_TRY(zkh_ws_reserve(c, 256));
    unsigned int* bad = (unsigned int*)c->ws;
    Fr s;
    memcpy(s.v, s32, 32);
    ZKH_CUDA(c, cudaMemsetAsync(bad, 0, sizeof(unsigned int), c->stream));
    g1_rows_check_kernel<<<warp_blocks(rows), G1_WARP, 0, c->stream>>>((const G1*)lhs_dev, (const G1*)a_dev, (const G1*)b_dev, s, rows, bad);
    ZKH_CUDA(c, cudaGetLastError());
    ZKH_CUDA(c, cudaMemcpyAsync(n_bad, bad, sizeof(unsigned int), cudaMemcpyDeviceToHost, c->stream));
    ZKH_CUDA(c, cudaStreamSynchronize(c->stream));
    return ZKH_OK;
}

extern "C" int zkh_g1_rows_add(zkh_ctx* c, const void* a_dev, const void* b_dev, uint32_t rows, void* out_dev) {
    if (!c || !a_dev || !b_dev || !out_dev) return zkh_fail(c, ZKH_ERR_ARG, "g1_rows_add: null pointer");
    if (!rows) return zkh_fail(c, ZKH_ERR_ARG, "g1_rows_add: no rows");
    if (((uintptr_t)a_dev | (uintptr_t)b_dev | (uintptr_t)out_dev) & 15) return zkh_fail(c, ZKH_ERR_ARG, "g1_rows_add: buffers must be 16-byte aligned");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    g1_rows_add_kernel<<<warp_blocks(rows), G1_WARP, 0, c->stream>>>((const G1*)a_dev, (const G1*)b_dev, rows, (G1*)out_dev);
    ZKH_CUDA(c, cudaGetLastError());
    return ZKH_OK;
}

extern "C" int zkh_g1_rows_lincomb(zkh_ctx* c, const void* a_dev, const void* s32, const void* b_dev, uint32_t rows, int mul_first, void* out_dev) {
    if (!c || !a_dev || !s32 || !b_dev || !out_dev) return zkh_fail(c, ZKH_ERR_ARG, "g1_rows_lincomb: null pointer");
    if (!rows) return zkh_fail(c, ZKH_ERR_ARG, "g1_rows_lincomb: no rows");
    if (((uintptr_t)a_dev | (uintptr_t)b_dev | (uintptr_t)out_dev) & 15) return zkh_fail(c, ZKH_ERR_ARG, "g1_rows_lincomb: buffers must be 16-byte aligned");
    if (!fr_canonical((const uint32_t*)s32)) return zkh_fail(c, ZKH_ERR_DOMAIN, "g1_rows_lincomb: scalar not below p");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    Fr s;
    memcpy(s.v, s32, 32);
    g1_rows_lincomb_kernel<<<warp_blocks(rows), G1_WARP, 0, c->stream>>>((const G1*)a_dev, s, (const G1*)b_dev, rows, mul_first, (G1*)out_dev);
    ZKH_CUDA(c, cudaGetLastError());
    return ZKH_OK;
}
