// logUp over BLS12-381 Fr as the reference's first stack runs it (tLookup): helper columns
// A = 1/(S+beta), B = 1/(T+beta) and the two-phase sumcheck that ties them to the witness S, the table T
// and the multiplicities m.
//
// Reference: tlookup_inv_kernel (zkllm-src/tlookup.cu:50-62, one Fermat inversion per element),
// tLookup_phase1_step_poly / phase2_step_poly (tlookup.cu:184-296: five to nine temporaries of half size, an
// MLE evaluation of each of them and several tree sums per round), fs_phase1 / fs_phase2
// (zkllm-src/zkob_lookup.cuh:143-198: transcript per round, five fold kernels).
//
// Per round the reference evaluates  sum_i eq(u_, i) * x_i(t)  by folding a temporary along u_.  The eq
// table of u_ for the next round is the pairwise sum of this round's table over its top bit, so here ONE
// table is built once and halved along with the columns.  A round is one kernel: bind the columns with the
// previous challenge, fold the eq table, accumulate the 5 (phase 1) or 11 (phase 2) sums the round
// polynomial needs, reduce over the grid, assemble p(0..3) from the sums and the running scalars on the
// device, absorb, draw the challenge, update the scalars.
#include "fr_dev.cuh"

namespace zkh {

// running scalars of one lookup sumcheck (plain values), device resident
struct FrLuState {
    Fr alpha_run;   // alpha * prod eq(u_last, v) so far
    Fr alpha_sq;    // alpha^2 * prod eq(...) over the phase-2 rounds so far
    Fr C;           // phase-1 constant, halved every phase-1 round
    Fr inv_ratio;   // N / D
    Fr beta;
    Fr u[32];       // the point, u[k-1] is consumed by the round on columns of 2^k entries
};

struct LuPtrs {
    const Fr* in[5];   // A S B T m
    Fr* out[5];
    const Fr* Ein;
    Fr* Eout;
};

__device__ __forceinline__ Fr fr_mulp(const Fr& a, const Fr& b) { return fr_mmul(fr_mmul(a, b), FR_RPOW[1]); }  // plain * plain
__device__ __forceinline__ Fr fr_small(uint32_t x) { Fr r = fr_zero(); r.v[0] = x; return r; }
// value at 3 of the quadratic through (0, a), (1, b), (2, c)
__device__ __forceinline__ Fr fr_extrap3(const Fr& a, const Fr& b, const Fr& c) {
    Fr d = fr_sub(c, b);
    Fr t = fr_add(fr_add(d, d), d);
    return fr_add(t, a);
}

// PHASE 1: arrays A, S.  PHASE 2: arrays A, S, B, T, m.
// pend bit k: array k arrives with 4h entries and is bound with *chal_prev first (else it has 2h entries);
// pend bit 5: the eq table arrives with 2h entries and is folded (else it has h entries).
template <int PHASE>
__global__ void __launch_bounds__(FR_THREADS)
fr_lu_round_kernel(LuPtrs P, size_t h, uint32_t pend, uint32_t k, FrLuState* stt, ZkhCtl* ctl, Fr* partials,
                   const Fr* chal_prev, Fr* msg_out, Fr* chal_out) {
    constexpr int NA = PHASE == 1 ? 2 : 5;
    constexpr int NS = PHASE == 1 ? 5 : 11;   // PA0..2, Q0, Q1 | PB0..2, M0..2
    __shared__ __align__(16) Fr sh[NS * 32];
    Fr xm = fr_zero();
    if (pend & 31u) xm = fr_to_mont(*chal_prev);
    const Fr beta = stt->beta;
    Fr acc[NS];
#pragma unroll
    for (int t = 0; t < NS; t++) acc[t] = fr_zero();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < h; i += stride) {
        Fr lo[NA], df[NA];
#pragma unroll
        for (int a = 0; a < NA; a++) {
            Fr x0, x1;
            if (pend & (1u << a)) {
                x0 = fr_lerp(fr_load(P.in[a] + i), fr_load(P.in[a] + i + 2 * h), xm);
                x1 = fr_lerp(fr_load(P.in[a] + i + h), fr_load(P.in[a] + i + 3 * h), xm);
                fr_store(P.out[a] + i, x0);
                fr_store(P.out[a] + i + h, x1);
            } else {
                x0 = fr_load(P.in[a] + i);
                x1 = fr_load(P.in[a] + i + h);
            }
            lo[a] = x0;
            df[a] = fr_sub(x1, x0);
        }
        Fr e;
        if (pend & 32u) {
            e = fr_add(fr_load(P.Ein + i), fr_load(P.Ein + i + h));
            fr_store(P.Eout + i, e);
        } else {
            e = fr_load(P.Ein + i);
        }
        acc[3] = fr_add(acc[3], lo[0]);
        acc[4] = fr_add(acc[4], df[0]);
        Fr a_t = lo[0], s_t = fr_add(lo[1], beta);
#pragma unroll
        for (int t = 0; t < 3; t++) {
            acc[t] = fr_add(acc[t], fr_mmul(fr_mmul(e, a_t), s_t));      // carries R^-2
            if (t < 2) { a_t = fr_add(a_t, df[0]); s_t = fr_add(s_t, df[1]); }
        }
        if (PHASE == 2) {
            Fr b_t = lo[2], t_t = fr_add(lo[3], beta), m_t = lo[4];
#pragma unroll
            for (int t = 0; t < 3; t++) {
                acc[5 + t] = fr_add(acc[5 + t], fr_mmul(fr_mmul(e, b_t), t_t));   // R^-2
                acc[8 + t] = fr_add(acc[8 + t], fr_mmul(m_t, b_t));               // R^-1
                if (t < 2) { b_t = fr_add(b_t, df[2]); t_t = fr_add(t_t, df[3]); m_t = fr_add(m_t, df[4]); }
            }
        }
    }
    // grid reduction through the last CTA to finish
    __shared__ int is_last;
    fr_block_sum<NS>(acc, sh);
    if (threadIdx.x == 0) {
#pragma unroll
        for (int t = 0; t < NS; t++) partials[(size_t)blockIdx.x * NS + t] = acc[t];
        __threadfence();
        is_last = (atomicAdd(&ctl->counter, 1u) == gridDim.x - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
#pragma unroll
    for (int t = 0; t < NS; t++) acc[t] = fr_zero();
    for (unsigned b = threadIdx.x; b < gridDim.x; b += blockDim.x)
#pragma unroll
        for (int t = 0; t < NS; t++) {
            const volatile uint32_t* src = reinterpret_cast<const volatile uint32_t*>(&partials[(size_t)b * NS + t]);
            Fr x;
#pragma unroll
            for (int j = 0; j < 8; j++) x.v[j] = src[j];
            acc[t] = fr_add(acc[t], x);
        }
    fr_block_sum<NS>(acc, sh);
    if (threadIdx.x >= 32) return;
    // ---- round end on warp 0 ----
    __shared__ uint32_t trbuf[ZKH_TRBUF_WORDS];
    __shared__ __align__(16) Fr ev[4];
    const uint32_t lane = threadIdx.x;
    if (lane == 0) {
        ctl->counter = 0;
        Fr pa[4], q[4], pb[4], mm[4];
        for (int t = 0; t < 3; t++) pa[t] = fr_mmul(acc[t], FR_RPOW[2]);
        pa[3] = fr_extrap3(pa[0], pa[1], pa[2]);
        q[0] = acc[3];
        for (int t = 1; t < 4; t++) q[t] = fr_add(q[t - 1], acc[4]);
        const Fr ul = stt->u[k - 1], one = fr_small(1);
        const Fr nul = fr_sub(one, ul), slope = fr_sub(ul, nul);        // eq_last(t) = (1-ul) + t*(2ul-1)
        Fr eqt = nul;
        const Fr ar = stt->alpha_run;
        Fr cterm = fr_zero(), coef = fr_zero(), ir = stt->inv_ratio;
        if (PHASE == 1) {
            Fr inv2 = fr_small(0);   // (p+1)/2
            inv2.v[0] = 0x80000001u; inv2.v[1] = 0x7fffffffu; inv2.v[2] = 0x7fff2dffu; inv2.v[3] = 0xa9ded201u;
            inv2.v[4] = 0x04d0ec02u; inv2.v[5] = 0x199cec04u; inv2.v[6] = 0x94cebea4u; inv2.v[7] = 0x39f6d3a9u;
            cterm = fr_mulp(stt->C, inv2);
            stt->C = cterm;                                              // halved for the next phase-1 round
        } else {
            for (int t = 0; t < 3; t++) { pb[t] = fr_mmul(acc[5 + t], FR_RPOW[2]); mm[t] = fr_mmul(acc[8 + t], FR_RPOW[1]); }
            pb[3] = fr_extrap3(pb[0], pb[1], pb[2]);
            mm[3] = fr_extrap3(mm[0], mm[1], mm[2]);
            coef = fr_mulp(ir, stt->alpha_sq);
        }
        for (int t = 0; t < 4; t++) {
            Fr inner = fr_mulp(ar, pa[t]);
            if (PHASE == 2) inner = fr_add(inner, fr_mulp(coef, pb[t]));
            Fr e = fr_add(fr_mulp(eqt, inner), q[t]);
            e = PHASE == 1 ? fr_add(e, cterm) : fr_sub(e, fr_mulp(ir, mm[t]));
            ev[t] = e;
            msg_out[t] = e;
            eqt = fr_add(eqt, slope);
        }
    }
    __syncwarp();
    uint32_t st[8];
#pragma unroll
    for (int j = 0; j < 8; j++) st[j] = ctl->st[j];
    const char lab[4][3] = {"p0", "p1", "p2", "p3"};
    for (int t = 0; t < 4; t++) tr_warp_absorb(st, lab[t], 2, reinterpret_cast<const uint64_t*>(&ev[t]), 4, trbuf);
    Fr v;
    bool ok = false;
    for (int tries = 0; tries < 8 && !ok; tries++) {
        tr_warp_challenge_limbs(st, v.v);
        v.v[7] %= 0x73eda753u;
        ok = !fr_is_zero(v);
    }
    if (lane == 0) {
        if (!ok) atomicOr(&ctl->err, 2u);
#pragma unroll
        for (int j = 0; j < 8; j++) ctl->st[j] = st[j];
        *chal_out = v;
        const Fr ul = stt->u[k - 1], one = fr_small(1);
        const Fr eqv = fr_add(fr_mulp(ul, v), fr_mulp(fr_sub(one, ul), fr_sub(one, v)));
        stt->alpha_run = fr_mulp(stt->alpha_run, eqv);
        if (PHASE == 2) stt->alpha_sq = fr_mulp(stt->alpha_sq, eqv);
    }
}

// alpha^2 and N/D = 2^-(logD-logN) from the values the host stored (alpha in alpha_run)
__global__ void fr_lu_setup_kernel(FrLuState* stt, uint32_t logD, uint32_t logN) {
    Fr inv2;
    inv2.v[0] = 0x80000001u; inv2.v[1] = 0x7fffffffu; inv2.v[2] = 0x7fff2dffu; inv2.v[3] = 0xa9ded201u;
    inv2.v[4] = 0x04d0ec02u; inv2.v[5] = 0x199cec04u; inv2.v[6] = 0x94cebea4u; inv2.v[7] = 0x39f6d3a9u;
    stt->alpha_sq = fr_mulp(stt->alpha_run, stt->alpha_run);
    Fr r = fr_small(1);
    for (uint32_t i = logN; i < logD; i++) r = fr_mulp(r, inv2);
    stt->inv_ratio = r;
}

// terminals: each array has two entries left; bind with the last challenge
__global__ void fr_lu_finals_kernel(LuPtrs P, uint32_t pend, const Fr* chal, Fr* out) {
    int a = threadIdx.x;
    if (a < 5) out[a] = (pend & (1u << a)) ? fr_lerp(P.in[a][0], P.in[a][1], fr_to_mont(*chal)) : P.in[a][0];
}

// out[i] = 1/(in[i] + beta), 0 where the denominator is 0 (as the reference's inverse of 0); plain values.
// Eight strided elements per thread share one Fermat inversion (prefix products, peel back).
#define FR_INV_K 8
__global__ void __launch_bounds__(FR_THREADS) fr_inv_add_kernel(const Fr* in, Fr beta, Fr* out, size_t n) {
    const size_t nth = (size_t)gridDim.x * blockDim.x, t0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    Fr d[FR_INV_K], pre[FR_INV_K];
    Fr run = FR_RPOW[0];
    uint32_t zero_mask = 0;
#pragma unroll
    for (int k = 0; k < FR_INV_K; k++) {
        const size_t i = t0 + (size_t)k * nth;
        Fr x = FR_RPOW[0];
        if (i < n) {
            Fr s = fr_add(fr_load(in + i), beta);
            if (fr_is_zero(s)) zero_mask |= 1u << k;
            else x = fr_to_mont(s);
        }
        d[k] = x;
        pre[k] = run;
        run = fr_mmul(run, x);
    }
    Fr inv = fr_inv_mont(run);
#pragma unroll
    for (int k = FR_INV_K - 1; k >= 0; k--) {
        const size_t i = t0 + (size_t)k * nth;
        Fr r = fr_mmul(inv, pre[k]);
        inv = fr_mmul(inv, d[k]);
        if (i < n) fr_store(out + i, (zero_mask >> k) & 1u ? fr_zero() : fr_from_mont(r));
    }
}

}  // namespace zkh

using namespace zkh;

extern "C" int zkh_fr_inv_add(zkh_ctx* c, const void* in_dev, uint64_t n, const void* beta, void* out_dev) {
    if (!c) return ZKH_ERR_ARG;
    if (!in_dev || !out_dev || !beta) return zkh_fail(c, ZKH_ERR_ARG, "fr_inv_add: null pointer");
    if (!fr_canonical((const uint32_t*)beta)) return zkh_fail(c, ZKH_ERR_DOMAIN, "fr_inv_add: beta not below p");
    if (!n) return ZKH_OK;
    ZKH_CUDA(c, cudaSetDevice(c->device));
    Fr b;
    memcpy(&b, beta, 32);
    const size_t threads = (n + FR_INV_K - 1) / FR_INV_K;
    fr_inv_add_kernel<<<(unsigned)((threads + FR_THREADS - 1) / FR_THREADS), FR_THREADS, 0, c->stream>>>((const Fr*)in_dev, b,
                                                                                                     (Fr*)out_dev, (size_t)n);
    return cudaGetLastError() == cudaSuccess ? ZKH_OK : zkh_fail(c, ZKH_ERR_CUDA, "fr_inv_add launch");
}

extern "C" int zkh_fr_lookup_sumcheck(zkh_ctx* c, const void* A_dev, const void* S_dev, const void* B_dev, const void* T_dev,
                                      const void* m_dev, uint32_t logD, uint32_t logN, const void* alpha, const void* beta,
                                      const void* Cc, const void* u, uint8_t state[32], void* evals, void* ws, void* terminals) {
    if (!c) return ZKH_ERR_ARG;
    if (!A_dev || !S_dev || !B_dev || !T_dev || !m_dev || !alpha || !beta || !Cc || !u || !state || !evals || !ws || !terminals)
        return zkh_fail(c, ZKH_ERR_ARG, "fr_lookup_sumcheck: null pointer");
    if (logN < 1 || logD < logN || logD > 30) return zkh_fail(c, ZKH_ERR_ARG, "fr_lookup_sumcheck: need 1 <= logN <= logD <= 30");
    const void* sc[3] = {alpha, beta, Cc};
    for (auto p : sc)
        if (!fr_canonical((const uint32_t*)p)) return zkh_fail(c, ZKH_ERR_DOMAIN, "fr_lookup_sumcheck: scalar not below p");
    for (uint32_t i = 0; i < logD; i++)
        if (!fr_canonical((const uint32_t*)u + 8 * i)) return zkh_fail(c, ZKH_ERR_DOMAIN, "fr_lookup_sumcheck: point not below p");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    const size_t D = (size_t)1 << logD, N = (size_t)1 << logN;
    const unsigned pcap = 4 * (unsigned)c->sm_count;
    // workspace: state | u copy | eq ping-pong | A,S ping-pong | B,T,m ping-pong | partials | evals | ws | terminals
    const size_t szSt = zkh_align(sizeof(FrLuState)), szE = zkh_align((D / 2 + 1) * 32), szE2 = zkh_align((D / 4 + 1) * 32);
    const size_t szAS = zkh_align(2 * (D / 2 + 1) * 32), szAS2 = zkh_align(2 * (D / 4 + 1) * 32);
    const size_t szB = zkh_align(3 * (N / 2 + 1) * 32), szB2 = zkh_align(3 * (N / 4 + 1) * 32);
    const size_t szP = zkh_align((size_t)pcap * 11 * 32), szEv = zkh_align((size_t)logD * 4 * 32), szW = zkh_align((size_t)logD * 32);
    ZKH_TRY(zkh_ws_reserve(c, szSt + szE + szE2 + szAS + szAS2 + szB + szB2 + szP + szEv + szW + 256));
    char* w = (char*)c->ws;
    FrLuState* stt = (FrLuState*)w; w += szSt;
    Fr* Ebuf[2] = {(Fr*)w, (Fr*)(w + szE)}; w += szE + szE2;
    Fr* ASbuf[2] = {(Fr*)w, (Fr*)(w + szAS)}; w += szAS + szAS2;
    Fr* Bbuf[2] = {(Fr*)w, (Fr*)(w + szB)}; w += szB + szB2;
    Fr* part = (Fr*)w; w += szP;
    Fr* ev = (Fr*)w; w += szEv;
    Fr* wsd = (Fr*)w; w += szW;
    Fr* term = (Fr*)w;
    // running scalars
    FrLuState hs;
    memset(&hs, 0, sizeof hs);
    memcpy(&hs.alpha_run, alpha, 32);
    memcpy(&hs.beta, beta, 32);
    memcpy(&hs.C, Cc, 32);
    memcpy(hs.u, u, (size_t)logD * 32);
    ZKH_CUDA(c, cudaMemcpyAsync(stt, &hs, sizeof hs, cudaMemcpyHostToDevice, c->stream));
    ZkhCtl* h = c->h_ctl;
    digest_from_bytes(state, h->st);
    h->counter = 0;
    h->err = 0;
    for (int i = 0; i < 8; i++) h->par[i] = 0;
    ZKH_CUDA(c, cudaMemcpyAsync(c->d_ctl, h, offsetof(ZkhCtl, local), cudaMemcpyHostToDevice, c->stream));
    fr_lu_setup_kernel<<<1, 1, 0, c->stream>>>(stt, logD, logN);
    // eq table of u[0 .. logD-2] (D/2 entries); every later round folds it by pairwise sums
    ZKH_TRY(fr_eq_enqueue(c, stt->u, (const Fr*)u, logD - 1, Ebuf[0]));
    LuPtrs P;
    memset(&P, 0, sizeof P);
    const Fr* cur[5] = {(const Fr*)A_dev, (const Fr*)S_dev, (const Fr*)B_dev, (const Fr*)T_dev, (const Fr*)m_dev};
    bool pend[5] = {false, false, false, false, false};
    const Fr* curE = Ebuf[0];
    bool pendE = false;
    int as_next = 0, b_next = 0, e_next = 1;
    auto grid_for = [&](size_t items) { unsigned g = fr_grid(c, items, 4); return g < pcap ? g : pcap; };
    uint32_t r = 0;
    for (uint32_t k = logD; k >= 1; k--, r++) {
        const size_t hh = (size_t)1 << (k - 1);          // pairs this round; bound columns have 2*hh entries
        const bool ph2 = k <= logN;
        const int used = ph2 ? 5 : 2;
        uint32_t mask = 0;
        for (int a = 0; a < used; a++) {
            P.in[a] = cur[a];
            P.out[a] = nullptr;
            if (pend[a]) {
                mask |= 1u << a;
                P.out[a] = a < 2 ? ASbuf[as_next] + (size_t)a * (2 * hh) : Bbuf[b_next] + (size_t)(a - 2) * (2 * hh);
            }
        }
        P.Ein = curE;
        P.Eout = nullptr;
        if (pendE) { mask |= 32u; P.Eout = Ebuf[e_next]; }
        const Fr* prev = r ? wsd + (r - 1) : nullptr;
        if (ph2)
            fr_lu_round_kernel<2><<<grid_for(hh), FR_THREADS, 0, c->stream>>>(P, hh, mask, k, stt, c->d_ctl, part, prev,
                                                                            ev + (size_t)r * 4, wsd + r);
        else
            fr_lu_round_kernel<1><<<grid_for(hh), FR_THREADS, 0, c->stream>>>(P, hh, mask, k, stt, c->d_ctl, part, prev,
                                                                            ev + (size_t)r * 4, wsd + r);
        for (int a = 0; a < used; a++) {
            if (pend[a]) cur[a] = P.out[a];
            pend[a] = true;
        }
        if (mask & 3u) as_next ^= 1;
        if (mask & 28u) b_next ^= 1;
        if (pendE) { curE = P.Eout; e_next ^= 1; }
        pendE = true;
    }
    uint32_t pendmask = 0;
    for (int a = 0; a < 5; a++) pendmask |= pend[a] ? (1u << a) : 0u;
    for (int a = 0; a < 5; a++) P.in[a] = cur[a];
    fr_lu_finals_kernel<<<1, 32, 0, c->stream>>>(P, pendmask, wsd + (logD - 1), term);
    if (cudaGetLastError() != cudaSuccess) return zkh_fail(c, ZKH_ERR_CUDA, "fr_lookup_sumcheck launch");
    ZKH_CUDA(c, cudaMemcpyAsync(h, c->d_ctl, offsetof(ZkhCtl, local), cudaMemcpyDeviceToHost, c->stream));
    ZKH_CUDA(c, cudaMemcpyAsync(evals, ev, (size_t)logD * 4 * 32, cudaMemcpyDeviceToHost, c->stream));
    ZKH_CUDA(c, cudaMemcpyAsync(ws, wsd, (size_t)logD * 32, cudaMemcpyDeviceToHost, c->stream));
    ZKH_CUDA(c, cudaMemcpyAsync(terminals, term, 5 * 32, cudaMemcpyDeviceToHost, c->stream));
    ZKH_CUDA(c, cudaStreamSynchronize(c->stream));
    if (h->err) return zkh_fail(c, ZKH_ERR_DEVICE, "fr_lookup_sumcheck: device error flag set");
    digest_to_bytes(h->st, state);
    return ZKH_OK;
}
