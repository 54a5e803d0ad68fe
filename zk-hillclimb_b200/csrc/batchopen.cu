// Batched Basefold openings of one size class for sm_100a (plain and, with per-column salt seeds, the hiding mode's
// salted round-0 openings: zkllm-src/p3_batchopen.cuh:969-1131).
//
// Protocol and transcript: zkllm-src/p3_batchopen.cuh:307-1147 (p3bo::prove_class).
//   mu -> G_t = sum_{claims j at point t} mu^j col_j -> reduction sumcheck of
//   sum_t sum_b G_t(b) eq(z_t,b) ("bo-rm") -> r* -> y*_c = col_c(r*) ("bo-ys") -> rho ->
//   U = sum_c rho^c col_c opened at r* on its own transcript seeded with the class label
//   (round 0 carries no root; its values are opened per column against the columns' own roots
//   at the sorted-unique query positions with a pruned node stream).
//
// The reference runs the reduction with one message kernel + three device-to-host copies +
// a bind launch per round, and builds every helper array (the T point arrays G_t, the T eq tables) with host
// round trips.  Here the T stacked point arrays are treated as ONE sumcheck column of length T*2^v (adjacent
// pairs never straddle two points) and neither G nor the eq tables are materialised at full size:
//   * round 0 reads the claims' columns directly and forms G_t(b) = sum_e mu^e col_e[b] in registers;
//     round 1 reads them once more, binds with the first challenge and stores the halved G (T * 2^(v-1));
//     later rounds run on that array, halving it each time;
//   * eq(z_t, b) is the product of two entries of small per-point factor tables (low and high variables),
//     which are bound with each round's challenge by a tiny kernel instead of being expanded to 2^v entries.
// Workspace of the reduction: 0.75 * T * 2^v elements (3.5 * T * 2^v before).  One kernel per round with the
// transcript on the device; the host synchronises three times per class (after the reduction, after "final",
// after the query gather).
#include <algorithm>
#include <vector>
#include "merkle.cuh"
#include "ntt.cuh"
#include "sumcheck.cuh"

namespace zkh {

int fold_enqueue(zkh_ctx* c, const gl_t* f, gl_t* out, size_t M, uint32_t logM_top, uint32_t shift,
                 const gl_t* beta_ptr, gl_t beta_val, const gl_t* tlo, const gl_t* thi, uint32_t tlb);
int ntt_inverse_tables(zkh_ctx* c, uint32_t logM, const gl_t** lo, const gl_t** hi, uint32_t* lb);

// Gs[t][i] = sum_{e in [estart[t], estart[t+1])} ew[e] * ecol[e][i]   (p3_batchopen.cuh:210-221)
__global__ void __launch_bounds__(256)
bo_gbuild_kernel(const gl_t* const* ecol, const gl_t* ew, const uint32_t* estart, gl_t* Gs, uint32_t T, size_t N) {
    const size_t tot = (size_t)T * N, stride = (size_t)gridDim.x * blockDim.x;
    for (size_t j = (size_t)blockIdx.x * blockDim.x + threadIdx.x; j < tot; j += stride) {
        uint32_t t = (uint32_t)(j / N);
        size_t i = j - (size_t)t * N;
        Acc192 acc;
        acc.clear();
        for (uint32_t e = estart[t]; e < estart[t + 1]; e++) acc.add_prod(ew[e], ecol[e][i]);
        Gs[j] = acc.reduce();
    }
}
// factor tables of eq(., z_t) for T points: out[t][b] = prod_{i<nv} (b_i ? z_t[v0+i] : 1 - z_t[v0+i])
__global__ void bo_eq_small_kernel(const gl_t* zs, uint32_t T, uint32_t v, uint32_t v0, uint32_t nv, gl_t* out) {
    uint32_t j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= (T << nv)) return;
    uint32_t t = j >> nv, b = j & ((1u << nv) - 1);
    const gl_t* z = zs + (size_t)t * v + v0;
    gl_t p = 1;
    for (uint32_t i = 0; i < nv; i++) p = gl_mul(p, ((b >> i) & 1) ? z[i] : gl_sub(1, z[i]));
    out[j] = p;
}
// out[x] = in[2x] + a * (in[2x+1] - in[2x]): one more variable of the eq factor tables bound (tables of 2^k entries per
// point, k >= 1, stacked: pairs never straddle two points)
__global__ void bo_tab_bind_kernel(const gl_t* in, gl_t* out, uint32_t count, const gl_t* chal) {
    const uint32_t x = blockIdx.x * blockDim.x + threadIdx.x;
    if (x < count) out[x] = gl_lerp(in[2 * x], in[2 * x + 1], *chal);
}

// One round of the reduction sumcheck  sum_t sum_b G_t(b) eq_t(b)  over the stacked arrays.
//   logL: log2 of the per-point length L of the arrays whose adjacent pairs form this round's message.
//   FIRST: those arrays are the round's input (round 0).  Otherwise the input has per-point length 2L and is bound with
//          *chal_prev first; the bound array (T * L) is stored to Gout.
//   FROM_COLS: the input G is not stored: G_t[b] = sum_{e in [estart[t], estart[t+1])} ew[e] * ecol[e][b]  (rounds 0 and 1).
//   eq_t(b) at this round's level = lo[(t << lw) | (b & (2^lw - 1))] * hi[(t << hw) | (b >> lw)].
struct BoRed {
    const gl_t* const* ecol;
    const gl_t* ew;
    const uint32_t* estart;
    const gl_t* G;
    gl_t* Gout;
    const gl_t* lo;
    const gl_t* hi;
    uint32_t lw, hw, T, logL;
};
template <bool FROM_COLS, bool FIRST>
__global__ void __launch_bounds__(256)
bo_reduce_kernel(BoRed P, ZkhCtl* ctl, gl_t* partials, const gl_t* chal_prev, gl_t* msg_out, gl_t* chal_out, ZkhTag tag) {
    __shared__ gl_t sh[3 * 32];
    Acc192 acc[3];
#pragma unroll
    for (int t = 0; t < 3; t++) acc[t].clear();
    const uint32_t lp = P.logL - 1;                       // pairs per point = 2^lp
    const size_t items = (size_t)P.T << lp, stride = (size_t)gridDim.x * blockDim.x;
    const gl_t a = FIRST ? 0 : *chal_prev;
    const uint32_t lmask = (1u << P.lw) - 1;
    for (size_t j = (size_t)blockIdx.x * blockDim.x + threadIdx.x; j < items; j += stride) {
        const uint32_t t = (uint32_t)(j >> lp);
        const size_t i = j & (((size_t)1 << lp) - 1);
        gl_t g0, g1;
        if (FIRST) {
            if (FROM_COLS) {
                Acc192 s0, s1;
                s0.clear(); s1.clear();
                for (uint32_t e = P.estart[t]; e < P.estart[t + 1]; e++) {
                    const gl_t w = P.ew[e];
                    const ulonglong2 v = ld2(P.ecol[e] + 2 * i);
                    s0.add_prod(w, v.x); s1.add_prod(w, v.y);
                }
                g0 = s0.reduce(); g1 = s1.reduce();
            } else {
                const ulonglong2 v = ld2(P.G + ((size_t)t << P.logL) + 2 * i);
                g0 = v.x; g1 = v.y;
            }
        } else {
            gl_t q[4];
            if (FROM_COLS) {
                Acc192 s4[4];
#pragma unroll
                for (int u = 0; u < 4; u++) s4[u].clear();
                for (uint32_t e = P.estart[t]; e < P.estart[t + 1]; e++) {
                    const gl_t w = P.ew[e];
                    const ulonglong2 v0 = ld2(P.ecol[e] + 4 * i), v1 = ld2(P.ecol[e] + 4 * i + 2);
                    s4[0].add_prod(w, v0.x); s4[1].add_prod(w, v0.y); s4[2].add_prod(w, v1.x); s4[3].add_prod(w, v1.y);
                }
#pragma unroll
                for (int u = 0; u < 4; u++) q[u] = s4[u].reduce();
            } else {
                const gl_t* src = P.G + ((size_t)t << (P.logL + 1)) + 4 * i;
                const ulonglong2 v0 = ld2(src), v1 = ld2(src + 2);
                q[0] = v0.x; q[1] = v0.y; q[2] = v1.x; q[3] = v1.y;
            }
            g0 = gl_lerp(q[0], q[1], a);
            g1 = gl_lerp(q[2], q[3], a);
            st2(P.Gout + ((size_t)t << P.logL) + 2 * i, g0, g1);
        }
        const size_t b0 = 2 * i, b1 = 2 * i + 1;
        const gl_t* lo = P.lo + ((size_t)t << P.lw);
        const gl_t* hi = P.hi + ((size_t)t << P.hw);
        const gl_t e0 = gl_mul(lo[b0 & lmask], hi[b0 >> P.lw]);
        const gl_t e1 = gl_mul(lo[b1 & lmask], hi[b1 >> P.lw]);
        acc[0].add_prod(g0, e0);
        acc[1].add_prod(g1, e1);
        acc[2].add_prod(gl_sub(g1, g0), gl_sub(e1, e0));
    }
    gl_t sm[3];
#pragma unroll
    for (int t = 0; t < 3; t++) sm[t] = acc[t].reduce();
    // evaluations at 0, 1, 2 from g(0), g(1) and the leading coefficient: g(2) = 2 g(1) - g(0) + 2 c2
    sm[2] = gl_add(gl_sub(gl_dbl(sm[1]), sm[0]), gl_dbl(sm[2]));
    grid_finish<3>(sm, sh, ctl, partials, msg_out, chal_out, tag, 0);
}
// ystar[c] = sum_i col_c[i] * w[i]: one CTA per (column, slice), then a per-column sum
__global__ void __launch_bounds__(256)
bo_dots_kernel(const gl_t* const* cols, const gl_t* __restrict__ w, size_t N, gl_t* partials, uint32_t nb) {
    __shared__ gl_t sh[32];
    const uint32_t c = blockIdx.y;
    const gl_t* col = cols[c];
    Acc192 acc;
    acc.clear();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < N; i += (size_t)nb * blockDim.x)
        acc.add_prod(col[i], w[i]);
    gl_t s[1] = {acc.reduce()};
    block_sum<1>(s, sh);
    if (threadIdx.x == 0) partials[(size_t)c * nb + blockIdx.x] = s[0];
}
__global__ void bo_dots_sum_kernel(const gl_t* partials, uint32_t nb, gl_t* out) {
    __shared__ gl_t sh[32];
    gl_t s[1] = {0};
    for (uint32_t i = threadIdx.x; i < nb; i += blockDim.x) s[0] = gl_add(s[0], partials[(size_t)blockIdx.x * nb + i]);
    block_sum<1>(s, sh);
    if (threadIdx.x == 0) out[blockIdx.x] = s[0];
}
// where the capped tree of every fold round starts inside the tree region, and how many low levels it leaves out
struct BoTrees { size_t off[32]; uint32_t cut[32]; };
// openings of rounds 1..v-1 straight into the proof's query section: values and the path siblings from the capped trees
// (levels below a round's cut come from merkle_low_paths_enqueue)
__global__ void bo_query_kernel(const gl_t* cw_rest, const uint8_t* trees, BoTrees bt, uint32_t logM0, uint32_t v, uint32_t Q,
                                const uint32_t* pos /* [Q][v] */, uint8_t* out, size_t per_query) {
    uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= Q * (v - 1) * 2) return;
    const uint32_t side = t & 1, e = t >> 1, q = e / (v - 1), r = 1 + e % (v - 1);
    const size_t M0 = (size_t)1 << logM0, Mr = M0 >> r, h = Mr / 2;
    const uint32_t plen = logM0 - r, cut = bt.cut[r];
    const gl_t* cw = cw_rest + (M0 - 2 * Mr);
    const uint8_t* tree = trees + bt.off[r];
    const size_t Mt = Mr >> cut;
    const size_t idx = (size_t)pos[q * v + r] + (side ? h : 0);
    // offset of round r within a query: sum_{i=1}^{r-1} (16 + 64*(logM0-i))
    const size_t rr = r - 1;
    size_t off = (size_t)q * per_query + rr * 16 + 64 * (rr * logM0 - rr * (rr + 1) / 2);
    uint8_t* o = out + off;
    *reinterpret_cast<gl_t*>(o + 8 * side) = cw[idx];
    uint4* po = reinterpret_cast<uint4*>(o + 16 + (size_t)side * plen * 32);
    size_t id = idx >> cut;
    for (uint32_t l = cut; l < plen; l++) {
        size_t cnt = Mt >> (l - cut);
        const uint4* src = reinterpret_cast<const uint4*>(tree + (2 * Mt - 2 * cnt + (id ^ 1)) * 32);
        po[2 * l] = src[0];
        po[2 * l + 1] = src[1];
        id >>= 1;
    }
}
// round-0 opening of one column: values and the authentication-path siblings of levels cut..logM0-1 at the nu positions,
// read from a capped tree (the lowest `cut` siblings come from merkle_low_paths_enqueue)
// out: [nu] values (8 bytes each) then [nu][logM0] digests
__global__ void bo_q0_kernel(const gl_t* cw, const uint8_t* tree, uint32_t logM0, uint32_t cut, const uint32_t* upos, uint32_t nu,
                             uint8_t* out) {
    uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= nu * (logM0 + 1)) return;
    const uint32_t i = t / (logM0 + 1), l = t % (logM0 + 1);
    if (l == logM0) {
        reinterpret_cast<gl_t*>(out)[i] = cw[upos[i]];
        return;
    }
    if (l < cut) return;
    const size_t Mt = (size_t)1 << (logM0 - cut);
    size_t cnt = Mt >> (l - cut), sib = ((size_t)upos[i] >> l) ^ 1;
    const uint4* src = reinterpret_cast<const uint4*>(tree + (2 * Mt - 2 * cnt + sib) * 32);
    uint4* dst = reinterpret_cast<uint4*>(out + (size_t)nu * 8 + ((size_t)i * logM0 + l) * 32);
    dst[0] = src[0];
    dst[1] = src[1];
}

static size_t bo_bound(uint32_t v, uint32_t R, uint32_t Q, uint32_t nc) {
    size_t s = 16 + (size_t)nc * 8 + (size_t)v * 48 + (size_t)(v ? v - 1 : 0) * 32 + ((size_t)8 << R);
    for (uint32_t r = 1; r < v; r++) s += (size_t)Q * (16 + 2 * (size_t)(v + R - r) * 32);
    s += (size_t)nc * (8 + (size_t)2 * Q * 8 + (size_t)2 * Q * (v + R) * 32);
    return s;
}

}  // namespace zkh

using namespace zkh;

extern "C" size_t zkh_batchopen_proof_bound(uint32_t v, uint32_t R, uint32_t Q, uint32_t ncols) {
    return bo_bound(v, R, Q, ncols);
}

static int batchopen_prove_class(zkh_ctx* c, uint32_t v, const uint64_t* pts, uint32_t T,
                                 const uint64_t* const* cols_dev, const uint8_t* roots, const uint32_t* zid,
                                 uint32_t k, uint32_t R, uint32_t Q, const char* label, uint8_t state[32],
                                 uint8_t* out, size_t cap, size_t* written, const uint64_t* const* kept_cw,
                                 const uint8_t* const* kept_tree, const uint64_t* sseeds = nullptr) {
    if (!c || !pts || !cols_dev || !roots || !zid || !label || !state || !out || !written)
        return zkh_fail(c, ZKH_ERR_ARG, "batchopen: null pointer");
    if (v < 1 || R < 1 || R > 3 || v + R > 30) return zkh_fail(c, ZKH_ERR_ARG, "batchopen: need v >= 1, R in 1..3, v+R <= 30");
    if (v > 64) return zkh_fail(c, ZKH_ERR_LIMIT, "batchopen: too many rounds");
    if (T < 1 || k < 1 || Q < 1 || Q > 4096) return zkh_fail(c, ZKH_ERR_ARG, "batchopen: empty ledger or bad Q");
    for (uint32_t j = 0; j < k; j++)
        if (zid[j] >= T || !cols_dev[j] || ((uintptr_t)cols_dev[j] & 15))
            return zkh_fail(c, ZKH_ERR_ARG, "batchopen: entry with bad point index, or a column that is null or not 16-byte aligned");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    const size_t N = (size_t)1 << v;
    const uint32_t logM0 = v + R;
    const size_t M0 = (size_t)1 << logM0;
    cudaStream_t s = c->stream;

    // distinct columns by root, first appearance (p3_batchopen.cuh:393-403)
    std::vector<uint32_t> colidx(k), first;
    for (uint32_t j = 0; j < k; j++) {
        uint32_t cc = 0;
        while (cc < first.size() && memcmp(roots + (size_t)first[cc] * 32, roots + (size_t)j * 32, 32)) cc++;
        if (cc == first.size()) first.push_back(j);
        colidx[j] = cc;
    }
    const uint32_t nc = (uint32_t)first.size();
    if (cap < bo_bound(v, R, Q, nc) + (sseeds ? (size_t)nc * 2 * Q * 32 : 0)) return zkh_fail(c, ZKH_ERR_ARG, "batchopen: output buffer smaller than zkh_batchopen_proof_bound");
    if ((size_t)T * N > ((size_t)1 << 36)) return zkh_fail(c, ZKH_ERR_LIMIT, "batchopen: T*2^v beyond 2^36");

    // ---- main transcript: mu and its powers (host; nothing on the device precedes it) ----
    gl_t mu = zkh_tr_chal(state);
    std::vector<uint32_t> estart(T + 1, 0);
    for (uint32_t j = 0; j < k; j++) estart[zid[j] + 1]++;
    for (uint32_t t = 0; t < T; t++) estart[t + 1] += estart[t];
    std::vector<const gl_t*> ecol(k + nc);
    std::vector<gl_t> ew(k + nc);
    {
        std::vector<uint32_t> fill(estart.begin(), estart.end() - 1);
        gl_t w = 1;
        for (uint32_t j = 0; j < k; j++) {   // ascending j inside each point
            uint32_t e = fill[zid[j]]++;
            ecol[e] = cols_dev[j];
            ew[e] = w;
            w = gl_mul(w, mu);
        }
    }

    // ---- workspace ----
    const uint32_t nb = (uint32_t)std::min<size_t>(64, std::max<size_t>(1, N / 1024));
    const uint32_t vl = v <= 1 ? v : (v / 2 > 14 ? 14 : v / 2), vh = v - vl;
    const size_t per_query = (size_t)(v - 1) * 16 + 64 * ((size_t)(v - 1) * logM0 - (size_t)(v - 1) * v / 2);
    const size_t q0_per_col = (size_t)2 * Q * 8 + (size_t)2 * Q * logM0 * 32;
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off += zkh_align(bytes); return o; };
    const size_t o_pa = take(((size_t)T * N / 2 + 2) * 8), o_pb = take(((size_t)T * N / 4 + 2) * 8);
    const size_t o_ecol = take((size_t)(k + nc) * 8), o_ew = take((size_t)(k + nc) * 8), o_es = take((size_t)(T + 3) * 4);
    const size_t o_zs = take((size_t)T * v * 8), o_tlo = take(((size_t)T << vl) * 8), o_thi = take(((size_t)T << vh) * 8);
    const size_t o_tlo2 = take(((size_t)T << vl) * 8), o_thi2 = take(((size_t)T << vh) * 8);
    const size_t o_eqr = take(N * 8), o_U = take(N * 8), o_ys = take((size_t)nc * 8), o_dp = take((size_t)nc * nb * 8);
    BoTrees bt;
    memset(&bt, 0, sizeof bt);
    size_t tree_bytes = 0;
    for (uint32_t r = 1; r < v; r++) {
        bt.off[r] = tree_bytes;
        bt.cut[r] = merkle_cut(M0 >> r);
        tree_bytes += merkle_capped_bytes(M0 >> r);
    }
    const size_t o_cw0 = take(M0 * 8), o_cwr = take(M0 * 8), o_trees = take(tree_bytes + 32);
    const size_t o_oa = take((N + 2) * 8), o_ob = take((N / 2 + 2) * 8);
    const size_t o_roots = take((size_t)v * 32), o_pos = take((size_t)Q * v * 4 + (size_t)2 * Q * 4);
    const size_t o_q = take((size_t)Q * per_query + 16);
    const uint32_t cut0 = merkle_cut(M0);
    const size_t o_cwc = take(M0 * 8), o_treec = take(merkle_capped_bytes(M0)), o_mks = take(merkle_scratch_bytes(M0)), o_q0 = take((size_t)nc * q0_per_col);
    const size_t o_misc = take(std::max(eq_scratch_bytes(v), ntt_scratch_bytes(logM0)));
    ZKH_TRY(zkh_ws_reserve(c, off));
    char* ws = (char*)c->ws;
    gl_t *pa = (gl_t*)(ws + o_pa), *pb = (gl_t*)(ws + o_pb);
    const gl_t** d_ecol = (const gl_t**)(ws + o_ecol);
    gl_t* d_ew = (gl_t*)(ws + o_ew);
    uint32_t* d_es = (uint32_t*)(ws + o_es);
    gl_t *d_zs = (gl_t*)(ws + o_zs), *tlo_e = (gl_t*)(ws + o_tlo), *thi_e = (gl_t*)(ws + o_thi);
    gl_t *tlo_2 = (gl_t*)(ws + o_tlo2), *thi_2 = (gl_t*)(ws + o_thi2);
    gl_t *eqr = (gl_t*)(ws + o_eqr), *U = (gl_t*)(ws + o_U), *d_ys = (gl_t*)(ws + o_ys), *d_dp = (gl_t*)(ws + o_dp);
    gl_t *cw0 = (gl_t*)(ws + o_cw0), *cwr = (gl_t*)(ws + o_cwr);
    uint8_t* trees = (uint8_t*)(ws + o_trees);
    gl_t *oa = (gl_t*)(ws + o_oa), *ob = (gl_t*)(ws + o_ob);
    uint8_t* d_roots = (uint8_t*)(ws + o_roots);
    uint32_t* d_pos = (uint32_t*)(ws + o_pos);
    uint8_t* d_q = (uint8_t*)(ws + o_q);
    gl_t* cwc = (gl_t*)(ws + o_cwc);
    uint8_t* treec = (uint8_t*)(ws + o_treec);
    uint8_t* d_q0 = (uint8_t*)(ws + o_q0);

    // the distinct columns ride behind the entries in the same pointer / weight arrays
    for (uint32_t cc = 0; cc < nc; cc++) ecol[k + cc] = cols_dev[first[cc]];
    ZKH_CUDA(c, cudaMemcpyAsync(d_ecol, ecol.data(), (size_t)(k + nc) * 8, cudaMemcpyHostToDevice, s));
    ZKH_CUDA(c, cudaMemcpyAsync(d_ew, ew.data(), (size_t)k * 8, cudaMemcpyHostToDevice, s));
    ZKH_CUDA(c, cudaMemcpyAsync(d_es, estart.data(), (size_t)(T + 1) * 4, cudaMemcpyHostToDevice, s));
    ZKH_CUDA(c, cudaMemcpyAsync(d_zs, pts, (size_t)T * v * 8, cudaMemcpyHostToDevice, s));
    ZkhCtl* h = c->h_ctl;
    digest_from_bytes(state, h->st);
    h->counter = 0;
    h->err = 0;
    for (int i = 0; i < 8; i++) h->par[i] = 0;
    ZKH_CUDA(c, cudaMemcpyAsync(c->d_ctl, h, offsetof(ZkhCtl, local), cudaMemcpyHostToDevice, s));

    auto grid_of = [&](size_t items) {
        size_t b = (items + 255) / 256, capb = (size_t)c->sm_count * 8;
        return (unsigned)(b < capb ? (b ? b : 1) : capb);
    };
    bo_eq_small_kernel<<<((T << vl) + 255) / 256, 256, 0, s>>>(d_zs, T, v, 0, vl, tlo_e);
    bo_eq_small_kernel<<<((T << vh) + 255) / 256, 256, 0, s>>>(d_zs, T, v, vl, vh, thi_e);
    ZKH_CUDA(c, cudaGetLastError());

    // ---- reduction sumcheck on the stacked arrays ----
    const ZkhTag tag_rm = zkh_make_tag("bo-rm");
    gl_t* msgs = c->d_ctl->msgs;
    gl_t* chals = c->d_ctl->chals;
    {
        BoRed P;
        memset(&P, 0, sizeof P);
        P.ecol = d_ecol; P.ew = d_ew; P.estart = d_es; P.T = T;
        const gl_t *lo_cur = tlo_e, *hi_cur = thi_e;
        gl_t *lo_nxt = tlo_2, *hi_nxt = thi_2;
        uint32_t lw = vl, hw = vh;
        const gl_t* g_cur = nullptr;
        gl_t* dst = pa;
        auto red_grid = [&](size_t items) {
            size_t b = (items + 255) / 256, capb = (size_t)c->sm_count * 4;
            if (capb > c->partials_cap / 5) capb = c->partials_cap / 5;
            return (unsigned)(b < capb ? (b ? b : 1) : capb);
        };
        for (uint32_t rd = 0; rd < v; rd++) {
            if (rd > 0) {   // the eq factor tables take the previous challenge: low variables first, then the high ones
                if (lw > 0) {
                    const uint32_t cnt = T << (lw - 1);
                    bo_tab_bind_kernel<<<(cnt + 255) / 256, 256, 0, s>>>(lo_cur, lo_nxt, cnt, chals + (rd - 1));
                    const gl_t* tswap = lo_cur; lo_cur = lo_nxt; lo_nxt = (gl_t*)tswap;
                    lw--;
                } else {
                    const uint32_t cnt = T << (hw - 1);
                    bo_tab_bind_kernel<<<(cnt + 255) / 256, 256, 0, s>>>(hi_cur, hi_nxt, cnt, chals + (rd - 1));
                    const gl_t* tswap = hi_cur; hi_cur = hi_nxt; hi_nxt = (gl_t*)tswap;
                    hw--;
                }
            }
            P.lo = lo_cur; P.hi = hi_cur; P.lw = lw; P.hw = hw;
            P.logL = v - rd;
            const size_t items = (size_t)T << (v - rd - 1);
            if (rd == 0) {
                bo_reduce_kernel<true, true><<<red_grid(items), 256, 0, s>>>(P, c->d_ctl, c->d_partials, nullptr, msgs, chals, tag_rm);
            } else {
                P.G = g_cur; P.Gout = dst;
                if (rd == 1)
                    bo_reduce_kernel<true, false><<<red_grid(items), 256, 0, s>>>(P, c->d_ctl, c->d_partials, chals, msgs + 3, chals + 1, tag_rm);
                else
                    bo_reduce_kernel<false, false><<<red_grid(items), 256, 0, s>>>(P, c->d_ctl, c->d_partials, chals + (rd - 1),
                                                                                  msgs + (size_t)rd * 3, chals + rd, tag_rm);
                g_cur = dst;
                dst = (dst == pa) ? pb : pa;
            }
        }
        ZKH_CUDA(c, cudaGetLastError());
    }
    // ---- y*_c = col_c(r*) ----
    ZKH_TRY(eq_enqueue(c, chals, v, eqr, ws + o_misc, /*z_on_device=*/true));
    bo_dots_kernel<<<dim3(nb, nc), 256, 0, s>>>(d_ecol + k, eqr, N, d_dp, nb);
    bo_dots_sum_kernel<<<nc, 64, 0, s>>>(d_dp, nb, d_ys);
    ZKH_CUDA(c, cudaGetLastError());
    uint8_t* p = out;
    memcpy(p, &v, 4); memcpy(p + 4, &R, 4); memcpy(p + 8, &Q, 4); memcpy(p + 12, &nc, 4);
    p += 16;
    uint8_t* p_ystar = p;  p += (size_t)nc * 8;
    uint8_t* p_rmsgs = p;  p += (size_t)v * 24;
    uint8_t* p_roots = p;  p += (size_t)(v - 1) * 32;
    uint8_t* p_omsgs = p;  p += (size_t)v * 24;
    uint8_t* p_final = p;  p += (size_t)8 << R;
    uint8_t* p_q = p;
    ZKH_CUDA(c, cudaMemcpyAsync(h, c->d_ctl, sizeof(ZkhCtl), cudaMemcpyDeviceToHost, s));
    ZKH_CUDA(c, cudaMemcpyAsync(p_ystar, d_ys, (size_t)nc * 8, cudaMemcpyDeviceToHost, s));
    ZKH_CUDA(c, cudaStreamSynchronize(s));   // sync 1
    if (h->err) return zkh_fail(c, ZKH_ERR_DEVICE, "batchopen: device error flag set");
    memcpy(p_rmsgs, h->msgs, (size_t)v * 24);
    std::vector<gl_t> rstar(h->chals, h->chals + v), ystar(nc);
    memcpy(ystar.data(), p_ystar, (size_t)nc * 8);
    digest_to_bytes(h->st, state);
    zkh_tr_absorb(state, "bo-ys", ystar.data(), (uint64_t)nc * 8);
    const gl_t rho = zkh_tr_chal(state);   // the main transcript is final here

    // ---- U = sum_c rho^c col_c, yU ----
    gl_t yU = 0;
    {
        gl_t w = 1;
        for (uint32_t cc = 0; cc < nc; cc++) { ew[k + cc] = w; yU = gl_add(yU, gl_mul(w, ystar[cc])); w = gl_mul(w, rho); }
        uint32_t es1[2] = {k, k + nc};
        ZKH_CUDA(c, cudaMemcpyAsync(d_ew + k, ew.data() + k, (size_t)nc * 8, cudaMemcpyHostToDevice, s));
        ZKH_CUDA(c, cudaMemcpyAsync(d_es + T + 1, es1, 8, cudaMemcpyHostToDevice, s));
        bo_gbuild_kernel<<<grid_of(N), 256, 0, s>>>(d_ecol, d_ew, d_es + T + 1, U, 1, N);
        ZKH_CUDA(c, cudaGetLastError());
    }
    // ---- opening transcript: seed = class label ----
    uint8_t ot[32];
    zkh_tr_init(ot, label, strlen(label));
    zkh_tr_absorb(ot, "z", rstar.data(), (uint64_t)v * 8);
    zkh_tr_absorb(ot, "y", &yU, 8);
    digest_from_bytes(ot, h->st);
    h->counter = 0;
    ZKH_CUDA(c, cudaMemcpyAsync(c->d_ctl, h, offsetof(ZkhCtl, local), cudaMemcpyHostToDevice, s));
    ZKH_TRY(ntt_enqueue(c, U, N, cw0, logM0, false, ws + o_misc));
    const gl_t *tlo, *thi;
    uint32_t tlb;
    ZKH_TRY(ntt_inverse_tables(c, logM0, &tlo, &thi, &tlb));
    const ZkhTag tag_sc = zkh_make_tag("sc");
    {
        const gl_t* cur[2] = {U, eqr};
        gl_t* dst = oa;
        const gl_t* cw_cur = cw0;
        for (uint32_t r = 0; r < v; r++) {
            const size_t Mr = M0 >> r, n = N >> r;
            if (r > 0) {
                ZKH_TRY(merkle_enqueue(c, cw_cur, Mr, trees + bt.off[r], ws + o_mks, d_roots + (size_t)(r - 1) * 32, nullptr, bt.cut[r]));
                ZKH_TRY(tr_absorb_enqueue(c, "root", (const uint64_t*)(d_roots + (size_t)(r - 1) * 32), 4));
            }
            if (r == 0) {
                ZKH_TRY(sc_enqueue_round(c, ZKH_F_PROD2, 3, true, cur, nullptr, n, nullptr, msgs, chals, tag_sc));
            } else {
                gl_t* outp[2] = {dst, dst + n};
                ZKH_TRY(sc_enqueue_round(c, ZKH_F_PROD2, 3, false, cur, outp, 2 * n, chals + (r - 1), msgs + (size_t)r * 3,
                                         chals + r, tag_sc));
                cur[0] = outp[0];
                cur[1] = outp[1];
                dst = (dst == oa) ? ob : oa;
            }
            gl_t* cw_next = cwr + (M0 - Mr);
            ZKH_TRY(fold_enqueue(c, cw_cur, cw_next, Mr, logM0, r, chals + r, 0, tlo, thi, tlb));
            cw_cur = cw_next;
        }
        ZKH_TRY(tr_absorb_enqueue(c, "final", cw_cur, 1u << R));
        ZKH_CUDA(c, cudaMemcpyAsync(p_final, cw_cur, (size_t)8 << R, cudaMemcpyDeviceToHost, s));
    }
    ZKH_CUDA(c, cudaMemcpyAsync(h, c->d_ctl, sizeof(ZkhCtl), cudaMemcpyDeviceToHost, s));
    if (v > 1) ZKH_CUDA(c, cudaMemcpyAsync(p_roots, d_roots, (size_t)(v - 1) * 32, cudaMemcpyDeviceToHost, s));
    ZKH_CUDA(c, cudaStreamSynchronize(s));   // sync 2
    if (h->err) return zkh_fail(c, ZKH_ERR_DEVICE, "batchopen: device error flag set");
    memcpy(p_omsgs, h->msgs, (size_t)v * 24);
    digest_to_bytes(h->st, ot);

    // ---- queries ----
    std::vector<uint32_t> pos((size_t)Q * v), upos;
    for (uint32_t q = 0; q < Q; q++) {
        uint64_t cur = zkh_tr_idx(ot, M0 / 2);
        for (uint32_t r = 0; r < v; r++) {
            cur = cur % ((M0 >> r) / 2);
            pos[(size_t)q * v + r] = (uint32_t)cur;
        }
        upos.push_back(pos[(size_t)q * v]);
        upos.push_back(pos[(size_t)q * v] + (uint32_t)(M0 / 2));
    }
    std::sort(upos.begin(), upos.end());
    upos.erase(std::unique(upos.begin(), upos.end()), upos.end());
    const uint32_t nu = (uint32_t)upos.size();
    uint32_t* d_upos = d_pos + (size_t)Q * v;
    ZKH_CUDA(c, cudaMemcpyAsync(d_pos, pos.data(), (size_t)Q * v * 4, cudaMemcpyHostToDevice, s));
    ZKH_CUDA(c, cudaMemcpyAsync(d_upos, upos.data(), (size_t)nu * 4, cudaMemcpyHostToDevice, s));
    if (v > 1) {
        const uint32_t nth = Q * (v - 1) * 2;
        bo_query_kernel<<<(nth + 127) / 128, 128, 0, s>>>(cwr, trees, bt, logM0, v, Q, d_pos, d_q, per_query);
        ZKH_CUDA(c, cudaGetLastError());
        for (uint32_t r = 1; r < v; r++) {                     // the lowest levels of both openings of every query, rebuilt from the codeword
            const size_t Mr = M0 >> r, rr = r - 1;
            const size_t roff = rr * 16 + 64 * (rr * logM0 - rr * (rr + 1) / 2);
            for (uint32_t side = 0; side < 2 && bt.cut[r]; side++)
                ZKH_TRY(merkle_low_paths_enqueue(c, cwr + (M0 - 2 * Mr), bt.cut[r], d_pos + r, Q, nullptr,
                                                 d_q + roff + 16 + (size_t)side * (logM0 - r) * 32, per_query, v,
                                                 side ? (uint32_t)(Mr / 2) : 0));
        }
        ZKH_CUDA(c, cudaMemcpyAsync(p_q, d_q, (size_t)Q * per_query, cudaMemcpyDeviceToHost, s));
    }
    // round-0 openings: re-encode each distinct column, hash its tree, gather values and paths
    const size_t q0_used = (size_t)nu * 8 + (size_t)nu * logM0 * 32;
    for (uint32_t cc = 0; cc < nc; cc++) {
        const gl_t* cw_use = cwc;
        const uint8_t* tree_use = treec;
        if (kept_cw && kept_tree && kept_cw[first[cc]] && kept_tree[first[cc]]) {
            cw_use = kept_cw[first[cc]];          // committed with zkh_basefold_commit_keep (capped tree): nothing to recompute
            tree_use = kept_tree[first[cc]];
        } else {
            ZKH_TRY(ntt_enqueue(c, cols_dev[first[cc]], N, cwc, logM0, false, ws + o_misc));
            ZKH_TRY(merkle_enqueue(c, cwc, M0, treec, ws + o_mks, nullptr, sseeds ? sseeds + first[cc] : nullptr, cut0));
        }
        const uint32_t nth = nu * (logM0 + 1);
        uint8_t* q0c = d_q0 + (size_t)cc * q0_per_col;
        bo_q0_kernel<<<(nth + 127) / 128, 128, 0, s>>>(cw_use, tree_use, logM0, cut0, d_upos, nu, q0c);
        ZKH_TRY(merkle_low_paths_enqueue(c, cw_use, cut0, d_upos, nu, sseeds ? sseeds + first[cc] : nullptr, q0c + (size_t)nu * 8,
                                         (size_t)logM0 * 32));
    }
    ZKH_CUDA(c, cudaGetLastError());
    std::vector<uint8_t> hq0((size_t)nc * q0_per_col);
    ZKH_CUDA(c, cudaMemcpyAsync(hq0.data(), d_q0, hq0.size(), cudaMemcpyDeviceToHost, s));
    ZKH_CUDA(c, cudaStreamSynchronize(s));   // sync 3
    (void)q0_used;
    p = p_q + (size_t)Q * per_query;
    // pruned node stream per column (p3_batchopen.cuh:75-106): where both children of a parent are
    // in the frontier nothing is emitted, otherwise the sibling comes from the path of the first
    // covered leaf below the node
    std::vector<uint32_t> fr_idx(nu), fr_slot(nu);
    for (uint32_t cc = 0; cc < nc; cc++) {
        const uint8_t* colq = hq0.data() + (size_t)cc * q0_per_col;
        const uint8_t* paths = colq + (size_t)nu * 8;
        memcpy(p, &nu, 4); p += 4;
        memcpy(p, colq, (size_t)nu * 8); p += (size_t)nu * 8;
        if (sseeds)   // the salts of the opened leaves (p3_batchopen.cuh:1047-1051, :1103-1104)
            for (uint32_t i = 0; i < nu; i++) {
                uint32_t hs[8];
                sha256_salt(sseeds[first[cc]], upos[i], hs);
                digest_to_bytes(hs, p);
                p += 32;
            }
        uint8_t* p_cnt = p; p += 4;
        uint32_t nn = 0, nf = nu;
        for (uint32_t i = 0; i < nu; i++) { fr_idx[i] = upos[i]; fr_slot[i] = i; }
        for (uint32_t l = 0; l < logM0; l++) {
            uint32_t w = 0, i = 0;
            while (i < nf) {
                uint32_t idx = fr_idx[i], slot = fr_slot[i];
                if (!(idx & 1) && i + 1 < nf && fr_idx[i + 1] == (idx | 1)) {
                    i += 2;
                } else {
                    memcpy(p, paths + ((size_t)slot * logM0 + l) * 32, 32);
                    p += 32; nn++; i += 1;
                }
                fr_idx[w] = idx >> 1; fr_slot[w] = slot; w++;
            }
            nf = w;
        }
        memcpy(p_cnt, &nn, 4);
    }
    *written = (size_t)(p - out);
    return ZKH_OK;
}

extern "C" int zkh_batchopen_prove_class(zkh_ctx* c, uint32_t v, const uint64_t* pts, uint32_t T,
                                         const uint64_t* const* cols_dev, const uint8_t* roots, const uint32_t* zid,
                                         uint32_t k, uint32_t R, uint32_t Q, const char* label, uint8_t state[32],
                                         uint8_t* out, size_t cap, size_t* written) {
    return batchopen_prove_class(c, v, pts, T, cols_dev, roots, zid, k, R, Q, label, state, out, cap, written, nullptr, nullptr);
}
// Hiding mode: every column was committed with zkh_basefold_commit_salted under sseeds[j]; the round-0 openings rebuild (or
// reuse) the salted trees and carry the 32-byte salt of every opened leaf after the values.  The class blinder column
// (p3_batchopen.cuh:315-384) is an ordinary entry the caller appends before the call.
extern "C" int zkh_batchopen_prove_class_salted(zkh_ctx* c, uint32_t v, const uint64_t* pts, uint32_t T,
                                                const uint64_t* const* cols_dev, const uint8_t* roots, const uint32_t* zid,
                                                const uint64_t* sseeds, uint32_t k, uint32_t R, uint32_t Q, const char* label,
                                                uint8_t state[32], uint8_t* out, size_t cap, size_t* written,
                                                const uint64_t* const* kept_cw, const uint8_t* const* kept_tree) {
    if (!sseeds) return zkh_fail(c, ZKH_ERR_ARG, "batchopen: salted openings need the salt seeds");
    return batchopen_prove_class(c, v, pts, T, cols_dev, roots, zid, k, R, Q, label, state, out, cap, written, kept_cw, kept_tree,
                                 sseeds);
}
// Same, with kept_cw[j] / kept_tree[j] (either may be NULL per entry) the codeword and Merkle tree that
// zkh_basefold_commit_keep left for entry j's column under the same R.
extern "C" int zkh_batchopen_prove_class_kept(zkh_ctx* c, uint32_t v, const uint64_t* pts, uint32_t T,
                                              const uint64_t* const* cols_dev, const uint8_t* roots, const uint32_t* zid,
                                              uint32_t k, uint32_t R, uint32_t Q, const char* label, uint8_t state[32],
                                              uint8_t* out, size_t cap, size_t* written, const uint64_t* const* kept_cw,
                                              const uint8_t* const* kept_tree) {
    return batchopen_prove_class(c, v, pts, T, cols_dev, roots, zid, k, R, Q, label, state, out, cap, written, kept_cw, kept_tree);
}
