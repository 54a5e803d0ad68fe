// Basefold commitment and evaluation opening over Goldilocks for sm_100a.
//
// commit  = Reed-Solomon encode (NTT) + SHA-256 Merkle root
//           (zkllm-src/p3_basefold.cuh:188-227: rs_encode_gpu_dev, commit_gpu_rootonly)
// open    = v rounds of { Merkle(codeword_r) -> absorb root; degree-2 sumcheck message of
//           sum_b c[b]*eq(b,z) -> absorb; alpha; bind c and eq; fold the codeword with alpha },
//           then the final word and Q query openings
//           (zkllm-src/p3_basefold.cuh:355-420, prove_eval_dev).
//
// The reference synchronises with the host several times per round (root copy, three
// partial-sum copies, per-round allocations).  Here the whole round chain is queued on the
// stream with the transcript on the device; the host synchronises twice per opening: once
// to learn the transcript state after "final" (the query positions derive from it), once to
// fetch the gathered query openings.
#include "merkle.cuh"
#include "ntt.cuh"
#include "sumcheck.cuh"

namespace zkh {

// out[c] = (1-beta)*E + beta*O with E=(a+b)/2, O=(a-b)/(2x), x=w^c, a=f[c], b=f[c+half]
//        = k1*(a+b) + k2*w^{-c}*(a-b),  k1=(1-beta)/2, k2=beta/2
// (zkllm-src/p3_basefold.cuh:239-245 computes w^{-c} with a per-thread gl_pow; here it is one
// lookup in the split inverse twiddle table of the top-level domain: w_r^{-c} = W0^{-(c<<r)}).
__global__ void __launch_bounds__(256)
fold_kernel(const gl_t* __restrict__ f, gl_t* __restrict__ out, size_t half, const gl_t* beta_ptr, gl_t beta_val,
            const gl_t* __restrict__ tlo, const gl_t* __restrict__ thi, uint32_t tlb, uint32_t shift) {
    const gl_t beta = beta_ptr ? *beta_ptr : beta_val;
    const gl_t inv2 = 0x7FFFFFFF80000001ULL;  // (p+1)/2
    const gl_t k1 = gl_mul(gl_sub(1, beta), inv2), k2 = gl_mul(beta, inv2);
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < half; i += stride) {
        gl_t a = f[i], b = f[i + half];
        uint64_t e = (uint64_t)i << shift;
        gl_t w = tlo[e & ((1ull << tlb) - 1)];
        uint64_t eh = e >> tlb;
        if (eh) w = gl_mul(w, thi[eh]);
        Acc192 acc;
        acc.clear();
        acc.add_prod(k1, gl_add(a, b));
        acc.add_prod(gl_mul(k2, w), gl_sub(a, b));
        out[i] = acc.reduce();
    }
}

// gathers every query opening straight into the proof's query section:
// per query q, per round r:  a(8) b(8) pa(plen*32) pb(plen*32), plen = logM0 - r
__global__ void bf_query_kernel(const gl_t* cw0, const gl_t* cw_rest, const uint8_t* trees, uint32_t logM0,
                                uint32_t v, uint32_t Q, const uint32_t* pos /* [Q][v] */, uint8_t* out,
                                size_t per_query) {
    uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= Q * v * 2) return;
    const uint32_t side = t & 1, e = t >> 1, q = e / v, r = e % v;
    const size_t M0 = (size_t)1 << logM0, Mr = M0 >> r, h = Mr / 2;
    const uint32_t plen = logM0 - r;
    // codeword r: round 0 is the caller's, rounds >= 1 are packed after one another
    const gl_t* cw = r == 0 ? cw0 : cw_rest + (M0 - 2 * Mr);  // sum_{i=1}^{r-1} M0>>i = M0 - 2*Mr
    // tree r starts after the trees of rounds < r: sum (2*M_i - 1) = 4*M0 - 4*Mr - r digests
    const uint8_t* tree = trees + (4 * M0 - 4 * Mr - r) * 32;
    const size_t idx = (size_t)pos[q * v + r] + (side ? h : 0);
    // byte offset of round r inside one query: sum_{i<r} (16 + 64*(logM0-i))
    size_t off = (size_t)q * per_query + (size_t)r * 16 + 64 * ((size_t)r * logM0 - (size_t)r * (r - 1) / 2);
    uint8_t* o = out + off;
    *reinterpret_cast<gl_t*>(o + 8 * side) = cw[idx];
    uint4* po = reinterpret_cast<uint4*>(o + 16 + (size_t)side * plen * 32);
    size_t id = idx;
    for (uint32_t l = 0; l < plen; l++) {
        size_t cnt = Mr >> l;
        const uint4* src = reinterpret_cast<const uint4*>(tree + (2 * Mr - 2 * cnt + (id ^ 1)) * 32);
        po[2 * l] = src[0];
        po[2 * l + 1] = src[1];
        id >>= 1;
    }
}

static size_t bf_proof_size(uint32_t v, uint32_t R, uint32_t Q) {
    size_t s = 12 + (size_t)v * 32 + (size_t)v * 24 + ((size_t)8 << R);
    for (uint32_t r = 0; r < v; r++) s += (size_t)Q * (16 + 2 * (size_t)(v + R - r) * 32);
    return s + (size_t)v * 8 + 8;
}

int fold_enqueue(zkh_ctx* c, const gl_t* f, gl_t* out, size_t M, uint32_t logM_top, uint32_t shift,
                 const gl_t* beta_ptr, gl_t beta_val, const gl_t* tlo, const gl_t* thi, uint32_t tlb) {
    (void)logM_top;
    size_t half = M / 2, blocks = (half + 255) / 256, cap = (size_t)c->sm_count * 8;
    fold_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, c->stream>>>(f, out, half, beta_ptr, beta_val, tlo,
                                                                              thi, tlb, shift);
    ZKH_CUDA(c, cudaGetLastError());
    return ZKH_OK;
}

// inverse split twiddle table of the 2^logM domain (cached in the context by the NTT module)
int ntt_inverse_tables(zkh_ctx* c, uint32_t logM, const gl_t** lo, const gl_t** hi, uint32_t* lb);

}  // namespace zkh

using namespace zkh;

extern "C" size_t zkh_basefold_proof_size(uint32_t v, uint32_t R, uint32_t Q) { return bf_proof_size(v, R, Q); }

extern "C" int zkh_gl_fold_codeword(zkh_ctx* c, const uint64_t* f_dev, uint64_t* out_dev, uint64_t M, uint64_t beta) {
    if (!c || !f_dev || !out_dev) return zkh_fail(c, ZKH_ERR_ARG, "fold_codeword: null pointer");
    if (M < 2 || (M & (M - 1)) || M > ((uint64_t)1 << 32)) return zkh_fail(c, ZKH_ERR_ARG, "fold_codeword: bad length");
    if (beta >= GL_P) return zkh_fail(c, ZKH_ERR_ARG, "fold_codeword: challenge not canonical");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    uint32_t logM = 0;
    while (((uint64_t)1 << logM) < M) logM++;
    const gl_t *tlo, *thi;
    uint32_t tlb;
    ZKH_TRY(ntt_inverse_tables(c, logM, &tlo, &thi, &tlb));
    return fold_enqueue(c, f_dev, out_dev, (size_t)M, logM, 0, nullptr, beta, tlo, thi, tlb);
}

extern "C" int zkh_basefold_commit(zkh_ctx* c, const uint64_t* c_dev, uint32_t v, uint32_t R, uint64_t* cw_dev,
                                   uint8_t root[32]) {
    if (!c || !c_dev || !root) return zkh_fail(c, ZKH_ERR_ARG, "basefold_commit: null pointer");
    if (v + R < 1 || v + R > 32 || R < 1 || R > 8) return zkh_fail(c, ZKH_ERR_ARG, "basefold_commit: need R in 1..8, v+R <= 32");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    const uint32_t logM = v + R;
    const size_t M = (size_t)1 << logM;
    const size_t cwb = cw_dev ? 0 : zkh_align(M * 8), nttb = ntt_scratch_bytes(logM), mkb = merkle_scratch_bytes(M);
    ZKH_TRY(zkh_ws_reserve(c, cwb + nttb + mkb));
    gl_t* cw = cw_dev ? cw_dev : (gl_t*)c->ws;
    void* ntt_s = (char*)c->ws + cwb;
    void* mk_s = (char*)c->ws + cwb + nttb;
    ZKH_TRY(ntt_enqueue(c, c_dev, (uint64_t)1 << v, cw, logM, false, ntt_s));
    uint8_t* root_dev = (uint8_t*)c->d_ctl->aux;
    ZKH_TRY(merkle_enqueue(c, cw, M, nullptr, mk_s, root_dev));
    ZKH_CUDA(c, cudaMemcpyAsync(c->h_ctl->aux, root_dev, 32, cudaMemcpyDeviceToHost, c->stream));
    ZKH_CUDA(c, cudaStreamSynchronize(c->stream));
    memcpy(root, c->h_ctl->aux, 32);
    return ZKH_OK;
}

// Commit and KEEP: the codeword and the capped Merkle tree (levels from 64 leaves per node upwards; the lowest six
// levels of an opened path are rebuilt from 64 codeword elements) stay in caller-owned device buffers, so that later
// openings of this column read authentication paths instead of encoding and hashing the column again.
extern "C" size_t zkh_basefold_kept_tree_bytes(uint32_t logM) {
    return logM >= 1 && logM <= 32 ? merkle_capped_bytes((size_t)1 << logM) : 0;
}
extern "C" int zkh_basefold_commit_keep(zkh_ctx* c, const uint64_t* c_dev, uint32_t v, uint32_t R, uint64_t* cw_dev,
                                        uint8_t* tree_dev, uint8_t root[32]) {
    if (!c || !c_dev || !root || !cw_dev || !tree_dev) return zkh_fail(c, ZKH_ERR_ARG, "basefold_commit_keep: null pointer");
    if (v + R < 1 || v + R > 32 || R < 1 || R > 8) return zkh_fail(c, ZKH_ERR_ARG, "basefold_commit_keep: need R in 1..8, v+R <= 32");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    const uint32_t logM = v + R;
    const size_t M = (size_t)1 << logM;
    const size_t nttb = ntt_scratch_bytes(logM);
    ZKH_TRY(zkh_ws_reserve(c, nttb + merkle_scratch_bytes(M)));
    ZKH_TRY(ntt_enqueue(c, c_dev, (uint64_t)1 << v, cw_dev, logM, false, c->ws));
    uint8_t* root_dev = (uint8_t*)c->d_ctl->aux;
    ZKH_TRY(merkle_enqueue(c, cw_dev, M, tree_dev, (char*)c->ws + nttb, root_dev, nullptr, merkle_cut(M)));
    ZKH_CUDA(c, cudaMemcpyAsync(c->h_ctl->aux, root_dev, 32, cudaMemcpyDeviceToHost, c->stream));
    ZKH_CUDA(c, cudaStreamSynchronize(c->stream));
    memcpy(root, c->h_ctl->aux, 32);
    return ZKH_OK;
}

// Commitment roots of k independent columns with ONE host synchronisation: a layer proof commits hundreds of small witness
// columns (the reference commits them one after another, each with its own device round trip, zkllm-src/p3_logup.cuh
// commit_col_nc -> p3_basefold.cuh:210-227); here every encode + tree build is queued on the stream and the k roots come
// back in one copy.
extern "C" int zkh_basefold_commit_many(zkh_ctx* c, const uint64_t* const* cols_dev, const uint32_t* vs, uint32_t k, uint32_t R,
                                        uint8_t* roots) {
    if (!c || !cols_dev || !vs || !roots) return zkh_fail(c, ZKH_ERR_ARG, "basefold_commit_many: null pointer");
    if (R < 1 || R > 8) return zkh_fail(c, ZKH_ERR_ARG, "basefold_commit_many: need R in 1..8");
    if (!k) return ZKH_OK;
    ZKH_CUDA(c, cudaSetDevice(c->device));
    size_t need = 0;
    for (uint32_t j = 0; j < k; j++) {
        if (!cols_dev[j] || vs[j] + R < 1 || vs[j] + R > 32) return zkh_fail(c, ZKH_ERR_ARG, "basefold_commit_many: bad column");
        const uint32_t logM = vs[j] + R;
        const size_t M = (size_t)1 << logM, b = zkh_align(M * 8) + ntt_scratch_bytes(logM) + merkle_scratch_bytes(M);
        if (b > need) need = b;
    }
    const size_t rootb = zkh_align((size_t)k * 32);
    ZKH_TRY(zkh_ws_reserve(c, need + rootb));            // one reservation: the workspace must not move while work is queued
    uint8_t* roots_dev = (uint8_t*)c->ws + need;
    for (uint32_t j = 0; j < k; j++) {
        const uint32_t logM = vs[j] + R;
        const size_t M = (size_t)1 << logM, cwb = zkh_align(M * 8), nttb = ntt_scratch_bytes(logM);
        gl_t* cw = (gl_t*)c->ws;
        ZKH_TRY(ntt_enqueue(c, cols_dev[j], (uint64_t)1 << vs[j], cw, logM, false, (char*)c->ws + cwb));
        ZKH_TRY(merkle_enqueue(c, cw, M, nullptr, (char*)c->ws + cwb + nttb, roots_dev + (size_t)j * 32));
    }
    ZKH_CUDA(c, cudaMemcpyAsync(roots, roots_dev, (size_t)k * 32, cudaMemcpyDeviceToHost, c->stream));
    ZKH_CUDA(c, cudaStreamSynchronize(c->stream));
    return ZKH_OK;
}

// Hiding commitment (zkllm-src/p3_zkc.cuh:320-397 salted_commit_root / salted_commit_root_dev): the same codeword, leaves
// salted with SHA-256(seed | leaf index).  cw_dev / tree_dev optional (both or none keep codeword and capped tree resident).
extern "C" int zkh_basefold_commit_salted(zkh_ctx* c, const uint64_t* c_dev, uint32_t v, uint32_t R, uint64_t sseed,
                                          uint64_t* cw_dev, uint8_t* tree_dev, uint8_t root[32]) {
    if (!c || !c_dev || !root) return zkh_fail(c, ZKH_ERR_ARG, "basefold_commit_salted: null pointer");
    if (v + R < 1 || v + R > 32 || R < 1 || R > 8) return zkh_fail(c, ZKH_ERR_ARG, "basefold_commit_salted: need R in 1..8, v+R <= 32");
    if (tree_dev && !cw_dev) return zkh_fail(c, ZKH_ERR_ARG, "basefold_commit_salted: a kept tree needs the kept codeword");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    const uint32_t logM = v + R;
    const size_t M = (size_t)1 << logM;
    const size_t cwb = cw_dev ? 0 : zkh_align(M * 8), nttb = ntt_scratch_bytes(logM), mkb = merkle_scratch_bytes(M);
    ZKH_TRY(zkh_ws_reserve(c, cwb + nttb + mkb));
    gl_t* cw = cw_dev ? cw_dev : (gl_t*)c->ws;
    ZKH_TRY(ntt_enqueue(c, c_dev, (uint64_t)1 << v, cw, logM, false, (char*)c->ws + cwb));
    uint8_t* root_dev = (uint8_t*)c->d_ctl->aux;
    ZKH_TRY(merkle_enqueue(c, cw, M, tree_dev, (char*)c->ws + cwb + nttb, root_dev, &sseed, tree_dev ? merkle_cut(M) : 0));
    ZKH_CUDA(c, cudaMemcpyAsync(c->h_ctl->aux, root_dev, 32, cudaMemcpyDeviceToHost, c->stream));
    ZKH_CUDA(c, cudaStreamSynchronize(c->stream));
    memcpy(root, c->h_ctl->aux, 32);
    return ZKH_OK;
}

extern "C" int zkh_basefold_commit_host(zkh_ctx* c, const uint64_t* coeffs, uint32_t v, uint32_t R, uint8_t root[32]) {
    if (!c || !coeffs || !root) return zkh_fail(c, ZKH_ERR_ARG, "basefold_commit_host: null pointer");
    if (v + R < 1 || v + R > 32 || R < 1 || R > 8) return zkh_fail(c, ZKH_ERR_ARG, "basefold_commit_host: need R in 1..8, v+R <= 32");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    const uint32_t logM = v + R;
    const size_t M = (size_t)1 << logM, N = (size_t)1 << v;
    const size_t inb = zkh_align(N * 8), cwb = zkh_align(M * 8), nttb = ntt_scratch_bytes(logM), mkb = merkle_scratch_bytes(M);
    ZKH_TRY(zkh_ws_reserve(c, inb + cwb + nttb + mkb));
    gl_t* d_in = (gl_t*)c->ws;
    gl_t* cw = (gl_t*)((char*)c->ws + inb);
    ZKH_CUDA(c, cudaMemcpyAsync(d_in, coeffs, N * 8, cudaMemcpyHostToDevice, c->stream));
    ZKH_TRY(ntt_enqueue(c, d_in, N, cw, logM, false, (char*)c->ws + inb + cwb));
    uint8_t* root_dev = (uint8_t*)c->d_ctl->aux;
    ZKH_TRY(merkle_enqueue(c, cw, M, nullptr, (char*)c->ws + inb + cwb + nttb, root_dev));
    ZKH_CUDA(c, cudaMemcpyAsync(c->h_ctl->aux, root_dev, 32, cudaMemcpyDeviceToHost, c->stream));
    ZKH_CUDA(c, cudaStreamSynchronize(c->stream));
    memcpy(root, c->h_ctl->aux, 32);
    return ZKH_OK;
}

extern "C" int zkh_basefold_open(zkh_ctx* c, const uint64_t* c_dev, const uint64_t* z, uint32_t v, uint64_t y,
                                 uint32_t R, uint32_t Q, const uint64_t* cw0_dev, const char* seed, uint8_t* out,
                                 size_t cap, size_t* written) {
    if (!c || !c_dev || !z || !seed || !out || !written) return zkh_fail(c, ZKH_ERR_ARG, "basefold_open: null pointer");
    if (v < 1 || R < 1 || R > 3 || v + R > 32) return zkh_fail(c, ZKH_ERR_ARG, "basefold_open: need v >= 1, R in 1..3, v+R <= 32");
    if (v > 64) return zkh_fail(c, ZKH_ERR_LIMIT, "basefold_open: too many rounds");
    if (Q < 1 || Q > 4096) return zkh_fail(c, ZKH_ERR_ARG, "basefold_open: Q must be 1..4096");
    const size_t need = bf_proof_size(v, R, Q);
    if (cap < need) return zkh_fail(c, ZKH_ERR_ARG, "basefold_open: output buffer smaller than zkh_basefold_proof_size");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    const uint32_t logM0 = v + R;
    const size_t M0 = (size_t)1 << logM0, N = (size_t)1 << v;

    // ---- workspace carve-up ----
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off += zkh_align(bytes); return o; };
    const size_t o_cw0 = cw0_dev ? 0 : take(M0 * 8);
    const size_t o_cwr = take(M0 * 8);                       // codewords of rounds 1..v (M0/2 + ... + 2^R < M0)
    const size_t o_trees = take((4 * M0) * 32);              // sum_r (2*M_r - 1) digests < 4*M0
    const size_t o_eq = take(N * 8);
    const size_t o_ba = take(2 * (N / 2 + 1) * 8), o_bb = take(2 * (N / 4 + 1) * 8);
    const size_t o_roots = take((size_t)v * 32);
    const size_t o_pos = take((size_t)Q * v * 4);
    const size_t per_query = (size_t)v * 16 + 64 * ((size_t)v * logM0 - (size_t)v * (v - 1) / 2);
    const size_t o_q = take((size_t)Q * per_query);
    const size_t o_misc = take(eq_scratch_bytes(v) > ntt_scratch_bytes(logM0) ? eq_scratch_bytes(v) : ntt_scratch_bytes(logM0));
    ZKH_TRY(zkh_ws_reserve(c, off));
    char* ws = (char*)c->ws;
    gl_t* cw0 = cw0_dev ? (gl_t*)cw0_dev : (gl_t*)(ws + o_cw0);
    gl_t* cwr = (gl_t*)(ws + o_cwr);
    uint8_t* trees = (uint8_t*)(ws + o_trees);
    gl_t* eqw = (gl_t*)(ws + o_eq);
    gl_t* bufA = (gl_t*)(ws + o_ba);
    gl_t* bufB = (gl_t*)(ws + o_bb);
    uint8_t* roots = (uint8_t*)(ws + o_roots);

    // ---- host transcript head: seed, "z", "y" ----
    uint8_t st[32];
    zkh_tr_init(st, seed, strlen(seed));
    zkh_tr_absorb(st, "z", z, (uint64_t)v * 8);
    zkh_tr_absorb(st, "y", &y, 8);
    ZkhCtl* h = c->h_ctl;
    digest_from_bytes(st, h->st);
    h->counter = 0;
    h->err = 0;
    for (int i = 0; i < 8; i++) h->par[i] = 0;
    ZKH_CUDA(c, cudaMemcpyAsync(c->d_ctl, h, offsetof(ZkhCtl, local), cudaMemcpyHostToDevice, c->stream));

    if (!cw0_dev) ZKH_TRY(ntt_enqueue(c, c_dev, N, cw0, logM0, false, ws + o_misc));
    ZKH_TRY(eq_enqueue(c, z, v, eqw, ws + o_misc));
    const gl_t *tlo, *thi;
    uint32_t tlb;
    ZKH_TRY(ntt_inverse_tables(c, logM0, &tlo, &thi, &tlb));

    const ZkhTag tag_sc = zkh_make_tag("sc");
    gl_t* msgs = c->d_ctl->msgs;    // [v][3]
    gl_t* chals = c->d_ctl->chals;  // [v]
    const gl_t* cur_in[2] = {c_dev, eqw};
    gl_t* dst = bufA;
    const gl_t* cw_cur = cw0;
    for (uint32_t r = 0; r < v; r++) {
        const size_t Mr = M0 >> r, n = N >> r;
        uint8_t* tree = trees + (4 * M0 - 4 * Mr - r) * 32;
        ZKH_TRY(merkle_enqueue(c, cw_cur, Mr, tree, nullptr, roots + (size_t)r * 32));
        ZKH_TRY(tr_absorb_enqueue(c, "root", (const uint64_t*)(roots + (size_t)r * 32), 4));
        if (r == 0) {
            ZKH_TRY(sc_enqueue_round(c, ZKH_F_PROD2, 3, true, cur_in, nullptr, n, nullptr, msgs, chals, tag_sc));
        } else {
            // columns entering this kernel have length 2n (round r-1 size); it binds them to length n
            gl_t* outp[2] = {dst, dst + n};
            ZKH_TRY(sc_enqueue_round(c, ZKH_F_PROD2, 3, false, cur_in, outp, 2 * n, chals + (r - 1), msgs + (size_t)r * 3,
                                     chals + r, tag_sc));
            cur_in[0] = outp[0];
            cur_in[1] = outp[1];
            dst = (dst == bufA) ? bufB : bufA;
        }
        gl_t* cw_next = cwr + (M0 - Mr);  // round r+1 codeword: offset sum_{i=1}^{r} M0>>i = M0 - Mr
        ZKH_TRY(fold_enqueue(c, cw_cur, cw_next, Mr, logM0, r, chals + r, 0, tlo, thi, tlb));
        cw_cur = cw_next;
    }
    // final word (2^R elements) -> absorb "final"
    ZKH_TRY(tr_absorb_enqueue(c, "final", cw_cur, 1u << R));
    ZKH_CUDA(c, cudaMemcpyAsync(h, c->d_ctl, sizeof(ZkhCtl), cudaMemcpyDeviceToHost, c->stream));
    uint8_t* p = out;
    memcpy(p, &v, 4); memcpy(p + 4, &R, 4); memcpy(p + 8, &Q, 4);
    p += 12;
    ZKH_CUDA(c, cudaMemcpyAsync(p, roots, (size_t)v * 32, cudaMemcpyDeviceToHost, c->stream));
    uint8_t* p_final = p + (size_t)v * 32 + (size_t)v * 24;
    ZKH_CUDA(c, cudaMemcpyAsync(p_final, cw_cur, (size_t)8 << R, cudaMemcpyDeviceToHost, c->stream));
    ZKH_CUDA(c, cudaStreamSynchronize(c->stream));
    if (h->err) return zkh_fail(c, ZKH_ERR_DEVICE, "basefold_open: device error flag set");
    memcpy(p + (size_t)v * 32, h->msgs, (size_t)v * 24);
    digest_to_bytes(h->st, st);

    // ---- queries: positions from the transcript, openings gathered on the device ----
    std::string posbuf((size_t)Q * v * 4, '\0');
    uint32_t* pos = (uint32_t*)&posbuf[0];
    for (uint32_t q = 0; q < Q; q++) {
        uint64_t cur = zkh_tr_idx(st, M0 / 2);
        for (uint32_t r = 0; r < v; r++) {
            uint64_t hh = (M0 >> r) / 2;
            cur = cur % hh;
            pos[q * v + r] = (uint32_t)cur;
        }
    }
    uint32_t* d_pos = (uint32_t*)(ws + o_pos);
    uint8_t* d_q = (uint8_t*)(ws + o_q);
    ZKH_CUDA(c, cudaMemcpyAsync(d_pos, pos, (size_t)Q * v * 4, cudaMemcpyHostToDevice, c->stream));
    const uint32_t nthreads = Q * v * 2;
    bf_query_kernel<<<(nthreads + 127) / 128, 128, 0, c->stream>>>(cw0, cwr, trees, logM0, v, Q, d_pos, d_q, per_query);
    ZKH_CUDA(c, cudaGetLastError());
    uint8_t* p_q = p_final + ((size_t)8 << R);
    ZKH_CUDA(c, cudaMemcpyAsync(p_q, d_q, (size_t)Q * per_query, cudaMemcpyDeviceToHost, c->stream));
    ZKH_CUDA(c, cudaStreamSynchronize(c->stream));
    uint8_t* p_z = p_q + (size_t)Q * per_query;
    memcpy(p_z, z, (size_t)v * 8);
    memcpy(p_z + (size_t)v * 8, &y, 8);
    *written = (size_t)(p_z + (size_t)v * 8 + 8 - out);
    if (*written != need) return zkh_fail(c, ZKH_ERR_DEVICE, "basefold_open: internal size mismatch");
    return ZKH_OK;
}
