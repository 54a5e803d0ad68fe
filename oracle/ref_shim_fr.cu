// C window on the UNMODIFIED reference's BLS12-381 Fr stack (test infrastructure; needs a GPU to run,
// because that stack does even scalar arithmetic in one-thread kernels).  Built by `make -C oracle ref_fr`
// into oracle/_ref/libfrref.so from the reference sources where they lie; nothing is copied.
//
// Exposes the reference's own: k_fr_fold, build_eq_tensor, FrTensor::partial_me / operator()(u),
// fs_hadamard, fs_quartic, and the zkob_fc inner-product rounds driven with the reference's
// zkip_poly_kernel / zkip_reduce_kernel, FrTensor::sum and lagrange-free host glue
// (zkllm-src/zkob_fc.cu:290-332 is inside that program's main flow, so the loop is restated here
// around the reference kernels).
#include "zkob_lookup.cuh"
#include "zkfc.cuh"
#include <chrono>

// defined in the reference's zkfc.cu (zkob_fc.cu declares them the same way before use)
KERNEL void zkip_poly_kernel(GLOBAL Fr_t* a, GLOBAL Fr_t* b, GLOBAL Fr_t* out0, GLOBAL Fr_t* out1, GLOBAL Fr_t* out2,
                             uint N_in, uint N_out);
KERNEL void zkip_reduce_kernel(GLOBAL Fr_t* a, GLOBAL Fr_t* b, GLOBAL Fr_t* new_a, GLOBAL Fr_t* new_b, Fr_t v, uint N_in,
                               uint N_out);

KERNEL void tlookup_inv_kernel(Fr_t* in_data, Fr_t beta, Fr_t* out_data, uint N);   // reference's tlookup.cu

namespace {
std::vector<Fr_t> vec_from(const uint32_t* p, uint32_t n) {
    std::vector<Fr_t> v(n);
    memcpy(v.data(), p, (size_t)n * 32);
    return v;
}
fs::Transcript tr_from(const uint8_t st[32]) {
    fs::Transcript tr("x");
    memcpy(tr.state, st, 32);
    return tr;
}
double now_ms() {
    return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now().time_since_epoch()).count();
}
void to_host(const FrTensor& t, uint32_t* out) {
    cudaMemcpy(out, t.gpu_data, (size_t)t.size * 32, cudaMemcpyDeviceToHost);
}
}  // namespace

extern "C" {

int refA_gpu_available() {
    int n = 0;
    return cudaGetDeviceCount(&n) == cudaSuccess && n > 0;
}
int refA_fold(const uint32_t* in, uint32_t n, const uint32_t* w, uint32_t* out) {
    FrTensor t(n, (const Fr_t*)in), o(n / 2);
    Fr_t wv; memcpy(&wv, w, 32);
    k_fr_fold<<<(n / 2 + 255) / 256, 256>>>(t.gpu_data, wv, o.gpu_data, n / 2);
    cudaDeviceSynchronize();
    to_host(o, out);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
int refA_eq(const uint32_t* u, uint32_t v, uint32_t* out) {
    FrTensor E = build_eq_tensor(vec_from(u, v));
    to_host(E, out);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
int refA_partial_me(const uint32_t* t, uint32_t n, const uint32_t* u, uint32_t nu, uint32_t cur_dim, uint32_t window,
                    uint32_t* out, double* ms_out) {
    try {
        FrTensor T(n, (const Fr_t*)t);
        cudaDeviceSynchronize();
        double t0 = now_ms();
        FrTensor R = T.partial_me(vec_from(u, nu), cur_dim, window);
        cudaDeviceSynchronize();
        if (ms_out) *ms_out = now_ms() - t0;
        to_host(R, out);
        return (int)R.size;
    } catch (...) { return -1; }
}
int refA_me(const uint32_t* t, uint32_t n, const uint32_t* u, uint32_t nu, uint32_t* out) {
    try {
        FrTensor T(n, (const Fr_t*)t);
        Fr_t y = T(vec_from(u, nu));
        memcpy(out, &y, 32);
        return 0;
    } catch (...) { return -1; }
}
// fs_hadamard (zkob_lookup.cuh:297-318): evals 4 per round, ws the challenges, terminals S, U
int refA_hadamard(uint8_t st[32], const uint32_t* E, const uint32_t* S, const uint32_t* U, uint32_t n, uint32_t* evals,
                  uint32_t* ws, uint32_t* fin, double* ms_out) {
    try {
        FrTensor e(n, (const Fr_t*)E), s(n, (const Fr_t*)S), u(n, (const Fr_t*)U);
        fs::Transcript tr = tr_from(st);
        std::vector<Fr_t> w;
        HadamardProof hp;
        cudaDeviceSynchronize();
        double t0 = now_ms();
        fs_hadamard(F_ZERO, e, s, u, tr, w, hp, false);
        cudaDeviceSynchronize();
        if (ms_out) *ms_out = now_ms() - t0;
        memcpy(evals, hp.ev.data(), hp.ev.size() * 32);
        memcpy(ws, w.data(), w.size() * 32);
        memcpy(fin, &hp.S_f2, 32); memcpy(fin + 8, &hp.U_f2, 32);
        memcpy(st, tr.state, 32);
        return 0;
    } catch (...) { return -1; }
}
// fs_quartic (zkob_lookup.cuh:402-425)
int refA_quartic(uint8_t st[32], const char* tag, const uint32_t* E, const uint32_t* A, const uint32_t* B,
                 const uint32_t* Cc, uint32_t n, uint32_t* evals, uint32_t* ws, uint32_t* fin, double* ms_out) {
    try {
        FrTensor e(n, (const Fr_t*)E), a(n, (const Fr_t*)A), b(n, (const Fr_t*)B), c(n, (const Fr_t*)Cc);
        fs::Transcript tr = tr_from(st);
        std::vector<Fr_t> w;
        QuarticProof qp;
        cudaDeviceSynchronize();
        double t0 = now_ms();
        fs_quartic(F_ZERO, e, a, b, c, tr, tag, w, qp, false);
        cudaDeviceSynchronize();
        if (ms_out) *ms_out = now_ms() - t0;
        memcpy(evals, qp.ev.data(), qp.ev.size() * 32);
        memcpy(ws, w.data(), w.size() * 32);
        memcpy(fin, &qp.A_f, 32); memcpy(fin + 8, &qp.B_f, 32); memcpy(fin + 16, &qp.C_f, 32);
        memcpy(st, tr.state, 32);
        return 0;
    } catch (...) { return -1; }
}
// inner-product rounds with the reference kernels (zkfc.cu:94-127) and the transcript schedule of
// zkob_fc.cu:290-332 (non-private mode): absorb p0, p1, p2; challenge; reduce.
int refA_ip_rounds(uint8_t st[32], const uint32_t* a, const uint32_t* b, uint32_t n, uint32_t* evals, uint32_t* xs,
                   uint32_t* fin, double* ms_out) {
    try {
        FrTensor A(n, (const Fr_t*)a), B(n, (const Fr_t*)b);
        fs::Transcript tr = tr_from(st);
        Fr_t *da = nullptr, *db = nullptr, *da2 = nullptr, *db2 = nullptr;
        cudaMalloc(&da, (size_t)n * 32); cudaMalloc(&db, (size_t)n * 32);
        cudaMalloc(&da2, (size_t)n * 32); cudaMalloc(&db2, (size_t)n * 32);
        cudaMemcpy(da, A.gpu_data, (size_t)n * 32, cudaMemcpyDeviceToDevice);
        cudaMemcpy(db, B.gpu_data, (size_t)n * 32, cudaMemcpyDeviceToDevice);
        uint32_t sz = n, r = 0;
        cudaDeviceSynchronize();
        double t0 = now_ms();
        while (sz > 1) {
            uint32_t N_out = sz / 2;
            FrTensor o0(N_out), o1(N_out), o2(N_out);
            zkip_poly_kernel<<<(N_out + 63) / 64, 64>>>(da, db, o0.gpu_data, o1.gpu_data, o2.gpu_data, sz, N_out);
            cudaDeviceSynchronize();
            Fr_t c0 = o0.sum(), c1 = o1.sum(), c2 = o2.sum();
            Fr_t p0 = c0;
            Fr_t p1 = h_scalar(h_scalar(c0, c1, 0), c2, 0);
            Fr_t p2 = h_scalar(h_scalar(c0, h_scalar(F_TWO, c1, 2), 0), h_scalar(h_scalar(F_TWO, F_TWO, 2), c2, 2), 0);
            absorb_fr(tr, "p0", p0); absorb_fr(tr, "p1", p1); absorb_fr(tr, "p2", p2);
            Fr_t x = fs_challenge_fr(tr);
            memcpy(evals + (size_t)r * 24, &p0, 32); memcpy(evals + (size_t)r * 24 + 8, &p1, 32);
            memcpy(evals + (size_t)r * 24 + 16, &p2, 32);
            memcpy(xs + (size_t)r * 8, &x, 32);
            zkip_reduce_kernel<<<(N_out + 63) / 64, 64>>>(da, db, da2, db2, x, sz, N_out);
            cudaDeviceSynchronize();
            std::swap(da, da2); std::swap(db, db2);
            sz = N_out; r++;
        }
        cudaDeviceSynchronize();
        if (ms_out) *ms_out = now_ms() - t0;
        cudaMemcpy(fin, da, 32, cudaMemcpyDeviceToHost);
        cudaMemcpy(fin + 8, db, 32, cudaMemcpyDeviceToHost);
        cudaFree(da); cudaFree(db); cudaFree(da2); cudaFree(db2);
        memcpy(st, tr.state, 32);
        return cudaGetLastError() == cudaSuccess ? 0 : -2;
    } catch (...) { return -1; }
}

// tLookup over Fr: tlookup_inv_kernel for A and B, then fs_phase1 / fs_phase2 (zkob_lookup.cuh:143-198) with
// the scalars set up as zkob_rescale.cu:119-142 does.  terms: A_f, S_f, B_f, T_f, m_f.
int refA_lookup(uint8_t st[32], const uint32_t* S, const uint32_t* T, const uint32_t* m, uint32_t D, uint32_t N,
                const uint32_t* alpha_, const uint32_t* beta_, const uint32_t* u, uint32_t* A_out, uint32_t* evals,
                uint32_t* ws_out, uint32_t* terms, double* ms_out) {
    try {
        FrTensor Sx(D, (const Fr_t*)S), Tx(N, (const Fr_t*)T), mx(N, (const Fr_t*)m);
        Fr_t alpha, beta;
        memcpy(&alpha, alpha_, 32); memcpy(&beta, beta_, 32);
        uint32_t logD = 0; while ((1u << logD) < D) logD++;
        std::vector<Fr_t> uu = vec_from(u, logD);
        fs::Transcript tr = tr_from(st);
        cudaDeviceSynchronize();
        double t0 = now_ms();
        FrTensor A(D), Bv(N);
        tlookup_inv_kernel<<<(D + FrNumThread - 1) / FrNumThread, FrNumThread>>>(Sx.gpu_data, beta, A.gpu_data, D);
        tlookup_inv_kernel<<<(N + FrNumThread - 1) / FrNumThread, FrNumThread>>>(Tx.gpu_data, beta, Bv.gpu_data, N);
        cudaDeviceSynchronize();
        Fr_t alpha_sq = alpha * alpha;
        Fr_t Cc = alpha_sq - (Bv * mx).sum();
        Fr_t claim = alpha + alpha_sq;
        Fr_t inv_ratio = Fr_t{N, 0, 0, 0, 0, 0, 0, 0} / Fr_t{D, 0, 0, 0, 0, 0, 0, 0};
        LookupProof pf;
        std::vector<Fr_t> ws;
        fs_phase1(claim, A, Sx, Bv, Tx, mx, alpha, beta, Cc, inv_ratio, alpha_sq, uu, tr, ws, pf, false);
        cudaDeviceSynchronize();
        if (ms_out) *ms_out = now_ms() - t0;
        to_host(A, A_out);
        memcpy(evals, pf.ev.data(), pf.ev.size() * 32);
        memcpy(ws_out, ws.data(), ws.size() * 32);
        memcpy(terms, &pf.A_f, 32); memcpy(terms + 8, &pf.S_f, 32); memcpy(terms + 16, &pf.B_f, 32);
        memcpy(terms + 24, &pf.T_f, 32); memcpy(terms + 32, &pf.m_f, 32);
        memcpy(st, tr.state, 32);
        return 0;
    } catch (...) { return -1; }
}

// Pedersen row commitments of the reference (Commitment::random / Commitment::commit, zkllm-src/commitment.cu:3-8, :41-103):
// generators and commitments as the reference's 144-byte Jacobian triples
int refA_commit_random(uint32_t n, uint8_t* gens_out) {
    Commitment g = Commitment::random(n);
    cudaMemcpy(gens_out, g.gpu_data, (size_t)n * sizeof(G1Jacobian_t), cudaMemcpyDeviceToHost);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
int refA_pedersen_commit(const uint8_t* gens, uint32_t n, const uint32_t* scalars, uint32_t m, uint8_t* out, double* ms) {
    Commitment g(n, (const G1Jacobian_t*)gens);
    FrTensor t(m * n, (const Fr_t*)scalars);
    cudaDeviceSynchronize();
    const double t0 = now_ms();
    G1TensorJacobian c = g.commit(t);          // synchronises after each of its two kernels
    if (ms) *ms = now_ms() - t0;
    cudaMemcpy(out, c.gpu_data, (size_t)m * sizeof(G1Jacobian_t), cudaMemcpyDeviceToHost);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// Openings of the reference (zkllm-src/vrf_common.cuh): dev_msm, fold_chain, ipa_prove and ipa_verify as they stand.
// Points: 144-byte Jacobian triples; scalars: 32-byte Fr_t; st: the transcript state, advanced in place.
int refA_msm(const uint8_t* gens, const uint32_t* scalars, uint32_t n, uint8_t* out, double* ms) {
    Commitment g(n, (const G1Jacobian_t*)gens);
    FrTensor a(n, (const Fr_t*)scalars);
    cudaDeviceSynchronize();
    const double t0 = now_ms();
    G1Jacobian_t r = dev_msm(g.gpu_data, a.gpu_data, n);
    if (ms) *ms = now_ms() - t0;
    memcpy(out, &r, sizeof r);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
int refA_fold_chain(const uint8_t* pts, uint32_t size, const uint32_t* us, uint32_t nu, int orientation, uint8_t* out, double* ms) {
    Commitment c(size, (const G1Jacobian_t*)pts);
    std::vector<Fr_t> u = vec_from(us, nu);
    cudaDeviceSynchronize();
    const double t0 = now_ms();
    G1Jacobian_t r = fold_chain(c.gpu_data, size, u, orientation);
    if (ms) *ms = now_ms() - t0;
    memcpy(out, &r, sizeof r);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
int refA_ipa_prove(const uint32_t* a, const uint32_t* b, const uint8_t* gens, const uint8_t* Q, uint32_t n, uint8_t st[32],
                   uint8_t* L, uint8_t* R, uint32_t* a_final, double* ms) {
    try {
        Commitment g(n, (const G1Jacobian_t*)gens);
        FrTensor av(n, (const Fr_t*)a);
        std::vector<Fr_t> bv = vec_from(b, n);
        G1Jacobian_t q; memcpy(&q, Q, sizeof q);
        fs::Transcript tr = tr_from(st);
        cudaDeviceSynchronize();
        const double t0 = now_ms();
        IpaProof pf = ipa_prove(av.gpu_data, bv, g.gpu_data, q, n, tr);
        if (ms) *ms = now_ms() - t0;
        if (!pf.L.empty()) {
            memcpy(L, pf.L.data(), pf.L.size() * sizeof(G1Jacobian_t));
            memcpy(R, pf.R.data(), pf.R.size() * sizeof(G1Jacobian_t));
        }
        memcpy(a_final, &pf.a_final, 32);
        memcpy(st, tr.state, 32);
        return cudaGetLastError() == cudaSuccess ? 0 : -1;
    } catch (...) { return -1; }
}
// single group operations of the reference's host helpers (h_add / subtraction through k_g1_addsub, h_mul)
int refA_g1_addsub(const uint8_t* a, const uint8_t* b, int sub, uint8_t* out) {
    G1Jacobian_t x, y, *d, h; memcpy(&x, a, sizeof x); memcpy(&y, b, sizeof y);
    cudaMalloc(&d, sizeof(G1Jacobian_t));
    k_g1_addsub<<<1, 1>>>(x, y, sub, d);
    cudaMemcpy(&h, d, sizeof h, cudaMemcpyDeviceToHost); cudaFree(d);
    memcpy(out, &h, sizeof h);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
int refA_g1_mul(const uint8_t* g, const uint32_t* c, uint8_t* out) {
    G1Jacobian_t x; Fr_t k; memcpy(&x, g, sizeof x); memcpy(&k, c, 32);
    G1Jacobian_t h = h_mul(x, k);
    memcpy(out, &h, sizeof h);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
// returns 1 = accepted, 0 = rejected, -1 = error
int refA_ipa_verify(const uint8_t* gens, uint32_t n, const uint8_t* Q, const uint8_t* P0, const uint32_t* u_b, uint32_t nu,
                    const uint8_t* L, const uint8_t* R, uint32_t rounds, const uint32_t* a_final, uint8_t st[32], double* ms) {
    try {
        Commitment g(n, (const G1Jacobian_t*)gens);
        G1Jacobian_t q, p0; memcpy(&q, Q, sizeof q); memcpy(&p0, P0, sizeof p0);
        IpaProof pf;
        pf.L.resize(rounds); pf.R.resize(rounds);
        if (rounds) { memcpy(pf.L.data(), L, rounds * sizeof(G1Jacobian_t)); memcpy(pf.R.data(), R, rounds * sizeof(G1Jacobian_t)); }
        memcpy(&pf.a_final, a_final, 32);
        fs::Transcript tr = tr_from(st);
        cudaDeviceSynchronize();
        const double t0 = now_ms();
        const bool ok = ipa_verify(g.gpu_data, n, q, p0, vec_from(u_b, nu), pf, tr);
        if (ms) *ms = now_ms() - t0;
        memcpy(st, tr.state, 32);
        return ok ? 1 : 0;
    } catch (...) { return -1; }
}
}  // extern "C"
