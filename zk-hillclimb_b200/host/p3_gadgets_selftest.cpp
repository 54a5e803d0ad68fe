// Host-side C++ over the C ABI, gadget level: a quantised matmul proof and the rescale of its output with range lookups
// (the reference's configs of p3imm::prove + p3irs::prove), standalone and composed on one transcript with a shared opening
// ledger, one merged-lookup flush and one batched-opening pass -- written against include/zkh_p3.hpp only.
// Prints "name hex" lines; the test suite recomputes every line with the Python host logic, which is pinned to the
// reference's provers and verifiers.
//
//   zkh_p3_gadgets_selftest [li] [lj] [lk] [sf] [R] [Q]       X: 2^li x 2^lj, W: 2^lj x 2^lk (default 4 6 5 16 1 24)
#include <cstdio>
#include <cstdlib>

#include "zkh_p3.hpp"

using namespace zkh_p3;

static int64_t next_i8(uint64_t& s) {
    s = s * 6364136223846793005ULL + 1442695040888963407ULL;
    return (int64_t)((s >> 33) % 255) - 127;
}
static gl_t lift(int64_t x) { return x >= 0 ? (gl_t)x : GL_P - (gl_t)(-x); }
static void put(const char* name, const void* p, size_t n) {
    const uint8_t* b = static_cast<const uint8_t*>(p);
    printf("%s ", name);
    for (size_t i = 0; i < n; i++) printf("%02x", b[i]);
    printf("\n");
}
static std::vector<uint8_t> cat(const std::vector<std::vector<uint8_t>>& v) {
    std::vector<uint8_t> out;
    for (auto& x : v) put_blob(out, x);
    return out;
}

int main(int argc, char** argv) {
    auto arg = [&](int i, uint32_t d) { return argc > i ? (uint32_t)atoi(argv[i]) : d; };
    const uint32_t li = arg(1, 4), lj = arg(2, 6), lk = arg(3, 5), sf = arg(4, 16), R = arg(5, 1), Q = arg(6, 24);
    const size_t I = (size_t)1 << li, J = (size_t)1 << lj, K = (size_t)1 << lk;
    try {
        Prover P(0);
        uint64_t s = 0x5EED;
        std::vector<int64_t> x(I * J), w(J * K), y(I * K, 0);
        for (auto& v : x) v = next_i8(s);
        for (auto& v : w) v = next_i8(s);
        for (size_t i = 0; i < I; i++)
            for (size_t j = 0; j < J; j++)
                for (size_t k = 0; k < K; k++) y[i * K + k] += x[i * J + j] * w[j * K + k];
        auto lifted = [](const std::vector<int64_t>& a) { std::vector<gl_t> o(a.size()); for (size_t t = 0; t < a.size(); t++) o[t] = lift(a[t]); return o; };
        DevCol dX(P, lifted(x)), dW(P, lifted(w)), dY(P, lifted(y));
        const CCol X{&dX, P.commit_gpu_rootonly(dX, R)}, W{&dW, P.commit_gpu_rootonly(dW, R)}, Y{&dY, P.commit_gpu_rootonly(dY, R)};
        put("root_Y", Y.root.data(), 32);
        {   // standalone matmul proof
            Transcript tr("cxx-imm");
            std::vector<uint8_t> pf = imm_prove(P, tr, X, W, Y, lj, lk, li, R, Q);
            put("imm_proof", pf.data(), pf.size());
            put("imm_state", tr.state, 32);
        }
        IrsTables T(sf > 16 && sf < 32 ? sf - 16 : 1);
        {   // standalone rescale of the accumulators
            Transcript tr("cxx-irs");
            DevCol yo;
            Hash ry;
            std::vector<uint8_t> pf = irs_prove(P, tr, T, Y, yo, ry, li + lk, sf, 1, R, Q);
            put("irs_proof", pf.data(), pf.size());
            put("irs_state", tr.state, 32);
            put("irs_rootY", ry.data(), 32);
        }
        {   // composed: one transcript, one ledger, one lookup flush, one batched-opening pass
            Transcript tr("cxx-c0");
            XCtx xc;
            std::vector<uint8_t> p1 = imm_prove(P, tr, X, W, Y, lj, lk, li, R, Q, &xc);
            DevCol yo;
            Hash ry;
            std::vector<uint8_t> p2 = irs_prove(P, tr, T, Y, yo, ry, li + lk, sf, 1, R, Q, &xc);
            std::vector<uint8_t> lug = cat(lu_flush(P, tr, xc, R));
            std::vector<uint8_t> bo = cat(tail_prove(P, tr, xc.lg, R, Q, "c0-bo"));
            put("c0_imm", p1.data(), p1.size());
            put("c0_irs", p2.data(), p2.size());
            put("c0_lug", lug.data(), lug.size());
            put("c0_batches", bo.data(), bo.size());
            put("c0_state", tr.state, 32);
        }
    } catch (const std::exception& e) {
        fprintf(stderr, "selftest failed: %s\n", e.what());
        return 1;
    }
    return 0;
}
