// Host-side C++ over the C ABI: one small proving flow written the way a gadget of the reference is written
// (commit columns, absorb roots, sumcheck, evaluation opening, fractional-sum GKR, batched opening), using only
// include/zkh_p3.hpp.  Prints "name hex" lines; the test suite recomputes every line with the CPU checker.
//
//   zkh_p3_selftest [v] [R] [Q]        columns of 2^v elements, rate 2^-R, Q queries (default 10 1 24)
#include <cstdio>
#include <cstdlib>

#include "zkh_p3.hpp"

using namespace zkh_p3;

static std::vector<gl_t> lcg_fill(size_t n, uint64_t& s) {
    std::vector<gl_t> out(n);
    for (size_t i = 0; i < n; i++) {
        s = s * 6364136223846793005ULL + 1442695040888963407ULL;
        out[i] = (s ^ (s >> 31)) % GL_P;
    }
    return out;
}

static void put(const char* name, const void* p, size_t n) {
    const uint8_t* b = static_cast<const uint8_t*>(p);
    printf("%s ", name);
    for (size_t i = 0; i < n; i++) printf("%02x", b[i]);
    printf("\n");
}

int main(int argc, char** argv) {
    const uint32_t v = argc > 1 ? (uint32_t)atoi(argv[1]) : 10, R = argc > 2 ? (uint32_t)atoi(argv[2]) : 1,
                   Q = argc > 3 ? (uint32_t)atoi(argv[3]) : 24;
    try {
        Prover prover(0);
        uint64_t s = 0xC0FFEEULL;
        std::vector<gl_t> ha = lcg_fill((size_t)1 << v, s), hb = lcg_fill((size_t)1 << v, s);
        DevCol a(prover, ha), b(prover, hb);

        Transcript tr("cxx-selftest");
        Hash ra = prover.commit_gpu_rootonly(a, R), rb = prover.commit_gpu_rootonly(b, R);
        tr.absorb("root", ra.data(), 32);
        tr.absorb("root", rb.data(), 32);
        put("root_a", ra.data(), 32);
        put("root_b", rb.data(), 32);

        std::vector<gl_t> msgs, fin;
        std::vector<gl_t> r = prover.sc_prove_gpu(tr, "sc", {a.data(), b.data()}, 1u << v, ZKH_F_PROD2, 3, nullptr, 0, msgs, &fin);
        put("sc_msgs", msgs.data(), msgs.size() * 8);
        put("sc_chals", r.data(), r.size() * 8);
        put("sc_finals", fin.data(), fin.size() * 8);
        const gl_t ya = prover.eval_h_gpu(a, r);
        if (ya != fin[0]) throw std::runtime_error("bound column differs from its multilinear evaluation");
        if (a.to_host() != ha) throw std::runtime_error("the sumcheck changed its input column");

        std::vector<uint8_t> ev = prover.prove_eval_dev(a, r, ya, R, Q);
        put("eval_proof", ev.data(), ev.size());

        std::vector<gl_t> rfin;
        gl_t cpq[2];
        std::vector<uint8_t> g = prover.gkr_prove(tr, "gkr", a, b, true, rfin, cpq);
        put("gkr_proof", g.data(), g.size());
        put("gkr_rfin", rfin.data(), rfin.size() * 8);
        put("gkr_cpq", cpq, 16);

        std::vector<Prover::Entry> ents = {{&a, ra, 0}, {&b, rb, 1}, {&a, ra, 1}};
        std::vector<uint8_t> bo = prover.prove_class(tr, {r, rfin}, ents, R, Q, "cxx-bo");
        put("batch_proof", bo.data(), bo.size());
        put("state", tr.state, 32);

        // error behaviour: an out-of-range argument throws with the library's message
        bool threw = false;
        try {
            std::vector<gl_t> m2;
            prover.sc_prove_gpu(tr, "sc", {a.data()}, 1u << v, ZKH_F_PROD2, 3, nullptr, 0, m2);
        } catch (const std::runtime_error&) { threw = true; }
        printf("bad_call_throws %d\n", threw ? 1 : 0);
    } catch (const std::exception& e) {
        fprintf(stderr, "selftest failed: %s\n", e.what());
        return 1;
    }
    return 0;
}
