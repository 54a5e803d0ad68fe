// The integer decoder layer proved from C++ (include/zkh_p3_layer.hpp over libzkh.so): reads the layer's inputs as signed 32-bit
// integers, runs the witness chain, the commitments and p3itf::prove on the GPU, writes the serialised layer proof.
//   zkh_p3_layer <inputs.i32> <proof.bin> <seq> <d> <nh> <dh> <dff> <batch> <R> <Q> <transcript seed> [repeats]
// inputs.i32: x0 (seq*batch*d) | the seven weights Wq Wk Wv Wo (d*d each) Wg Wu (d*dff) Wd (dff*d) | g1 g2 (d) | cos, sin tables
// (seq * dh/2 each), all little-endian int32.  Exit code 0 on success, 2 on a usage or I/O error, 3 on a library error.
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <fstream>

#include "zkh_p3_layer.hpp"

using namespace zkh_p3;

static bool read_i32(std::ifstream& f, std::vector<int32_t>& v, size_t n) {
    v.resize(n);
    f.read(reinterpret_cast<char*>(v.data()), (std::streamsize)(n * 4));
    return (size_t)f.gcount() == n * 4;
}

int main(int argc, char** argv) {
    if (argc < 12) {
        fprintf(stderr, "usage: %s <inputs.i32> <proof.bin> <seq> <d> <nh> <dh> <dff> <batch> <R> <Q> <seed> [repeats]\n", argv[0]);
        return 2;
    }
    try {
        const ItfConfig c((uint32_t)atoi(argv[3]), (uint32_t)atoi(argv[4]), (uint32_t)atoi(argv[5]), (uint32_t)atoi(argv[6]),
                          (uint32_t)atoi(argv[7]), (uint32_t)atoi(argv[8]));
        const uint32_t R = (uint32_t)atoi(argv[9]), Q = (uint32_t)atoi(argv[10]);
        const std::string seed = argv[11];
        const int reps = argc > 12 ? atoi(argv[12]) : 1;
        std::ifstream f(argv[1], std::ios::binary);
        if (!f) { fprintf(stderr, "cannot open %s\n", argv[1]); return 2; }
        ItfInputs in;
        bool ok = read_i32(f, in.x0, (size_t)c.seq * c.batch * c.d);
        for (int i = 0; i < 7 && ok; i++) ok = read_i32(f, in.w[i], c.wrows(i) * c.wcols(i));
        ok = ok && read_i32(f, in.g1, c.d) && read_i32(f, in.g2, c.d) && read_i32(f, in.ct, (size_t)c.seq * c.dh / 2) &&
             read_i32(f, in.st, (size_t)c.seq * c.dh / 2);
        if (!ok) { fprintf(stderr, "%s is shorter than the configuration needs\n", argv[1]); return 2; }
        Prover P(0);
        IgTables T(c.d, c.btop);
        std::vector<uint8_t> proof;
        for (int rep = 0; rep < reps; rep++) {
            auto t0 = std::chrono::steady_clock::now();
            ItfWit w;
            itf_build_witness(P, c, T, in, w);
            auto t1 = std::chrono::steady_clock::now();
            ItfCom o = itf_commit_all(P, w, R);
            auto t2 = std::chrono::steady_clock::now();
            Transcript tr(seed);
            proof = itf_prove(P, tr, c, T, w, o, R, Q);
            auto t3 = std::chrono::steady_clock::now();
            auto ms = [](auto a, auto b) { return std::chrono::duration<double, std::milli>(b - a).count(); };
            printf("{\"rep\": %d, \"witness_ms\": %.3f, \"commit_ms\": %.3f, \"prove_ms\": %.3f, \"proof_bytes\": %zu}\n", rep, ms(t0, t1),
                   ms(t1, t2), ms(t2, t3), proof.size());
            fflush(stdout);
        }
        std::ofstream g(argv[2], std::ios::binary);
        g.write(reinterpret_cast<const char*>(proof.data()), (std::streamsize)proof.size());
        if (!g) { fprintf(stderr, "cannot write %s\n", argv[2]); return 2; }
        return 0;
    } catch (const std::exception& e) {
        fprintf(stderr, "zkh_p3_layer: %s\n", e.what());
        return 3;
    }
}
