// The integer decoder layer proved from C++ (include/zkh_p3_layer.hpp over libzkh.so): reads the layer's inputs as signed 32-bit
// integers, runs the witness chain, the commitments and p3itf::prove on the GPU, writes the serialised layer proof.
//   zkh_p3_layer <inputs.i32> <proof.bin> <seq> <d> <nh> <dh> <dff> <batch> <R> <Q> <transcript seed> [layers] [workers] [warmup]
// layers > 1 proves the same inputs that many times (a stand-in for independent layers; layer l > 0 runs on the transcript
// "<seed>-<l>"); workers > 1 keeps that many proofs in flight, each on its own host thread, library context and stream;
// warmup = 1 lets every worker prove one untimed layer first (table uploads, workspace growth, the allocator's pool) and starts
// the clock when all are done.  The last line reports the wall time per layer of the timed pass (upload of the inputs from
// page-locked memory, witness chain, commitments, proof).  The GPU is device $ZKH_DEVICE (default 0).  Beside the proof it writes
// <proof.bin>.pub: the commitment roots of the input, the seven weights and the two gains (10 x 32 bytes), then the output grid
// (field elements), i.e. what a verifier holds besides the public input and the RoPE tables.
//   zkh_p3_layer verify <inputs.i32> <proof.bin> <seq> <d> <nh> <dh> <dff> <batch> <R> <Q> <transcript seed>
// checks the proof on the host (no GPU work) against x0 and the RoPE tables of inputs.i32 and <proof.bin>.pub; prints ACCEPT or
// REJECT <reason>; exit code 0 / 1.
// inputs.i32: x0 (seq*batch*d) | the seven weights Wq Wk Wv Wo (d*d each) Wg Wu (d*dff) Wd (dff*d) | g1 g2 (d) | cos, sin tables
// (seq * dh/2 each), all little-endian int32.  Exit code 0 on success, 2 on a usage or I/O error, 3 on a library error.
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <atomic>
#include <fstream>
#include <iterator>
#include <mutex>
#include <thread>

#include "zkh_p3_layer_verify.hpp"

using namespace zkh_p3;

static bool read_i32(std::ifstream& f, HostI32& v) {
    f.read(reinterpret_cast<char*>(v.data()), (std::streamsize)(v.size() * 4));
    return (size_t)f.gcount() == v.size() * 4;
}

static int verify_main(int argc, char** argv) {
    if (argc < 13) { fprintf(stderr, "usage: %s verify <inputs.i32> <proof.bin> <seq> <d> <nh> <dh> <dff> <batch> <R> <Q> <seed>\n", argv[0]); return 2; }
    const ItfConfig c((uint32_t)atoi(argv[4]), (uint32_t)atoi(argv[5]), (uint32_t)atoi(argv[6]), (uint32_t)atoi(argv[7]), (uint32_t)atoi(argv[8]),
                      (uint32_t)atoi(argv[9]));
    const uint32_t R = (uint32_t)atoi(argv[10]), Q = (uint32_t)atoi(argv[11]);
    auto slurp = [](const std::string& path, std::vector<uint8_t>& b) {
        std::ifstream f(path, std::ios::binary);
        if (!f) return false;
        b.assign(std::istreambuf_iterator<char>(f), std::istreambuf_iterator<char>());
        return true;
    };
    std::vector<uint8_t> in, proof, pubb;
    if (!slurp(argv[2], in) || !slurp(argv[3], proof) || !slurp(std::string(argv[3]) + ".pub", pubb)) { fprintf(stderr, "cannot read the inputs\n"); return 2; }
    const size_t ne = (size_t)c.seq * c.batch * c.d, nt = (size_t)c.seq * c.dh / 2;
    size_t wsum = 0;
    for (int i = 0; i < 7; i++) wsum += c.wrows(i) * c.wcols(i);
    if (in.size() < (ne + wsum + 2 * c.d + 2 * nt) * 4 || pubb.size() != 320 + ne * 8) { fprintf(stderr, "input files do not match the configuration\n"); return 2; }
    const int32_t* iv = reinterpret_cast<const int32_t*>(in.data());
    zkh_p3v::ItfPublic pub;
    pub.x0.resize(ne);
    for (size_t k = 0; k < ne; k++) pub.x0[k] = zkh_p3v::lift(iv[k]);
    const int32_t* tabs = iv + ne + wsum + 2 * c.d;
    pub.ct.assign(tabs, tabs + nt);
    pub.st.assign(tabs + nt, tabs + 2 * nt);
    const uint8_t* q = pubb.data();
    memcpy(pub.rX0.data(), q, 32);
    for (int i = 0; i < 7; i++) memcpy(pub.rW[i].data(), q + 32 * (1 + i), 32);
    memcpy(pub.rG1.data(), q + 256, 32);
    memcpy(pub.rG2.data(), q + 288, 32);
    pub.out.resize(ne);
    memcpy(pub.out.data(), q + 320, ne * 8);
    for (gl_t v : pub.out)
        if (v >= GL_P) { printf("REJECT output grid not canonical\n"); return 1; }
    IgTables T(c.d, c.btop);
    Transcript tr(argv[12]);
    const zkh_p3v::Verdict vd = zkh_p3v::guarded([&] { return zkh_p3v::itf_verify(tr, zkh_p3v::Reader(proof), c, T, pub, R, Q); });
    if (vd) { printf("ACCEPT\n"); return 0; }
    printf("REJECT %s\n", vd.why.c_str());
    return 1;
}

int main(int argc, char** argv) {
    if (argc > 1 && std::string(argv[1]) == "verify") {
        try {
            return verify_main(argc, argv);
        } catch (const std::exception& e) {
            fprintf(stderr, "zkh_p3_layer verify: %s\n", e.what());
            return 3;
        }
    }
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
        const int workers = argc > 13 ? std::max(1, atoi(argv[13])) : 1;
        const bool warm = argc > 14 && atoi(argv[14]) > 0;
        const int device = getenv("ZKH_DEVICE") ? atoi(getenv("ZKH_DEVICE")) : 0;
        Prover P0(device);
        ItfInputs in(P0, c);
        bool ok = read_i32(f, in.x0);
        for (int i = 0; i < 7 && ok; i++) ok = read_i32(f, in.w[i]);
        ok = ok && read_i32(f, in.g1) && read_i32(f, in.g2) && read_i32(f, in.ct) && read_i32(f, in.st);
        if (!ok) { fprintf(stderr, "%s is shorter than the configuration needs\n", argv[1]); return 2; }
        std::vector<uint8_t> proof, pubdata;
        std::mutex mu;
        std::atomic<int> next{0}, ready{0};
        std::chrono::steady_clock::time_point w0;
        std::string failure;
        std::atomic<bool> failed{false};
        auto ms = [](auto a, auto b) { return std::chrono::duration<double, std::milli>(b - a).count(); };
        auto worker = [&](int id) {
            try {
                Prover P(device);
                P.keep_trees = getenv("ZKH_LAYER_NO_KEEP") == nullptr;   // codewords and capped trees stay resident for the openings
                IgTables T(c.d, c.btop);
                if (warm) {
                    ItfWit w;
                    itf_build_witness(P, c, T, in, w);
                    ItfCom o = itf_commit_all(P, w, R);
                    Transcript tr(seed + "-warm");
                    itf_prove(P, tr, c, T, w, o, R, Q);
                    P.release_kept();
                }
                if (++ready == workers) w0 = std::chrono::steady_clock::now();      // the last worker to get here starts the clock
                while (ready.load() < workers && !failed.load()) std::this_thread::yield();
                for (int rep = next++; rep < reps; rep = next++) {
                    auto t0 = std::chrono::steady_clock::now();
                    ItfWit w;
                    itf_build_witness(P, c, T, in, w);
                    auto t1 = std::chrono::steady_clock::now();
                    ItfCom o = itf_commit_all(P, w, R);
                    auto t2 = std::chrono::steady_clock::now();
                    Transcript tr(rep ? seed + "-" + std::to_string(rep) : seed);
                    std::vector<uint8_t> pf = itf_prove(P, tr, c, T, w, o, R, Q);
                    auto t3 = std::chrono::steady_clock::now();
                    P.release_kept();
                    std::lock_guard<std::mutex> lk(mu);
                    printf("{\"layer\": %d, \"worker\": %d, \"witness_ms\": %.3f, \"commit_ms\": %.3f, \"prove_ms\": %.3f, \"proof_bytes\": %zu}\n", rep, id,
                           ms(t0, t1), ms(t1, t2), ms(t2, t3), pf.size());
                    fflush(stdout);
                    if (rep == 0) {
                        proof.swap(pf);
                        const CCol* rr[10] = {&o.x0, &o.w[0], &o.w[1], &o.w[2], &o.w[3], &o.w[4], &o.w[5], &o.w[6], &o.g1, &o.g2};
                        pubdata.clear();
                        for (const CCol* r : rr) pubdata.insert(pubdata.end(), r->root.begin(), r->root.end());
                        const std::vector<gl_t> og = w.out.to_host();
                        const uint8_t* ob = reinterpret_cast<const uint8_t*>(og.data());
                        pubdata.insert(pubdata.end(), ob, ob + og.size() * 8);
                    }
                }
            } catch (const std::exception& e) {
                std::lock_guard<std::mutex> lk(mu);
                failure = e.what();
                failed = true;
                ready += workers;                 // nobody waits for a worker that failed
            }
        };
        std::vector<std::thread> th;
        for (int i = 1; i < workers; i++) th.emplace_back(worker, i);
        worker(0);
        for (auto& t : th) t.join();
        const auto w1 = std::chrono::steady_clock::now();
        if (failed) throw std::runtime_error(failure);
        printf("{\"layers\": %d, \"workers\": %d, \"wall_ms\": %.3f, \"ms_per_layer\": %.3f}\n", reps, workers, ms(w0, w1), ms(w0, w1) / reps);
        std::ofstream g(argv[2], std::ios::binary);
        g.write(reinterpret_cast<const char*>(proof.data()), (std::streamsize)proof.size());
        if (!g) { fprintf(stderr, "cannot write %s\n", argv[2]); return 2; }
        std::ofstream gp(std::string(argv[2]) + ".pub", std::ios::binary);
        gp.write(reinterpret_cast<const char*>(pubdata.data()), (std::streamsize)pubdata.size());
        if (!gp) { fprintf(stderr, "cannot write %s.pub\n", argv[2]); return 2; }
        return 0;
    } catch (const std::exception& e) {
        fprintf(stderr, "zkh_p3_layer: %s\n", e.what());
        return 3;
    }
}
