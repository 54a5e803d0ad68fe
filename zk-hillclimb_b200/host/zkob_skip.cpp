// Driver for the skip-connection obligation of the reference's first proof stack: Z = A + B, checked purely on the public row
// commitments, com_Z[j] == com_A[j] + com_B[j], with the command line and exit codes of the reference's zkob_skip
// (zkllm-src/zkob_skip.cu:1-27).  The commitment files are the proof: no witness, no transcript.
//
//   zkob_skip add    <com_A.bin> <com_B.bin> <com_Z_out.bin> [--claims <accdir> <obid>]      (prover side)
//   zkob_skip verify <com_A.bin> <com_B.bin> <com_Z.bin>     [--claims <vaccdir> <obid>]
//   zkob_skip serve
//
// The sums written by `add` are the reference's Jacobian triples byte for byte.  --claims is accepted for uniformity with the
// other drivers and emits nothing: the verdict of this obligation is final.  Exit 0 = success / ACCEPT, 1 = REJECT.
#include "zkob_common.hpp"

using namespace zkob;

namespace {

std::vector<uint8_t> load_points(const std::string& path) {
    std::vector<uint8_t> b = read_file(path);
    if (b.empty() || b.size() % G1B) throw std::runtime_error(path + ": not a vector of 144-byte points");
    return b;
}
int base_argc(int argc, char** argv, bool& claims) {
    claims = false;
    for (int i = 2; i < argc; i++) {
        if (strncmp(argv[i], "--", 2)) continue;
        if (std::string(argv[i]) != "--claims") throw std::invalid_argument(std::string("flag not built in this driver: ") + argv[i]);
        claims = true;
        return i;
    }
    return argc;
}
int run1(int argc, char** argv) {
    const std::string mode = argc > 1 ? argv[1] : "";
    try {
        bool claims = false;
        const int n = base_argc(argc, argv, claims);
        if (mode == "add" && n == 5) {
            const std::vector<uint8_t> a = load_points(argv[2]), b = load_points(argv[3]);
            if (a.size() != b.size()) throw std::runtime_error("commitment row counts differ");
            Ctx x;
            Dev da(x, a.data(), a.size()), db(x, b.data(), b.size()), dz(x, a.size());
            x.ck(zkh_g1_rows_add(x.c, da.p, db.p, (uint32_t)(a.size() / G1B), dz.p), "homomorphic sum");
            write_file(argv[4], dz.host());
            std::cout << "WROTE homomorphic sum -> " << argv[4] << std::endl;
            if (claims) std::cout << "claim mode: 0 claims emitted (skip has no opening tail)" << std::endl;
            return 0;
        }
        if (mode == "verify" && n == 5) {
            const std::vector<uint8_t> a = load_points(argv[2]), b = load_points(argv[3]), z = load_points(argv[4]);
            if (a.size() != b.size() || a.size() != z.size()) { std::cout << "REJECT: commitment row counts" << std::endl; return 1; }
            Ctx x;
            Dev da(x, a.data(), a.size()), db(x, b.data(), b.size()), dz(x, z.data(), z.size());
            const Fr one = fr_u32(1);
            uint32_t bad = 0;
            x.ck(zkh_g1_rows_check(x.c, dz.p, da.p, one.v, db.p, (uint32_t)(a.size() / G1B), &bad), "row sums");
            if (bad) { std::cout << "REJECT: skip add fails at " << bad << " rows" << std::endl; return 1; }
            std::cout << "ACCEPT" << std::endl;
            if (claims) std::cout << "claim mode: 0 claims emitted; verdict FINAL (not gated on opening_batch)" << std::endl;
            return 0;
        }
    } catch (const std::invalid_argument& e) {
        std::cerr << "zkob_skip: " << e.what() << std::endl;
        return 2;
    }
    std::cerr << "usage: zkob_skip add a b z [--claims <accdir> <obid>] | verify a b z [--claims <vaccdir> <obid>] | serve" << std::endl;
    return 2;
}

}  // namespace

int main(int argc, char** argv) {
    try {
        if (argc > 1 && std::string(argv[1]) == "serve") return serve_loop(argv[0], run1);
        return run1(argc, argv);
    } catch (const std::exception& e) {
        std::cerr << "zkob_skip: " << e.what() << std::endl;
        return 3;
    }
}
