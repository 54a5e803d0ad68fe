// Driver for ONE quantised linear obligation over the Goldilocks / Basefold stack: Y = X . W in integers, then
// Yr = round(Y / 2^sf) with range lookups -- the work the reference splits over its zkob_fc and zkob_rescale drivers
// (zkllm-src/zkob_fc.cu:32-40, zkob_rescale.cu), here as one proof on one transcript (p3imm + p3irs composed: shared
// opening ledger, one merged-lookup flush, one batched opening per size class).
//
// It speaks the orchestrator's driver protocol (orchestrator/common.py:144-184 run_driver, :231-276 DriverPool):
//   exit 0 = success / ACCEPT, 1 = REJECT, anything else = crash;  `serve` prints ZKW-READY, then runs one request per
//   stdin line through the same entry as the one-shot command line and answers "ZKW-RC <rc>" (zkllm-src/zkob_serve.cuh:26-52);
//   the obligation directory is created by the caller, never here; the transcript seed is "<run_seed>:<obligation id>".
//
//   zkob_p3fc commit   <M.i32> <rows> <cols> <R> <root_out.bin>        (a weight IN x OUT, or the input activations B x IN)
//   zkob_p3fc prove    <obdir> <seed> <X.i32> <W.i32> <B> <IN> <OUT> <sf> <R> <Q> [Yr-out.i32] [--claims <accdir> <obid>]
//   zkob_p3fc verify   <obdir> <seed> <B> <IN> <OUT> <sf> <R> <Q> <root_W.bin> [--claims <vaccdir> <obid>]
//   zkob_p3fc selftest
//   zkob_p3fc serve
//
// Files in <obdir>: roots.bin (root_X root_Y root_Yr, 32 bytes each: the prover-supplied commitments that chain to the
// neighbouring obligations) and proof.bin.  The weight commitment is NOT taken from the obligation directory: verify
// absorbs the registered copy, so a prover whose W differs from the registration diverges the transcript.
// With --claims the opening claims the proof discharges are also appended to <dir>/claims.bin (prover and verifier
// each recompute them; a caller may compare the two lists byte for byte) and verify answers "ACCEPT-conditional".
// commit, prove and selftest need a GPU; verify does not.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <exception>
#include <iostream>
#include <sstream>
#include <string>
#include <vector>

#include "zkh_p3.hpp"
#include "zkh_p3_verify.hpp"

using namespace zkh_p3;
namespace V = zkh_p3v;

static std::vector<uint8_t> read_file(const std::string& path) {
    FILE* f = fopen(path.c_str(), "rb");
    if (!f) throw std::runtime_error("cannot open " + path);
    std::vector<uint8_t> b;
    uint8_t buf[1 << 16];
    size_t n;
    while ((n = fread(buf, 1, sizeof buf, f)) > 0) b.insert(b.end(), buf, buf + n);
    fclose(f);
    return b;
}
static void write_file(const std::string& path, const void* p, size_t n, const char* mode = "wb") {
    FILE* f = fopen(path.c_str(), mode);
    if (!f) throw std::runtime_error("cannot write " + path);
    if (n && fwrite(p, 1, n, f) != n) { fclose(f); throw std::runtime_error("short write to " + path); }
    fclose(f);
}
static uint32_t clog2(uint32_t n) { uint32_t l = 0; while ((1u << l) < n) l++; return l; }
static gl_t lift(int64_t x) { return x >= 0 ? (gl_t)x : GL_P - (gl_t)(-x); }

// rows x cols int32 matrix from a file, zero-padded to 2^lr x 2^lc, lifted into the field, row-major
static std::vector<gl_t> load_matrix(const std::string& path, uint32_t rows, uint32_t cols, uint32_t lr, uint32_t lc) {
    std::vector<uint8_t> raw = read_file(path);
    if (raw.size() != (size_t)rows * cols * 4) throw std::runtime_error(path + ": expected " + std::to_string((size_t)rows * cols) + " int32 values");
    const int32_t* v = reinterpret_cast<const int32_t*>(raw.data());
    std::vector<gl_t> out((size_t)1 << (lr + lc), 0);
    for (uint32_t r = 0; r < rows; r++)
        for (uint32_t c = 0; c < cols; c++) out[((size_t)r << lc) | c] = lift(v[(size_t)r * cols + c]);
    return out;
}

struct Shape { uint32_t B, IN, OUT, sf, R, Q, li, lj, lk; };
static Shape shape_of(char** a) {      // <B> <IN> <OUT> <sf> <R> <Q>
    Shape s;
    s.B = (uint32_t)atoi(a[0]); s.IN = (uint32_t)atoi(a[1]); s.OUT = (uint32_t)atoi(a[2]);
    s.sf = (uint32_t)atoi(a[3]); s.R = (uint32_t)atoi(a[4]); s.Q = (uint32_t)atoi(a[5]);
    if (!s.B || !s.IN || !s.OUT || s.sf < 1 || s.sf > 32 || s.R < 1 || s.R > 3 || s.Q < 1) throw std::runtime_error("bad dimensions");
    s.li = clog2(s.B); s.lj = clog2(s.IN); s.lk = clog2(s.OUT);
    if (s.li + s.lk < 1) s.li = 1;      // a column holds at least two elements
    return s;
}

// opening claims of one proof, for a caller that compares the prover's list with the verifier's
static void append_claims(const std::string& dir, const std::string& obid, const std::vector<std::pair<Hash, std::pair<std::vector<gl_t>, gl_t>>>& claims) {
    std::vector<uint8_t> b;
    for (auto& c : claims) {
        put_u32(b, (uint32_t)obid.size());
        put_raw(b, obid.data(), obid.size());
        put_raw(b, c.first.data(), 32);
        put_u32(b, (uint32_t)c.second.first.size());
        put_raw(b, c.second.first.data(), c.second.first.size() * 8);
        put_raw(b, &c.second.second, 8);
    }
    write_file(dir + "/claims.bin", b.data(), b.size(), "ab");
}

static Prover& gpu() {
    static Prover P(0);
    return P;
}

static int do_commit(int argc, char** argv) {
    if (argc != 7) throw std::runtime_error("usage: commit <M.i32> <rows> <cols> <R> <root_out.bin>");
    const uint32_t IN = (uint32_t)atoi(argv[3]), OUT = (uint32_t)atoi(argv[4]), R = (uint32_t)atoi(argv[5]);
    Prover& P = gpu();
    DevCol dW(P, load_matrix(argv[2], IN, OUT, clog2(IN), clog2(OUT)));
    Hash r = P.commit_gpu_rootonly(dW, R);
    write_file(argv[6], r.data(), 32);
    printf("committed %ux%u (R=%u) -> %s\n", IN, OUT, R, argv[6]);
    return 0;
}

struct Proved { std::vector<uint8_t> proof; Hash rX, rW, rY, rYr; std::vector<int32_t> yr; };

static Proved prove_linear(Prover& P, const std::string& seed, const std::vector<gl_t>& X, const std::vector<gl_t>& W, const Shape& s,
                           Ledger* claims_out = nullptr) {
    zkh_ctx* ctx = P.ctx();
    const size_t I = (size_t)1 << s.li, J = (size_t)1 << s.lj, K = (size_t)1 << s.lk;
    DevCol dX(P, X), dW(P, W), dY(P, I * K);
    const int64_t sa[4] = {0, 0, (int64_t)J, 1}, sb[4] = {0, 0, (int64_t)K, 1}, sc[4] = {0, 0, (int64_t)K, 1};
    P.ck(zkh_ig_matmul(ctx, dX.data(), sa, dW.data(), sb, dY.data(), sc, 1, 1, (uint32_t)I, (uint32_t)J, (uint32_t)K));
    Proved out;
    out.rX = P.commit_gpu_rootonly(dX, s.R);
    out.rW = P.commit_gpu_rootonly(dW, s.R);
    out.rY = P.commit_gpu_rootonly(dY, s.R);
    const CCol cX{&dX, out.rX}, cW{&dW, out.rW}, cY{&dY, out.rY};
    Transcript tr(seed);
    XCtx xc;
    IrsTables T(s.sf > 16 && s.sf < 32 ? s.sf - 16 : 1);
    std::vector<uint8_t> pf_imm = imm_prove(P, tr, cX, cW, cY, s.lj, s.lk, s.li, s.R, s.Q, &xc);
    DevCol dYr;
    std::vector<uint8_t> pf_irs = irs_prove(P, tr, T, cY, dYr, out.rYr, s.li + s.lk, s.sf, 1, s.R, s.Q, &xc);
    std::vector<std::vector<uint8_t>> lug = lu_flush(P, tr, xc, s.R);
    if (claims_out) *claims_out = xc.lg;
    std::vector<std::vector<uint8_t>> batches = tail_prove(P, tr, xc.lg, s.R, s.Q, "fc-bo");
    put_blob(out.proof, pf_imm);
    put_blob(out.proof, pf_irs);
    put_tail(out.proof, lug, batches);
    std::vector<gl_t> yr = dYr.to_host();
    out.yr.resize((size_t)s.B * s.OUT);
    for (uint32_t i = 0; i < s.B; i++)
        for (uint32_t k = 0; k < s.OUT; k++) {
            const gl_t v = yr[((size_t)i << s.lk) | k];
            out.yr[(size_t)i * s.OUT + k] = v > GL_P / 2 ? -(int32_t)(GL_P - v) : (int32_t)v;
        }
    return out;
}

static V::Verdict verify_linear(const std::string& seed, const std::vector<uint8_t>& proof, const Hash& rX, const Hash& rW, const Hash& rY,
                                const Hash& rYr, const Shape& s, V::VLedger* claims_out = nullptr) {
    return V::guarded([&]() -> V::Verdict {
        V::Reader pf(proof);
        Transcript tr(seed);
        V::VCtx vc;
        IrsTables T(s.sf > 16 && s.sf < 32 ? s.sf - 16 : 1);
        V::Reader a = pf.blob();
        V::Verdict vd = V::imm_verify(tr, a, rX, rW, rY, s.lj, s.lk, s.li, s.Q, s.R, &vc);
        if (!vd) return vd;
        if (!a.done()) return V::Verdict::reject("imm trailing bytes");
        V::Reader b = pf.blob();
        vd = V::irs_verify(tr, T, b, rY, rYr, s.li + s.lk, s.sf, 1, s.Q, s.R, &vc);
        if (!vd) return vd;
        if (!b.done()) return V::Verdict::reject("irs trailing bytes");
        vd = V::lu_verify_flush(tr, vc, pf);
        if (!vd) return vd;
        if (claims_out) *claims_out = vc.vlg;
        if (pf.u32() != vc.vlg.cls.size()) return V::Verdict::reject("batch count");
        for (size_t i = 0; i < vc.vlg.cls.size(); i++) {
            vd = V::verify_class(tr, vc.vlg.cls[i], pf.blob(), s.Q, s.R, "fc-bo" + std::to_string(i));
            if (!vd) return vd;
        }
        if (!pf.done()) return V::Verdict::reject("trailing bytes");
        return V::Verdict();
    });
}

static void flag_claims(int argc, char** argv, int& base_argc, std::string& dir, std::string& obid) {
    base_argc = argc;
    for (int i = 2; i < argc; i++)
        if (std::string(argv[i]) == "--claims") {
            if (i + 2 >= argc) throw std::runtime_error("--claims <dir> <obligation id>");
            dir = argv[i + 1];
            obid = argv[i + 2];
            base_argc = i;
            return;
        }
}

static int do_prove(int argc, char** argv) {
    int base;
    std::string cdir, obid;
    flag_claims(argc, argv, base, cdir, obid);
    if (base != 12 && base != 13)
        throw std::runtime_error("usage: prove <obdir> <seed> <X.i32> <W.i32> <B> <IN> <OUT> <sf> <R> <Q> [Yr-out.i32] [--claims <accdir> <obid>]");
    const std::string obdir = argv[2], seed = argv[3];
    const Shape s = shape_of(argv + 6);
    const std::vector<gl_t> X = load_matrix(argv[4], s.B, s.IN, s.li, s.lj), W = load_matrix(argv[5], s.IN, s.OUT, s.lj, s.lk);
    Ledger lg;
    Proved p = prove_linear(gpu(), seed, X, W, s, cdir.empty() ? nullptr : &lg);
    uint8_t roots[96];
    memcpy(roots, p.rX.data(), 32); memcpy(roots + 32, p.rY.data(), 32); memcpy(roots + 64, p.rYr.data(), 32);
    write_file(obdir + "/roots.bin", roots, 96);
    write_file(obdir + "/proof.bin", p.proof.data(), p.proof.size());
    if (base == 13) write_file(argv[12], p.yr.data(), p.yr.size() * 4);
    if (!cdir.empty()) {
        std::vector<std::pair<Hash, std::pair<std::vector<gl_t>, gl_t>>> cl;
        for (auto& c : lg.cls)
            for (size_t j = 0; j < c.ents.size(); j++) cl.push_back({c.ents[j].root, {c.pts[c.ents[j].zid], c.ys[j]}});
        append_claims(cdir, obid, cl);
    }
    printf("proved %ux%u . %ux%u, rescale 2^%u: proof %zu bytes -> %s/proof.bin\n", s.B, s.IN, s.IN, s.OUT, s.sf, p.proof.size(), obdir.c_str());
    return 0;
}

static int do_verify(int argc, char** argv) {
    int base;
    std::string cdir, obid;
    flag_claims(argc, argv, base, cdir, obid);
    if (base != 11)
        throw std::runtime_error("usage: verify <obdir> <seed> <B> <IN> <OUT> <sf> <R> <Q> <root_W.bin> [--claims <vaccdir> <obid>]");
    const std::string obdir = argv[2], seed = argv[3];
    const Shape s = shape_of(argv + 4);
    const std::vector<uint8_t> roots = read_file(obdir + "/roots.bin"), rw = read_file(argv[10]), proof = read_file(obdir + "/proof.bin");
    if (roots.size() != 96 || rw.size() != 32) { printf("REJECT: malformed roots\n"); return 1; }
    Hash rX, rW, rY, rYr;
    memcpy(rX.data(), roots.data(), 32); memcpy(rY.data(), roots.data() + 32, 32); memcpy(rYr.data(), roots.data() + 64, 32);
    memcpy(rW.data(), rw.data(), 32);
    V::VLedger lg;
    V::Verdict vd = verify_linear(seed, proof, rX, rW, rY, rYr, s, cdir.empty() ? nullptr : &lg);
    if (!vd) { printf("REJECT: %s\n", vd.why.c_str()); return 1; }
    if (!cdir.empty()) {
        std::vector<std::pair<Hash, std::pair<std::vector<gl_t>, gl_t>>> cl;
        for (auto& c : lg.cls)
            for (auto& e : c.ents) cl.push_back({e.root, {c.pts[e.zid], e.y}});
        append_claims(cdir, obid, cl);
        printf("ACCEPT-conditional (%zu opening claims recomputed and discharged by the proof's batched openings)\n", cl.size());
    } else {
        printf("ACCEPT\n");
    }
    return 0;
}

// honest proof accepted; tampered proof, wrong weight registration and wrong seed rejected
static int do_selftest() {
    Prover& P = gpu();
    Shape s{6, 20, 12, 8, 1, 24, 0, 0, 0};
    s.li = clog2(s.B); s.lj = clog2(s.IN); s.lk = clog2(s.OUT);
    uint64_t st = 0x5EED;
    auto next = [&]() { st = st * 6364136223846793005ULL + 1442695040888963407ULL; return (int64_t)((st >> 33) % 255) - 127; };
    std::vector<gl_t> X((size_t)1 << (s.li + s.lj), 0), W((size_t)1 << (s.lj + s.lk), 0);
    for (uint32_t i = 0; i < s.B; i++) for (uint32_t j = 0; j < s.IN; j++) X[((size_t)i << s.lj) | j] = lift(next());
    for (uint32_t j = 0; j < s.IN; j++) for (uint32_t k = 0; k < s.OUT; k++) W[((size_t)j << s.lk) | k] = lift(next());
    Proved p = prove_linear(P, "selftest:fc", X, W, s);
    int bad = 0;
    auto expect = [&](const char* name, bool got, bool want) {
        printf("%-44s %s\n", name, got == want ? (want ? "ACCEPT" : "REJECT (as it must)") : "WRONG VERDICT (!!)");
        bad += got != want;
    };
    expect("honest proof", (bool)verify_linear("selftest:fc", p.proof, p.rX, p.rW, p.rY, p.rYr, s), true);
    expect("other transcript seed", (bool)verify_linear("selftest:fd", p.proof, p.rX, p.rW, p.rY, p.rYr, s), false);
    Hash other = p.rW;
    other[5] ^= 1;
    expect("weight root differs from the registration", (bool)verify_linear("selftest:fc", p.proof, p.rX, other, p.rY, p.rYr, s), false);
    for (size_t pos : {(size_t)40, p.proof.size() / 3, p.proof.size() / 2, p.proof.size() - 9}) {
        std::vector<uint8_t> t = p.proof;
        t[pos] ^= 0x10;
        expect(("one bit flipped at byte " + std::to_string(pos)).c_str(), (bool)verify_linear("selftest:fc", t, p.rX, p.rW, p.rY, p.rYr, s), false);
    }
    std::vector<uint8_t> cut(p.proof.begin(), p.proof.begin() + p.proof.size() - 100);
    expect("truncated proof", (bool)verify_linear("selftest:fc", cut, p.rX, p.rW, p.rY, p.rYr, s), false);
    printf(bad ? "SELFTEST FAILED\n" : "SELFTEST OK\n");
    return bad ? 1 : 0;
}

static int run1(int argc, char** argv) {
    const std::string mode = argc > 1 ? argv[1] : "";
    if (mode == "commit") return do_commit(argc, argv);
    if (mode == "prove") return do_prove(argc, argv);
    if (mode == "verify") return do_verify(argc, argv);
    if (mode == "selftest") return do_selftest();
    fprintf(stderr, "usage: zkob_p3fc commit|prove|verify|selftest|serve ...\n");
    return 2;
}

// one request per stdin line, the same entry as the one-shot command line, "ZKW-RC <rc>" after each
static int serve(char* argv0) {
    std::cout << "ZKW-READY" << std::endl;
    std::string line;
    while (std::getline(std::cin, line)) {
        std::istringstream iss(line);
        std::vector<std::string> toks;
        for (std::string t; iss >> t;) toks.push_back(t);
        if (toks.empty()) continue;
        std::vector<char*> av{argv0};
        for (auto& t : toks) av.push_back(const_cast<char*>(t.c_str()));
        int rc;
        try {
            rc = run1((int)av.size(), av.data());
        } catch (const std::exception& e) {
            std::cout << "serve: request failed: " << e.what() << std::endl;
            rc = 3;
        }
        fflush(stdout);
        std::cout << "ZKW-RC " << rc << std::endl;
    }
    return 0;
}

int main(int argc, char** argv) {
    try {
        if (argc > 1 && std::string(argv[1]) == "serve") return serve(argv[0]);
        return run1(argc, argv);
    } catch (const std::exception& e) {
        fprintf(stderr, "zkob_p3fc: %s\n", e.what());
        return 3;
    }
}
