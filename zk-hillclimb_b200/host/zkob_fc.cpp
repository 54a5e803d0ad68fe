// Driver for the fully connected (matmul) obligation of the reference's first proof stack (BLS12-381: Pedersen row
// commitments, an inner-product sumcheck over the contraction dimension, three Fiat-Shamir inner-product arguments), with
// the command line, the files and the exit codes of the reference's zkob_fc (zkllm-src/zkob_fc.cu:17-40, :189-484 prove,
// :488-720 verify): a program the orchestrator can launch in its place (orchestrator/common.py:144-184).
//
//   zkob_fc commit  <W-int.bin> <IN> <OUT> <gen_out.bin> <com_out.bin>
//   zkob_fc prove   <obdir> <seed> <X-int.bin> <W-int.bin> <B> <IN> <OUT> <gen_in.bin> <gen_out.bin> <q.bin> [Y-int-out.bin]
//   zkob_fc verify  <obdir> <seed> <B> <IN> <OUT> <com_W.bin> <gen_in.bin> <gen_out.bin> <q.bin>
//   zkob_fc selftest
//   zkob_fc serve
//
// Files in <obdir> (byte for byte the reference's): dims.bin, com_X.bin, com_Y.bin, sumcheck.bin, ipa_W.bin, ipa_X.bin,
// ipa_Y.bin.  Exit 0 = success / ACCEPT, 1 = REJECT, anything else = failure; `serve` prints ZKW-READY and answers
// "ZKW-RC <rc>" per request line (zkllm-src/zkob_serve.cuh:26-52).  The obligation directory is the caller's.
// The claim-accumulator and weight-privacy variants of the reference (--claims, --wpriv, --apriv, --hiding) are not built:
// those flags are refused with exit code 2.
//
// Everything heavy runs through the C ABI of libzkh (commitments, partial evaluations, the sumcheck with its transcript on
// the device, the arguments, fold chains); the host keeps the transcript between those calls and a few scalars.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <exception>
#include <iostream>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#include "zkh.h"

namespace {

constexpr size_t G1B = 144, FRB = 32;

// ------------------------------------------------------------------ scalars on the host (a handful per proof)
struct Fr { uint32_t v[8]; };
const Fr FR_MOD = {{0x00000001u, 0xffffffffu, 0xfffe5bfeu, 0x53bda402u, 0x09a1d805u, 0x3339d808u, 0x299d7d48u, 0x73eda753u}};
Fr fr_u32(uint32_t x) { Fr r{}; r.v[0] = x; return r; }
bool fr_is_zero(const Fr& a) { uint32_t o = 0; for (int i = 0; i < 8; i++) o |= a.v[i]; return o == 0; }
bool fr_eq(const Fr& a, const Fr& b) { return memcmp(a.v, b.v, FRB) == 0; }
bool fr_lt(const Fr& a, const Fr& b) {
    for (int i = 7; i >= 0; i--) if (a.v[i] != b.v[i]) return a.v[i] < b.v[i];
    return false;
}
Fr raw_sub(const Fr& a, const Fr& b) {
    Fr r; int64_t br = 0;
    for (int i = 0; i < 8; i++) { int64_t d = (int64_t)a.v[i] - b.v[i] - br; r.v[i] = (uint32_t)d; br = d < 0; }
    return r;
}
Fr fr_add(const Fr& a, const Fr& b) {
    Fr r; uint64_t c = 0;
    for (int i = 0; i < 8; i++) { c += (uint64_t)a.v[i] + b.v[i]; r.v[i] = (uint32_t)c; c >>= 32; }
    return (c || !fr_lt(r, FR_MOD)) ? raw_sub(r, FR_MOD) : r;      // 2p < 2^256: no carry out for reduced operands
}
Fr fr_sub(const Fr& a, const Fr& b) { return fr_lt(a, b) ? raw_sub(FR_MOD, raw_sub(b, a)) : raw_sub(a, b); }
Fr fr_mul(const Fr& a, const Fr& b) {                               // double-and-add: a few hundred calls per proof
    Fr r{};
    for (int i = 255; i >= 0; i--) {
        r = fr_add(r, r);
        if ((b.v[i >> 5] >> (i & 31)) & 1u) r = fr_add(r, a);
    }
    return r;
}
Fr fr_from_i64(int64_t x) {
    Fr r{};
    const uint64_t m = x < 0 ? (uint64_t)(-(x + 1)) + 1 : (uint64_t)x;
    r.v[0] = (uint32_t)m; r.v[1] = (uint32_t)(m >> 32);
    return x < 0 ? raw_sub(FR_MOD, r) : r;
}
// p(u) from p(0), p(1), p(2) (lagrange3, zkllm-src/vrf_common.cuh:130-140)
Fr lagrange3(const Fr& p0, const Fr& p1, const Fr& p2, const Fr& u) {
    const Fr one = fr_u32(1), two = fr_u32(2);
    const Fr inv2 = {{2147483649u, 2147483647u, 2147429887u, 2849952257u, 80800770u, 429714436u, 2496577188u, 972477353u}};
    const Fr um1 = fr_sub(u, one), um2 = fr_sub(u, two);
    const Fr l0 = fr_mul(fr_mul(um1, um2), inv2), l1 = fr_mul(u, fr_sub(two, u)), l2 = fr_mul(fr_mul(u, um1), inv2);
    return fr_add(fr_add(fr_mul(p0, l0), fr_mul(p1, l1)), fr_mul(p2, l2));
}

// ------------------------------------------------------------------ files
std::vector<uint8_t> read_file(const std::string& path) {
    FILE* f = fopen(path.c_str(), "rb");
    if (!f) throw std::runtime_error("cannot open " + path);
    std::vector<uint8_t> b;
    uint8_t buf[1 << 16];
    size_t n;
    while ((n = fread(buf, 1, sizeof buf, f)) > 0) b.insert(b.end(), buf, buf + n);
    fclose(f);
    return b;
}
void write_file(const std::string& path, const std::vector<uint8_t>& b) {
    FILE* f = fopen(path.c_str(), "wb");
    if (!f) throw std::runtime_error("cannot write " + path);
    if (!b.empty() && fwrite(b.data(), 1, b.size(), f) != b.size()) { fclose(f); throw std::runtime_error("short write to " + path); }
    fclose(f);
}
void put(std::vector<uint8_t>& b, const void* p, size_t n) { const uint8_t* q = (const uint8_t*)p; b.insert(b.end(), q, q + n); }
uint32_t clog2(uint32_t n) { uint32_t l = 0; while ((1u << l) < n) l++; return l; }

std::vector<int32_t> load_ints(const std::string& path, size_t expect) {
    std::vector<uint8_t> raw = read_file(path);
    if (raw.size() < expect * 4) throw std::runtime_error("short read / wrong dims: " + path);
    std::vector<int32_t> v(expect);
    memcpy(v.data(), raw.data(), expect * 4);
    return v;
}

// ------------------------------------------------------------------ the library
struct Ctx {
    zkh_ctx* c = nullptr;
    Ctx() {
        const char* d = getenv("ZKH_DEVICE");
        if (zkh_ctx_create(d ? atoi(d) : 0, nullptr, &c) != ZKH_OK) throw std::runtime_error("no CUDA device for libzkh");
    }
    ~Ctx() { if (c) zkh_ctx_destroy(c); }
    void ck(int rc, const char* what) const {
        if (rc != ZKH_OK) throw std::runtime_error(std::string(what) + ": " + zkh_last_error(c));
    }
};
struct Dev {                                                        // device buffer
    Ctx& x; void* p = nullptr; size_t bytes = 0;
    Dev(Ctx& x_, size_t n) : x(x_), bytes(n) { x.ck(zkh_dev_alloc(x.c, n ? n : 16, &p), "device allocation"); }
    Dev(Ctx& x_, const void* host, size_t n) : Dev(x_, n) { x.ck(zkh_upload(x.c, p, host, n), "upload"); }
    Dev(const Dev&) = delete;
    ~Dev() { if (p) zkh_dev_free(x.c, p); }
    std::vector<uint8_t> host() const {
        std::vector<uint8_t> h(bytes);
        x.ck(zkh_download(x.c, h.data(), p, bytes), "download");
        return h;
    }
};

// rows x cols integers, zero-padded to rows_pad x cols_pad scalars (FrTensor(int*) then pad, zkllm-src/fr-tensor.cu:727-736, :809-828)
std::vector<Fr> pad_matrix(const int64_t* v, uint32_t rows, uint32_t cols, uint32_t rp, uint32_t cp) {
    std::vector<Fr> out((size_t)rp * cp, Fr{});
    for (uint32_t r = 0; r < rows; r++)
        for (uint32_t c = 0; c < cols; c++) out[(size_t)r * cp + c] = fr_from_i64(v[(size_t)r * cols + c]);
    return out;
}
std::vector<int64_t> widen(const std::vector<int32_t>& v) { return std::vector<int64_t>(v.begin(), v.end()); }

// Pedersen commitments of the rows of a rows x n scalar matrix
std::vector<uint8_t> commit_rows(Ctx& x, const Dev& gens, const Dev& mat, uint32_t rows, uint32_t n) {
    Dev out(x, (size_t)rows * G1B);
    x.ck(zkh_g1_pedersen_commit(x.c, gens.p, mat.p, rows, n, out.p), "commitment");
    return out.host();
}

// fs::Transcript over the library's host functions, with the reference's helpers (zkllm-src/vrf_common.cuh:219-250)
struct Transcript {
    uint8_t st[32];
    explicit Transcript(const std::string& seed) { zkh_tr_init(st, seed.data(), seed.size()); }
    void absorb(const char* label, const void* p, size_t n) { zkh_tr_absorb(st, label, p, n); }
    void absorb_u32(const char* label, uint32_t v) { absorb(label, &v, 4); }
    void absorb_fr(const char* label, const Fr& v) { absorb(label, v.v, FRB); }
    Fr challenge_fr() {
        for (;;) {
            uint8_t b[32];
            zkh_tr_challenge_bytes(st, b);
            Fr r;
            for (int i = 0; i < 8; i++) r.v[i] = (uint32_t)b[4 * i] | ((uint32_t)b[4 * i + 1] << 8) | ((uint32_t)b[4 * i + 2] << 16) | ((uint32_t)b[4 * i + 3] << 24);
            r.v[7] %= 1944954707u;
            if (!fr_is_zero(r)) return r;
        }
    }
    std::vector<Fr> challenge_vec(uint32_t n) { std::vector<Fr> o(n); for (auto& e : o) e = challenge_fr(); return o; }
};

struct Dims { uint32_t B, IN, OUT, lb, lj, lk, Bp, INp, OUTp; };
Dims dims_of(const char* b, const char* in, const char* out) {
    Dims d;
    d.B = (uint32_t)atoi(b); d.IN = (uint32_t)atoi(in); d.OUT = (uint32_t)atoi(out);
    if (!d.B || d.IN < 2 || !d.OUT) throw std::runtime_error("bad dimensions (B >= 1, IN >= 2, OUT >= 1)");
    d.lb = clog2(d.B); d.lj = clog2(d.IN); d.lk = clog2(d.OUT);
    d.Bp = 1u << d.lb; d.INp = 1u << d.lj; d.OUTp = 1u << d.lk;
    return d;
}
void refuse_flags(int argc, char** argv) {
    for (int i = 1; i < argc; i++)
        if (!strncmp(argv[i], "--", 2)) throw std::invalid_argument(std::string("flag not built in this driver: ") + argv[i]);
}

// partial evaluation of a device tensor viewed as [other][2^logd][window] at u (FrTensor::partial_me)
void partial_me(Ctx& x, const Dev& t, uint64_t other, uint32_t logd, uint64_t window, const std::vector<Fr>& u, Dev& out) {
    if (logd == 0) {                                                // a dimension of one: nothing to fold
        const std::vector<uint8_t> h = t.host();
        x.ck(zkh_upload(x.c, out.p, h.data(), (size_t)other * window * FRB), "copy");
        return;
    }
    x.ck(zkh_fr_partial_me(x.c, t.p, other, logd, window, u.data(), out.p), "partial_me");
}
// the multilinear extension of a 2^la x 2^lb matrix at (ua for the rows, ub for the columns) (FrTensor::multi_dim_me)
Fr eval2(Ctx& x, const Dev& t, uint32_t la, uint32_t lb, const std::vector<Fr>& ua, const std::vector<Fr>& ub) {
    Dev rows(x, ((size_t)1 << la) * FRB);
    partial_me(x, t, (uint64_t)1 << la, lb, 1, ub, rows);
    Fr r;
    if (la == 0) x.ck(zkh_download(x.c, r.v, rows.p, FRB), "download");
    else x.ck(zkh_fr_mle_eval(x.c, rows.p, ua.data(), la, r.v), "mle_eval");
    return r;
}
// one inner-product argument into a file (ipa_prove + write_ipa, zkllm-src/vrf_common.cuh:286-292, :302-336)
void ipa_to_file(Ctx& x, const std::string& path, const Dev& a, const std::vector<Fr>& u_b, const Dev& gens, const uint8_t* Q, uint32_t n,
                 Transcript& tr) {
    const uint32_t rounds = clog2(n);
    Dev b(x, (size_t)n * FRB);
    const Fr one = fr_u32(1);
    if (rounds == 0) x.ck(zkh_upload(x.c, b.p, one.v, FRB), "upload");
    else x.ck(zkh_fr_eq_build(x.c, u_b.data(), rounds, b.p), "eq_build");                       // me_weights(u_b)
    std::vector<uint8_t> L((size_t)rounds * G1B + 1), R((size_t)rounds * G1B + 1);
    Fr af;
    x.ck(zkh_g1_ipa_prove(x.c, a.p, b.p, gens.p, Q, n, tr.st, L.data(), R.data(), af.v), "ipa_prove");
    std::vector<uint8_t> f;
    put(f, &rounds, 4); put(f, L.data(), (size_t)rounds * G1B);
    put(f, &rounds, 4); put(f, R.data(), (size_t)rounds * G1B);
    put(f, af.v, FRB);
    write_file(path, f);
}

int do_commit(int argc, char** argv) {
    refuse_flags(argc, argv);
    if (argc != 7) throw std::invalid_argument("commit <W-int.bin> <IN> <OUT> <gen_out.bin> <com_out.bin>");
    const Dims d = dims_of("1", argv[3], argv[4]);
    const std::vector<int32_t> W = load_ints(argv[2], (size_t)d.IN * d.OUT);
    const std::vector<uint8_t> g = read_file(argv[5]);
    if (g.size() != (size_t)d.OUTp * G1B) throw std::runtime_error("generator sizes don't match padded dims");
    Ctx x;
    const std::vector<Fr> Wp = pad_matrix(widen(W).data(), d.IN, d.OUT, d.INp, d.OUTp);
    Dev gd(x, g.data(), g.size()), wd(x, Wp.data(), Wp.size() * FRB);
    write_file(argv[6], commit_rows(x, gd, wd, d.INp, d.OUTp));
    std::cout << "registered commitment -> " << argv[6] << std::endl;
    return 0;
}

int do_prove(int argc, char** argv) {
    refuse_flags(argc, argv);
    if (argc != 12 && argc != 13) throw std::invalid_argument("prove <obdir> <seed> <X> <W> <B> <IN> <OUT> <gen_in> <gen_out> <q> [Y-out]");
    const std::string obdir = argv[2], seed = argv[3];
    const Dims d = dims_of(argv[6], argv[7], argv[8]);
    const std::vector<int32_t> X = load_ints(argv[4], (size_t)d.B * d.IN), W = load_ints(argv[5], (size_t)d.IN * d.OUT);
    const std::vector<uint8_t> gi = read_file(argv[9]), go = read_file(argv[10]), q = read_file(argv[11]);
    if (gi.size() != (size_t)d.INp * G1B || go.size() != (size_t)d.OUTp * G1B) throw std::runtime_error("generator sizes don't match padded dims");
    if (q.size() < G1B) throw std::runtime_error("q.bin holds no point");
    // Y = X . W in integers (zkFC, zkllm-src/zkfc.cu); pre-rescale products fit 64 bits
    std::vector<int64_t> Y((size_t)d.B * d.OUT, 0);
    for (uint32_t b = 0; b < d.B; b++)
        for (uint32_t j = 0; j < d.IN; j++) {
            const int64_t xv = X[(size_t)b * d.IN + j];
            if (!xv) continue;
            const int32_t* wr = &W[(size_t)j * d.OUT];
            int64_t* yr = &Y[(size_t)b * d.OUT];
            for (uint32_t k = 0; k < d.OUT; k++) yr[k] += xv * wr[k];
        }
    if (argc == 13) {
        std::vector<uint8_t> yb(Y.size() * 8);
        memcpy(yb.data(), Y.data(), yb.size());
        write_file(argv[12], yb);
    }
    Ctx x;
    const std::vector<Fr> Xp = pad_matrix(widen(X).data(), d.B, d.IN, d.Bp, d.INp), Wp = pad_matrix(widen(W).data(), d.IN, d.OUT, d.INp, d.OUTp),
                          Yp = pad_matrix(Y.data(), d.B, d.OUT, d.Bp, d.OUTp);
    Dev gid(x, gi.data(), gi.size()), god(x, go.data(), go.size());
    Dev xd(x, Xp.data(), Xp.size() * FRB), wd(x, Wp.data(), Wp.size() * FRB), yd(x, Yp.data(), Yp.size() * FRB);
    const std::vector<uint8_t> comX = commit_rows(x, gid, xd, d.Bp, d.INp), comW = commit_rows(x, god, wd, d.INp, d.OUTp),
                               comY = commit_rows(x, god, yd, d.Bp, d.OUTp);
    write_file(obdir + "/com_X.bin", comX);
    write_file(obdir + "/com_Y.bin", comY);
    { std::vector<uint8_t> f; const uint32_t dm[3] = {d.B, d.IN, d.OUT}; put(f, dm, 12); write_file(obdir + "/dims.bin", f); }

    Transcript tr(seed);
    tr.absorb_u32("B", d.B); tr.absorb_u32("IN", d.IN); tr.absorb_u32("OUT", d.OUT);
    tr.absorb("com_X", comX.data(), comX.size());
    tr.absorb("com_W", comW.data(), comW.size());
    tr.absorb("com_Y", comY.data(), comY.size());
    const std::vector<Fr> u_batch = tr.challenge_vec(d.lb), u_output = tr.challenge_vec(d.lk);
    const Fr claim = eval2(x, yd, d.lb, d.lk, u_batch, u_output);
    tr.absorb_fr("claim", claim);

    // inner-product sumcheck over the contraction dimension: X folded by u_batch against W folded by u_output
    Dev xr(x, (size_t)d.INp * FRB), wr(x, (size_t)d.INp * FRB);
    partial_me(x, xd, 1, d.lb, d.INp, u_batch, xr);
    partial_me(x, wd, d.INp, d.lk, 1, u_output, wr);
    const uint32_t L = d.lj;
    std::vector<Fr> ev((size_t)3 * L), xs(L);
    Fr fin[2];
    const void* cols[2] = {xr.p, wr.p};
    const char* labels[3] = {"p0", "p1", "p2"};
    x.ck(zkh_fr_sumcheck(x.c, cols, 2, L, labels, tr.st, ev.data(), xs.data(), fin), "sumcheck");
    Fr cur = claim;
    for (uint32_t r = 0; r < L; r++) {
        if (!fr_eq(cur, fr_add(ev[3 * r], ev[3 * r + 1]))) throw std::runtime_error("prover sumcheck round inconsistency (witness bug)");
        cur = lagrange3(ev[3 * r], ev[3 * r + 1], ev[3 * r + 2], xs[r]);
    }
    std::vector<Fr> u_input(L);                                     // round r bound u_input[L - 1 - r]
    for (uint32_t i = 0; i < L; i++) u_input[i] = xs[L - 1 - i];
    const Fr claim_X = fin[0], claim_W = fin[1];
    if (!fr_eq(cur, fr_mul(claim_X, claim_W))) throw std::runtime_error("folded terminals do not multiply to the last claim");
    tr.absorb_fr("claim_X", claim_X); tr.absorb_fr("claim_W", claim_W);
    {
        std::vector<uint8_t> f;
        const uint32_t n = 3 * L;
        put(f, &n, 4); put(f, ev.data(), ev.size() * FRB);
        put(f, claim.v, FRB); put(f, claim_X.v, FRB); put(f, claim_W.v, FRB);
        write_file(obdir + "/sumcheck.bin", f);
    }
    // openings on the same transcript, in the order W, X, Y
    {
        Dev aW(x, (size_t)d.OUTp * FRB);
        partial_me(x, wd, 1, d.lj, d.OUTp, u_input, aW);            // fold the IN_pad rows
        ipa_to_file(x, obdir + "/ipa_W.bin", aW, u_output, god, q.data(), d.OUTp, tr);
    }
    ipa_to_file(x, obdir + "/ipa_X.bin", xr, u_input, gid, q.data(), d.INp, tr);       // X folded by u_batch: the column above
    {
        Dev aY(x, (size_t)d.OUTp * FRB);
        partial_me(x, yd, 1, d.lb, d.OUTp, u_batch, aY);
        ipa_to_file(x, obdir + "/ipa_Y.bin", aY, u_output, god, q.data(), d.OUTp, tr);
    }
    std::cout << "PROVED matmul obligation -> " << obdir << std::endl;
    return 0;
}

struct Ipa { uint32_t rounds = 0; std::vector<uint8_t> L, R; Fr af; };
Ipa read_ipa(const std::string& path) {
    const std::vector<uint8_t> f = read_file(path);
    Ipa p;
    size_t o = 0;
    auto need = [&](size_t n) { if (o + n > f.size()) throw std::runtime_error("read_ipa: truncated " + path); };
    uint32_t nl, nr;
    need(4); memcpy(&nl, &f[o], 4); o += 4;
    if (nl > 32) throw std::runtime_error("read_ipa: round count");
    need((size_t)nl * G1B); p.L.assign(f.begin() + o, f.begin() + o + (size_t)nl * G1B); o += (size_t)nl * G1B;
    need(4); memcpy(&nr, &f[o], 4); o += 4;
    if (nr > 32) throw std::runtime_error("read_ipa: round count");
    need((size_t)nr * G1B); p.R.assign(f.begin() + o, f.begin() + o + (size_t)nr * G1B); o += (size_t)nr * G1B;
    need(FRB); memcpy(p.af.v, &f[o], FRB);
    p.rounds = nl == nr ? nl : 0xffffffffu;
    return p;
}
// one opening of the verifier: fold the row commitments, P0 = C0 + eval Q, then the argument's verifier
bool open_verify(Ctx& x, const std::vector<uint8_t>& com, uint32_t rows, const std::vector<Fr>& u_rows, const Fr& eval, const Dev& gens,
                 uint32_t n, const uint8_t* Q, const std::vector<Fr>& u_b, const Ipa& pf, Transcript& tr) {
    if (pf.rounds != clog2(n) || u_b.size() != pf.rounds) return false;
    if (!fr_lt(pf.af, FR_MOD)) return false;
    Dev cd(x, com.data(), com.size());
    uint8_t pair[2 * G1B];
    Fr none{};
    x.ck(zkh_g1_fold_chain(x.c, cd.p, rows, u_rows.empty() ? &none : u_rows.data(), (uint32_t)u_rows.size(), 0, pair), "fold_chain");
    memcpy(pair + G1B, Q, G1B);
    // C0 + eval Q as the halving sum of (1 C0, eval Q): the reference's h_add(C0, h_mul(Q, eval))
    const Fr sc[2] = {fr_u32(1), eval};
    Dev pd(x, pair, sizeof pair), sd(x, sc, sizeof sc);
    uint8_t P0[G1B];
    x.ck(zkh_g1_msm(x.c, pd.p, sd.p, 2, P0), "statement point");
    int ok = 0;
    x.ck(zkh_g1_ipa_verify(x.c, gens.p, n, Q, P0, u_b.empty() ? &none : u_b.data(), pf.L.data(), pf.R.data(), pf.af.v, tr.st, &ok), "ipa_verify");
    return ok == 1;
}

bool verify(Ctx& x, const std::string& obdir, const std::string& seed, const Dims& d, const std::string& comW_path, const std::vector<uint8_t>& gi,
            const std::vector<uint8_t>& go, const std::vector<uint8_t>& q) {
    if (gi.size() != (size_t)d.INp * G1B || go.size() != (size_t)d.OUTp * G1B) { std::cout << "REJECT: generator sizes don't match dims" << std::endl; return false; }
    {
        const std::vector<uint8_t> f = read_file(obdir + "/dims.bin");
        uint32_t dm[3];
        if (f.size() < 12) return false;
        memcpy(dm, f.data(), 12);
        if (dm[0] != d.B || dm[1] != d.IN || dm[2] != d.OUT) { std::cout << "REJECT: dims.bin mismatch" << std::endl; return false; }
    }
    const std::vector<uint8_t> comX = read_file(obdir + "/com_X.bin"), comW = read_file(comW_path), comY = read_file(obdir + "/com_Y.bin");
    if (comX.size() != (size_t)d.Bp * G1B || comW.size() != (size_t)d.INp * G1B || comY.size() != (size_t)d.Bp * G1B) {
        std::cout << "REJECT: commitment row counts" << std::endl; return false;
    }
    const uint32_t L = d.lj;
    std::vector<Fr> ev((size_t)3 * L);
    Fr claim, claim_X, claim_W;
    {
        const std::vector<uint8_t> f = read_file(obdir + "/sumcheck.bin");
        uint32_t n = 0;
        if (f.size() >= 4) memcpy(&n, f.data(), 4);
        if (f.size() < 4 || n != 3 * L) { std::cout << "REJECT: round count" << std::endl; return false; }
        if (f.size() != 4 + (size_t)(n + 3) * FRB) { std::cout << "REJECT: sumcheck.bin size" << std::endl; return false; }
        memcpy(ev.data(), &f[4], (size_t)n * FRB);
        memcpy(claim.v, &f[4 + (size_t)n * FRB], FRB);
        memcpy(claim_X.v, &f[4 + (size_t)(n + 1) * FRB], FRB);
        memcpy(claim_W.v, &f[4 + (size_t)(n + 2) * FRB], FRB);
    }
    for (const Fr& e : ev) if (!fr_lt(e, FR_MOD)) { std::cout << "REJECT: non-canonical round evaluation" << std::endl; return false; }
    if (!fr_lt(claim, FR_MOD) || !fr_lt(claim_X, FR_MOD) || !fr_lt(claim_W, FR_MOD)) { std::cout << "REJECT: non-canonical claim" << std::endl; return false; }

    Transcript tr(seed);
    tr.absorb_u32("B", d.B); tr.absorb_u32("IN", d.IN); tr.absorb_u32("OUT", d.OUT);
    tr.absorb("com_X", comX.data(), comX.size());
    tr.absorb("com_W", comW.data(), comW.size());
    tr.absorb("com_Y", comY.data(), comY.size());
    const std::vector<Fr> u_batch = tr.challenge_vec(d.lb), u_output = tr.challenge_vec(d.lk);
    tr.absorb_fr("claim", claim);
    Fr cur = claim;
    std::vector<Fr> xs;
    for (uint32_t r = 0; r < L; r++) {
        const Fr &p0 = ev[3 * r], &p1 = ev[3 * r + 1], &p2 = ev[3 * r + 2];
        if (!fr_eq(cur, fr_add(p0, p1))) { std::cout << "REJECT: sumcheck round " << r << " p(0)+p(1) != claim" << std::endl; return false; }
        tr.absorb_fr("p0", p0); tr.absorb_fr("p1", p1); tr.absorb_fr("p2", p2);
        const Fr xr = tr.challenge_fr();
        cur = lagrange3(p0, p1, p2, xr);
        xs.push_back(xr);
    }
    std::vector<Fr> u_input(L);
    for (uint32_t i = 0; i < L; i++) u_input[i] = xs[L - 1 - i];
    if (!fr_eq(cur, fr_mul(claim_X, claim_W))) { std::cout << "REJECT: terminal claim != claim_X * claim_W" << std::endl; return false; }
    tr.absorb_fr("claim_X", claim_X); tr.absorb_fr("claim_W", claim_W);

    Dev gid(x, gi.data(), gi.size()), god(x, go.data(), go.size());
    if (!open_verify(x, comW, d.INp, u_input, claim_W, god, d.OUTp, q.data(), u_output, read_ipa(obdir + "/ipa_W.bin"), tr)) {
        std::cout << "REJECT: IPA opening of claim_W vs registered weight commitment" << std::endl; return false;
    }
    if (!open_verify(x, comX, d.Bp, u_batch, claim_X, gid, d.INp, q.data(), u_input, read_ipa(obdir + "/ipa_X.bin"), tr)) {
        std::cout << "REJECT: IPA opening of claim_X vs com_X" << std::endl; return false;
    }
    if (!open_verify(x, comY, d.Bp, u_batch, claim, god, d.OUTp, q.data(), u_output, read_ipa(obdir + "/ipa_Y.bin"), tr)) {
        std::cout << "REJECT: IPA opening of claim vs com_Y" << std::endl; return false;
    }
    std::cout << "ACCEPT" << std::endl;
    return true;
}

int do_verify(int argc, char** argv) {
    refuse_flags(argc, argv);
    if (argc != 11) throw std::invalid_argument("verify <obdir> <seed> <B> <IN> <OUT> <com_W.bin> <gen_in> <gen_out> <q>");
    const Dims d = dims_of(argv[4], argv[5], argv[6]);
    const std::vector<uint8_t> gi = read_file(argv[8]), go = read_file(argv[9]), q = read_file(argv[10]);
    if (q.size() < G1B) throw std::runtime_error("q.bin holds no point");
    Ctx x;
    return verify(x, argv[2], argv[3], d, argv[7], gi, go, q) ? 0 : 1;
}

int run1(int argc, char** argv);

// prove -> verify on small shapes with generators made here (multiples of the group's generator), then changed proofs
int do_selftest() {
    static const uint32_t GEN[36] = {
        0xfd530c16u, 0x5cb38790u, 0x9976fff5u, 0x7817fc67u, 0x143ba1c1u, 0x154f95c7u, 0xf3d0e747u, 0xf0ae6acdu, 0x21dbf440u,
        0xedce6eccu, 0x9e0bfb75u, 0x12017741u, 0x0ce72271u, 0xbaac93d5u, 0x7918fd8eu, 0x8c22631au, 0x570725ceu, 0xdd595f13u,
        0x50405194u, 0x51ac5829u, 0xad0059c0u, 0x0e1c8c3fu, 0x5008a26au, 0x0bbc3efcu, 0x0002fffdu, 0x76090000u, 0xc40c0002u,
        0xebf4000bu, 0x53c758bau, 0x5f489857u, 0x70525745u, 0x77ce5853u, 0xa256ec6du, 0x5c071a97u, 0xfa80e493u, 0x15f65ec3u};
    if (!fr_eq(fr_mul(fr_u32(2), Fr{{2147483649u, 2147483647u, 2147429887u, 2849952257u, 80800770u, 429714436u, 2496577188u, 972477353u}}), fr_u32(1)))
        throw std::runtime_error("1/2 self-check failed");
    char tmpl[] = "/tmp/zkob_fc_selftest_XXXXXX";
    const char* dir = mkdtemp(tmpl);
    if (!dir) throw std::runtime_error("no temporary directory");
    const std::string D = dir;
    bool all = true;
    const uint32_t cases[3][3] = {{4, 6, 3}, {8, 8, 8}, {16, 12, 5}};
    for (const auto& cs : cases) {
        const uint32_t B = cs[0], IN = cs[1], OUT = cs[2], INp = 1u << clog2(IN), OUTp = 1u << clog2(OUT);
        uint64_t s = 0x9E3779B97F4A7C15ull * (B + 31 * IN + 977 * OUT);
        auto next = [&]() { s = s * 6364136223846793005ull + 1442695040888963407ull; return (uint32_t)(s >> 33); };
        {   // generators and Q: k G for distinct odd k
            Ctx x;
            Dev gd(x, GEN, sizeof GEN);
            std::vector<uint8_t> pts((size_t)(INp + OUTp + 1) * G1B);
            for (uint32_t i = 0; i < INp + OUTp + 1; i++) {
                const Fr k = fr_u32(2 * next() + 1);
                Dev kd(x, k.v, FRB);
                x.ck(zkh_g1_msm(x.c, gd.p, kd.p, 1, &pts[(size_t)i * G1B]), "generator");
            }
            write_file(D + "/gen_in.bin", std::vector<uint8_t>(pts.begin(), pts.begin() + (size_t)INp * G1B));
            write_file(D + "/gen_out.bin", std::vector<uint8_t>(pts.begin() + (size_t)INp * G1B, pts.begin() + (size_t)(INp + OUTp) * G1B));
            write_file(D + "/q.bin", std::vector<uint8_t>(pts.begin() + (size_t)(INp + OUTp) * G1B, pts.end()));
        }
        std::vector<int32_t> X((size_t)B * IN), W((size_t)IN * OUT);
        for (auto& v : X) v = (int32_t)(next() % 2001) - 1000;
        for (auto& v : W) v = (int32_t)(next() % 2001) - 1000;
        std::vector<uint8_t> xb(X.size() * 4), wb(W.size() * 4);
        memcpy(xb.data(), X.data(), xb.size()); memcpy(wb.data(), W.data(), wb.size());
        write_file(D + "/X.i32", xb); write_file(D + "/W.i32", wb);
        const std::string sB = std::to_string(B), sI = std::to_string(IN), sO = std::to_string(OUT);
        const std::string gi = D + "/gen_in.bin", go = D + "/gen_out.bin", q = D + "/q.bin", cw = D + "/com_W.bin", xi = D + "/X.i32", wi = D + "/W.i32";
        auto call = [&](std::vector<std::string> a) {
            std::vector<char*> av;
            for (auto& t : a) av.push_back(const_cast<char*>(t.c_str()));
            return run1((int)av.size(), av.data());
        };
        bool ok = call({"zkob_fc", "commit", wi, sI, sO, go, cw}) == 0;
        ok = ok && call({"zkob_fc", "prove", D, "selftest-seed", xi, wi, sB, sI, sO, gi, go, q}) == 0;
        ok = ok && call({"zkob_fc", "verify", D, "selftest-seed", sB, sI, sO, cw, gi, go, q}) == 0;
        const bool wrong_seed = call({"zkob_fc", "verify", D, "another-seed", sB, sI, sO, cw, gi, go, q}) == 1;
        std::vector<uint8_t> f = read_file(D + "/ipa_Y.bin");
        f[f.size() - 1 - FRB / 2] ^= 1;                         // the final scalar of the last opening
        write_file(D + "/ipa_Y.bin", f);
        const bool bad_ipa = call({"zkob_fc", "verify", D, "selftest-seed", sB, sI, sO, cw, gi, go, q}) == 1;
        std::cout << "case " << B << "x" << IN << "x" << OUT << ": honest " << (ok ? "ACCEPT" : "FAIL") << ", wrong seed " << (wrong_seed ? "REJECT" : "FAIL")
                  << ", changed opening " << (bad_ipa ? "REJECT" : "FAIL") << std::endl;
        all = all && ok && wrong_seed && bad_ipa;
    }
    for (const char* n : {"gen_in.bin", "gen_out.bin", "q.bin", "X.i32", "W.i32", "com_W.bin", "com_X.bin", "com_Y.bin", "dims.bin", "sumcheck.bin",
                          "ipa_W.bin", "ipa_X.bin", "ipa_Y.bin"})
        remove((D + "/" + n).c_str());
    remove(D.c_str());
    std::cout << (all ? "ZKOB-FC SELFTEST: ALL PASS" : "ZKOB-FC SELFTEST: FAIL") << std::endl;
    return all ? 0 : 1;
}

int run1(int argc, char** argv) {
    const std::string mode = argc > 1 ? argv[1] : "";
    try {
        if (mode == "selftest") return do_selftest();
        if (mode == "commit") return do_commit(argc, argv);
        if (mode == "prove") return do_prove(argc, argv);
        if (mode == "verify") return do_verify(argc, argv);
    } catch (const std::invalid_argument& e) {
        std::cerr << "zkob_fc: " << e.what() << std::endl;
        return 2;
    }
    std::cerr << "usage: zkob_fc commit ... | prove ... | verify ... | selftest | serve" << std::endl;
    return 2;
}

// one request per stdin line through the same entry as the one-shot command line, "ZKW-RC <rc>" after each
int serve(char* argv0) {
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

}  // namespace

int main(int argc, char** argv) {
    try {
        if (argc > 1 && std::string(argv[1]) == "serve") return serve(argv[0]);
        return run1(argc, argv);
    } catch (const std::exception& e) {
        std::cerr << "zkob_fc: " << e.what() << std::endl;
        return 3;
    }
}
