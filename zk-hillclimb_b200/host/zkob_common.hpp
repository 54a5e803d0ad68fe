// Host-side glue shared by the driver programs of the first proof stack (zkob_fc, zkob_rescale): a handful of scalars over the
// BLS12-381 scalar field on the host, file helpers, the library context, the reference's transcript helpers
// (zkllm-src/vrf_common.cuh:219-250), and the row-committed openings open_prove / open_verify (zkllm-src/zkob_lookup.cuh:112-138)
// over the C ABI.
#pragma once
#include <array>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <exception>
#include <iostream>
#include <memory>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#include "zkh.h"

namespace zkob {

// stage timer: with ZKOB_TIMING set, lap() prints the milliseconds since the previous lap to stderr
struct Laps {
    const char* who;
    bool on;
    std::chrono::steady_clock::time_point t;
    explicit Laps(const char* w) : who(w), on(getenv("ZKOB_TIMING") != nullptr), t(std::chrono::steady_clock::now()) {}
    void lap(const char* what) {
        if (!on) return;
        const auto n = std::chrono::steady_clock::now();
        fprintf(stderr, "[%s] %-18s %8.2f ms\n", who, what, std::chrono::duration<double, std::milli>(n - t).count());
        t = n;
    }
};


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

// The optional claim-mode block at the end of a command line: --claims <accdir> <obid> [<registered commitment>]
// (zkllm-src/zkob_fc.cu:1213-1236, zkob_rescale.cu:525-534).  Every other flag is refused.
struct ClaimFlags {
    int base_argc;
    std::string accdir, obid, comref;
    bool on() const { return !accdir.empty(); }
};
inline ClaimFlags claim_flags(int argc, char** argv) {
    ClaimFlags f;
    f.base_argc = argc;
    for (int i = 2; i < argc; i++) {
        if (strncmp(argv[i], "--", 2)) continue;
        if (std::string(argv[i]) != "--claims") throw std::invalid_argument(std::string("flag not built in this driver: ") + argv[i]);
        f.base_argc = i;
        if (i + 1 < argc) f.accdir = argv[i + 1];
        if (i + 2 < argc) f.obid = argv[i + 2];
        if (i + 3 < argc) f.comref = argv[i + 3];
        for (int j = i + 1; j < argc; j++)
            if (!strncmp(argv[j], "--", 2)) throw std::invalid_argument(std::string("flag not built in this driver: ") + argv[j]);
        if (f.accdir.empty() || f.obid.empty()) throw std::invalid_argument("--claims needs <accdir> <obid>");
        break;
    }
    return f;
}

// ------------------------------------------------------------------ the claim accumulator's files (zkllm-src/zkob_claims.cuh:76-270)
// An opening claim: the tensor committed row-wise in the file `comref` (n_rows rows over `domain` generators) evaluates to
// `eval` at `point` (column bits first).  claims.bin = "ZKCL", version 1, count, then per claim: id, comref (length-prefixed),
// domain, n_rows, point (count-prefixed), tag 0, eval.  The claim-mode drivers append to it instead of opening inline; a
// separate batch program discharges the list.
struct Claim {
    std::string id, comref;
    uint32_t domain = 0, n_rows = 0;
    std::vector<Fr> point;
    Fr eval{};
};
inline void put_u32(std::vector<uint8_t>& b, uint32_t v) { for (int i = 0; i < 4; i++) b.push_back((uint8_t)(v >> (8 * i))); }
inline bool file_exists(const std::string& path) { FILE* f = fopen(path.c_str(), "rb"); if (f) fclose(f); return f != nullptr; }
// append one record to a file of the form magic, version 1, count, records
inline void append_record(const std::string& path, const char magic[4], const std::vector<uint8_t>& rec) {
    std::vector<uint8_t> b;
    if (file_exists(path)) {
        b = read_file(path);
        if (b.size() < 12 || memcmp(b.data(), magic, 4)) throw std::runtime_error(path + ": bad magic");
        uint32_t ver, n;
        memcpy(&ver, &b[4], 4); memcpy(&n, &b[8], 4);
        if (ver != 1) throw std::runtime_error(path + ": bad version");
        n++;
        memcpy(&b[8], &n, 4);
    } else {
        put(b, magic, 4); put_u32(b, 1); put_u32(b, 1);
    }
    put(b, rec.data(), rec.size());
    write_file(path, b);
}
// the canonical bytes of one claim: the record of claims.bin and what the batch transcript absorbs (claim_blob)
inline std::vector<uint8_t> claim_blob(const Claim& c) {
    std::vector<uint8_t> r;
    put_u32(r, (uint32_t)c.id.size()); put(r, c.id.data(), c.id.size());
    put_u32(r, (uint32_t)c.comref.size()); put(r, c.comref.data(), c.comref.size());
    put_u32(r, c.domain); put_u32(r, c.n_rows);
    put_u32(r, (uint32_t)c.point.size()); put(r, c.point.data(), c.point.size() * FRB);
    r.push_back(0);                                                 // the evaluation is given in the clear
    put(r, c.eval.v, FRB);
    return r;
}
inline void claim_emit(const std::string& accdir, const Claim& c) { append_record(accdir + "/claims.bin", "ZKCL", claim_blob(c)); }
// bounds-checked reader of the accumulator's files
struct Reader {
    const std::vector<uint8_t>& b;
    size_t off = 0;
    explicit Reader(const std::vector<uint8_t>& bb) : b(bb) {}
    void bytes(void* p, size_t n) {
        if (off + n > b.size()) throw std::runtime_error("accumulator file truncated");
        memcpy(p, b.data() + off, n);
        off += n;
    }
    uint32_t u32() { uint32_t v; bytes(&v, 4); return v; }
    std::string str(uint32_t n) {
        if (off + n > b.size()) throw std::runtime_error("accumulator file truncated");
        std::string s((const char*)b.data() + off, n);
        off += n;
        return s;
    }
};
// claims.bin -> claims (claims_parse, zkllm-src/zkob_claims.cuh:165-192); committed evaluations are not accepted here
inline std::vector<Claim> claims_load(const std::string& path) {
    const std::vector<uint8_t> bytes = read_file(path);
    Reader r(bytes);
    char magic[4];
    r.bytes(magic, 4);
    if (memcmp(magic, "ZKCL", 4)) throw std::runtime_error("claims: bad magic");
    if (r.u32() != 1) throw std::runtime_error("claims: bad version");
    std::vector<Claim> cs(r.u32());
    for (Claim& c : cs) {
        c.id = r.str(r.u32());
        c.comref = r.str(r.u32());
        c.domain = r.u32();
        c.n_rows = r.u32();
        const uint32_t np = r.u32();
        if (np > 64) throw std::runtime_error("claims: point too long");
        c.point.resize(np);
        r.bytes(c.point.data(), (size_t)np * FRB);
        uint8_t tag;
        r.bytes(&tag, 1);
        if (tag != 0) throw std::invalid_argument("claims: committed evaluations are not built in this program (claim " + c.id + ")");
        r.bytes(c.eval.v, FRB);
    }
    if (r.off != bytes.size()) throw std::runtime_error("claims: trailing bytes");
    return cs;
}
inline std::vector<uint8_t> claims_serialize(const std::vector<Claim>& cs) {
    std::vector<uint8_t> b;
    put(b, "ZKCL", 4); put_u32(b, 1); put_u32(b, (uint32_t)cs.size());
    for (const Claim& c : cs) { const std::vector<uint8_t> r = claim_blob(c); put(b, r.data(), r.size()); }
    return b;
}
struct DrvState { std::string id; uint8_t state[32]; };
inline std::vector<DrvState> drvstates_load(const std::string& path) {
    const std::vector<uint8_t> bytes = read_file(path);
    Reader r(bytes);
    char magic[4];
    r.bytes(magic, 4);
    if (memcmp(magic, "ZKDS", 4)) throw std::runtime_error("drvstates: bad magic");
    if (r.u32() != 1) throw std::runtime_error("drvstates: bad version");
    std::vector<DrvState> ds(r.u32());
    for (DrvState& d : ds) { d.id = r.str(r.u32()); r.bytes(d.state, 32); }
    return ds;
}
// 1 + 2uv - u - v: the equality polynomial on one variable (my_eq / bo_eq1)
inline Fr eq1(const Fr& u, const Fr& v) {
    const Fr uv = fr_mul(u, v);
    return fr_add(fr_sub(fr_add(uv, uv), fr_add(u, v)), fr_u32(1));
}
// the prover's pointer from a commitment file to the witness tensor behind it: one line per distinct tensor
inline void witref_emit(const std::string& accdir, const std::string& comref, const std::string& witpath) {
    const std::string path = accdir + "/witrefs.txt";
    if (file_exists(path)) {
        const std::vector<uint8_t> b = read_file(path);
        const std::string all((const char*)b.data(), b.size());
        if (all.find(comref + "\t") != std::string::npos) return;
    }
    FILE* f = fopen(path.c_str(), "ab");
    if (!f) throw std::runtime_error("cannot write " + path);
    fprintf(f, "%s\t%s\n", comref.c_str(), witpath.c_str());
    fclose(f);
}
// the driver's final transcript state, which the batch absorbs
inline void drvstate_emit(const std::string& accdir, const std::string& obid, const uint8_t state[32]) {
    std::vector<uint8_t> r;
    put_u32(r, (uint32_t)obid.size()); put(r, obid.data(), obid.size());
    put(r, state, 32);
    append_record(accdir + "/drvstates.bin", "ZKDS", r);
}
inline Claim make_claim(const std::string& obid, const char* tensor, const std::string& comref, uint32_t domain, uint32_t n_rows,
                        const std::vector<Fr>& u_col, const std::vector<Fr>& u_row, const Fr& eval) {
    Claim c;
    c.id = obid + ":" + tensor;
    c.comref = comref;
    c.domain = domain; c.n_rows = n_rows;
    c.point = u_col;
    c.point.insert(c.point.end(), u_row.begin(), u_row.end());
    c.eval = eval;
    return c;
}
// a padded witness tensor as the raw scalars the batch program reads (FrTensor::save)
inline void save_scalars(const std::string& path, const std::vector<Fr>& t) {
    std::vector<uint8_t> b(t.size() * FRB);
    memcpy(b.data(), t.data(), b.size());
    write_file(path, b);
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
    Laps laps("open_verify");
    Dev cd(x, com.data(), com.size());
    uint8_t pair[2 * G1B];
    Fr none{};
    // The folded commitment as a group element: sum_k eq(u_rows, k) com[k], one multi-scalar product instead of log2(rows)
    // dependent fold levels (the verdict depends on the point, not on its Jacobian representative; zkllm-src/zkob_claims.cuh:490-570
    // folds its batches the same way)
    if (rows > 1 && (rows & (rows - 1)) == 0 && u_rows.size() == clog2(rows)) {
        Dev wd(x, (size_t)rows * FRB);
        x.ck(zkh_fr_eq_build(x.c, u_rows.data(), (uint32_t)u_rows.size(), wd.p), "row weights");
        x.ck(zkh_g1_msm(x.c, cd.p, wd.p, rows, pair), "folded commitment");
    } else {
        x.ck(zkh_g1_fold_chain(x.c, cd.p, rows, u_rows.empty() ? &none : u_rows.data(), (uint32_t)u_rows.size(), 0, pair), "fold_chain");
    }
    laps.lap("fold");
    memcpy(pair + G1B, Q, G1B);
    // C0 + eval Q as the halving sum of (1 C0, eval Q): the reference's h_add(C0, h_mul(Q, eval))
    const Fr sc[2] = {fr_u32(1), eval};
    Dev pd(x, pair, sizeof pair), sd(x, sc, sizeof sc);
    uint8_t P0[G1B];
    x.ck(zkh_g1_msm(x.c, pd.p, sd.p, 2, P0), "statement point");
    laps.lap("statement");
    int ok = 0;
    x.ck(zkh_g1_ipa_verify(x.c, gens.p, n, Q, P0, u_b.empty() ? &none : u_b.data(), pf.L.data(), pf.R.data(), pf.af.v, tr.st, &ok), "ipa_verify");
    laps.lap("ipa_verify");
    return ok == 1;
}

// one request per stdin line through the same entry as the one-shot command line, "ZKW-RC <rc>" after each
inline int serve_loop(char* argv0, int (*run1)(int, char**)) {
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

// x^-1 by Fermat (a few per proof)
inline Fr fr_inv(const Fr& a) {
    const Fr e = raw_sub(FR_MOD, fr_u32(2));
    Fr r = fr_u32(1);
    for (int i = 255; i >= 0; i--) {
        r = fr_mul(r, r);
        if ((e.v[i >> 5] >> (i & 31)) & 1u) r = fr_mul(r, a);
    }
    return r;
}

// p(v) from p(0..3) (lagrange4, zkllm-src/zkob_lookup.cuh:62-73)
Fr lagrange4(const std::array<Fr, 4>& p, const Fr& v, const Fr& inv6, const Fr& inv2) {
    const Fr zero{}, vm1 = fr_sub(v, fr_u32(1)), vm2 = fr_sub(v, fr_u32(2)), vm3 = fr_sub(v, fr_u32(3));
    const Fr l0 = fr_sub(zero, fr_mul(fr_mul(fr_mul(vm1, vm2), vm3), inv6));
    const Fr l1 = fr_mul(fr_mul(fr_mul(v, vm2), vm3), inv2);
    const Fr l2 = fr_sub(zero, fr_mul(fr_mul(fr_mul(v, vm1), vm3), inv2));
    const Fr l3 = fr_mul(fr_mul(fr_mul(v, vm1), vm2), inv6);
    return fr_add(fr_add(fr_add(fr_mul(p[0], l0), fr_mul(p[1], l1)), fr_mul(p[2], l2)), fr_mul(p[3], l3));
}

// p(v) from p(0..4) (lagrange5, zkllm-src/zkob_lookup.cuh:356-375)
Fr lagrange5(const std::array<Fr, 5>& p, const Fr& v, const Fr& inv24, const Fr& inv6, const Fr& inv4) {
    const Fr m1 = fr_sub(v, fr_u32(1)), m2 = fr_sub(v, fr_u32(2)), m3 = fr_sub(v, fr_u32(3)), m4 = fr_sub(v, fr_u32(4)), zero = fr_u32(0);
    auto mul4 = [](const Fr& a, const Fr& b, const Fr& c, const Fr& d) { return fr_mul(fr_mul(a, b), fr_mul(c, d)); };
    const Fr l0 = fr_mul(mul4(m1, m2, m3, m4), inv24), l1 = fr_sub(zero, fr_mul(mul4(v, m2, m3, m4), inv6)), l2 = fr_mul(mul4(v, m1, m3, m4), inv4),
             l3 = fr_sub(zero, fr_mul(mul4(v, m1, m2, m4), inv6)), l4 = fr_mul(mul4(v, m1, m2, m3), inv24);
    Fr acc = fr_mul(p[0], l0);
    acc = fr_add(acc, fr_mul(p[1], l1)); acc = fr_add(acc, fr_mul(p[2], l2)); acc = fr_add(acc, fr_mul(p[3], l3)); acc = fr_add(acc, fr_mul(p[4], l4));
    return acc;
}

// ------------------------------------------------------------------ helpers shared by the structural drivers
// the verifier's verdict line
bool rj(const std::string& msg) { std::cout << "REJECT: " << msg << std::endl; return false; }
// signed integers as field elements (the FrTensor integer constructors)
std::vector<Fr> lift(const std::vector<int64_t>& v) {
    std::vector<Fr> o(v.size());
    for (size_t i = 0; i < v.size(); i++) o[i] = fr_from_i64(v[i]);
    return o;
}
// a Hadamard proof file: claim, count, 4 evaluations per round, the two terminals (write_hp / read_hp, zkllm-src/zkob_lookup.cuh:262-289)
void write_hp(const std::string& path, const Fr& claim, const std::vector<Fr>& hev, const Fr& S_f2, const Fr& U_f2) {
    std::vector<uint8_t> f;
    const uint32_t n = (uint32_t)hev.size();
    put(f, claim.v, FRB); put(f, &n, 4); put(f, hev.data(), hev.size() * FRB); put(f, S_f2.v, FRB); put(f, U_f2.v, FRB);
    write_file(path, f);
}
struct Hp { Fr claim, S_f2, U_f2; std::vector<Fr> ev; };
// false on a wrong size, a wrong count or a non-canonical scalar
bool read_hp(const std::string& path, uint32_t want, Hp& p) {
    const std::vector<uint8_t> f = read_file(path);
    if (f.size() != FRB + 4 + (size_t)want * FRB + 2 * FRB) return false;
    uint32_t n;
    memcpy(p.claim.v, &f[0], FRB);
    memcpy(&n, &f[FRB], 4);
    if (n != want) return false;
    p.ev.resize(n);
    memcpy(p.ev.data(), &f[FRB + 4], (size_t)n * FRB);
    memcpy(p.S_f2.v, &f[FRB + 4 + (size_t)n * FRB], FRB);
    memcpy(p.U_f2.v, &f[FRB + 4 + (size_t)(n + 1) * FRB], FRB);
    for (const Fr& e : p.ev) if (!fr_lt(e, FR_MOD)) return false;
    return fr_lt(p.claim, FR_MOD) && fr_lt(p.S_f2, FR_MOD) && fr_lt(p.U_f2, FR_MOD);
}
// a public weight tensor folded over the round challenges, in place (fold_public of the drivers)
Fr fold_public(Ctx& x, Dev& w, uint64_t n, const std::vector<Fr>& ws) {
    for (const Fr& c : ws) { x.ck(zkh_fr_fold(x.c, w.p, n / 2, c.v, w.p), "fold weights"); n /= 2; }
    Fr out;
    x.ck(zkh_download(x.c, out.v, w.p, FRB), "download");
    return out;
}

// a flat tensor of rows x G scalars committed row-wise, opened at u_pt = (column bits, then row bits) (open_prove)
void open_prove(Ctx& x, const Dev& t, uint32_t rows, uint32_t G, const Dev& gens, const uint8_t* Q, const std::vector<Fr>& u_pt, const std::string& path,
                Transcript& tr) {
    const uint32_t logG = clog2(G);
    const std::vector<Fr> u_col(u_pt.begin(), u_pt.begin() + logG), u_row(u_pt.begin() + logG, u_pt.end());
    if ((1u << u_row.size()) != rows) throw std::runtime_error("open_prove: point does not match the tensor");
    Dev a(x, (size_t)G * FRB);
    partial_me(x, t, 1, (uint32_t)u_row.size(), G, u_row, a);
    ipa_to_file(x, path, a, u_col, gens, Q, G, tr);
}
bool open_check(Ctx& x, const std::vector<uint8_t>& com, uint32_t G, const Dev& gens, const uint8_t* Q, const std::vector<Fr>& u_pt, const Fr& eval,
                const std::string& path, Transcript& tr) {
    const uint32_t logG = clog2(G);
    if (u_pt.size() < logG) return false;
    const uint32_t rows = (uint32_t)(com.size() / G1B);
    if (rows != (1u << (u_pt.size() - logG))) return false;
    const std::vector<Fr> u_col(u_pt.begin(), u_pt.begin() + logG), u_row(u_pt.begin() + logG, u_pt.end());
    return open_verify(x, com, rows, u_row, eval, gens, G, Q, u_col, read_ipa(path), tr);
}

// The verifier's side of the logUp lookup sumcheck (zkllm-src/zkob_rescale.cu:256-313, zkob_glu.cu:341-394): the round checks with
// the anchor alpha + alpha^2 recomputed, B_f and T_f from the PUBLIC table (T_dev, 2^logN scalars, consumed) folded with the
// phase-2 challenges in round order, and the terminal identity.  Prints the reference's REJECT lines (tag names the lookup in them).
// ws: the round challenges.
inline bool lookup_verify(Ctx& x, Transcript& tr, const std::vector<Fr>& ev, const Fr& A_f, const Fr& S_f, const Fr& m_f, const Fr& alpha,
                          const Fr& beta, const std::vector<Fr>& u, Dev& T_dev, uint32_t logD, uint32_t logN, std::vector<Fr>& ws, Laps& laps,
                          const char* tag = "lookup") {
    const uint32_t n1 = logD - logN, N = 1u << logN;
    const Fr inv2 = fr_inv(fr_u32(2)), inv6 = fr_inv(fr_u32(6));
    Fr alpha_acc = alpha, alphasq_acc = fr_mul(alpha, alpha), cur = fr_add(alpha, alphasq_acc);
    ws.clear();
    for (uint32_t k = 0; k < logD; k++) {
        const std::array<Fr, 4> e = {ev[4 * k], ev[4 * k + 1], ev[4 * k + 2], ev[4 * k + 3]};
        if (!fr_eq(cur, fr_add(e[0], e[1]))) { std::cout << "REJECT: " << tag << " round " << k << " p(0)+p(1) != claim" << std::endl; return false; }
        tr.absorb_fr("p0", e[0]); tr.absorb_fr("p1", e[1]); tr.absorb_fr("p2", e[2]); tr.absorb_fr("p3", e[3]);
        const Fr w = tr.challenge_fr();
        ws.push_back(w);
        cur = lagrange4(e, w, inv6, inv2);
        const Fr eqv = eq1(u[logD - 1 - k], w);
        alpha_acc = fr_mul(alpha_acc, eqv);
        if (k >= n1) alphasq_acc = fr_mul(alphasq_acc, eqv);
    }
    laps.lap("rounds");
    Fr B_f, T_f;
    {
        Dev bd(x, (size_t)N * FRB);
        x.ck(zkh_fr_inv_add(x.c, T_dev.p, N, beta.v, bd.p), "B = 1 / (T + beta)");
        for (uint32_t k = 0, sz = N; k < logN; k++, sz >>= 1) {         // each fold binds the current top bit, in place
            x.ck(zkh_fr_fold(x.c, bd.p, sz / 2, ws[n1 + k].v, bd.p), "fold B");
            x.ck(zkh_fr_fold(x.c, T_dev.p, sz / 2, ws[n1 + k].v, T_dev.p), "fold T");
        }
        x.ck(zkh_download(x.c, B_f.v, bd.p, FRB), "download");
        x.ck(zkh_download(x.c, T_f.v, T_dev.p, FRB), "download");
    }
    laps.lap("table_fold");
    const Fr inv_ratio = fr_mul(fr_u32(N), fr_inv(fr_u32(1u << logD)));
    const Fr t1 = fr_mul(alpha_acc, fr_mul(A_f, fr_add(S_f, beta)));
    const Fr t2 = fr_mul(inv_ratio, fr_mul(alphasq_acc, fr_mul(B_f, fr_add(T_f, beta))));
    const Fr t4 = fr_mul(inv_ratio, fr_mul(m_f, B_f));
    if (!fr_eq(cur, fr_sub(fr_add(fr_add(t1, t2), A_f), t4))) { std::cout << "REJECT: " << tag << " terminal identity" << std::endl; return false; }
    laps.lap("terminal");
    return true;
}

}  // namespace zkob
