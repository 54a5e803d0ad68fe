// Driver for the rescaling obligation of the reference's first proof stack: X = sf * Xr + rem with rem range-checked in
// [-sf/2, sf/2) by the logUp lookup against the public table, with the command line, the files and the exit codes of the
// reference's zkob_rescale (zkllm-src/zkob_rescale.cu:1-57, :70-211 prove, :213-370 verify).
//
//   zkob_rescale prove  <obdir> <seed> <X-int64.bin> <B> <C> <LOG_SF> <gen.bin> <q.bin> [Xr-int-out.bin]
//   zkob_rescale verify <obdir> <seed> <B> <C> <LOG_SF> <gen.bin> <q.bin>
//   zkob_rescale selftest
//   zkob_rescale serve
//
// Files in <obdir> (byte for byte the reference's): dims.bin, com_X.bin, com_Xr.bin, com_rem.bin, com_m.bin, com_A.bin,
// lookup.bin, ipa_A.bin, ipa_rem.bin, ipa_m.bin.  Exit 0 = success / ACCEPT, 1 = REJECT, anything else = failure; `serve`
// prints ZKW-READY and answers "ZKW-RC <rc>" per request line.  With --claims <accdir> <obid> (zkob_rescale.cu:47-57) prove
// appends its three lookup-terminal claims, the witness tensors and its final transcript state to the accumulator directory
// instead of opening inline, and verify recomputes the claims into the verifier's accumulator and answers "ACCEPT-conditional".
//
// Transcript schedule (zkob_rescale.cu:19-28): B, C, LOG_SF, com_X, com_Xr, com_rem, com_m -> beta; A = 1 / (rem + beta),
// com_A -> alpha, u; per round p(0..3) -> w_r; A_f, S_f, m_f; the three openings at the reversed round challenges.
#include "zkob_common.hpp"

using namespace zkob;

namespace {

struct Lay { uint32_t B, C, log_sf, sf, Bp, Cp, D, N, logD, logN, n1, logG; };
Lay lay_of(const char* b, const char* c, const char* l) {
    Lay y;
    y.B = (uint32_t)atoi(b); y.C = (uint32_t)atoi(c); y.log_sf = (uint32_t)atoi(l);
    if (!y.B || !y.C || y.log_sf < 1 || y.log_sf > 24) throw std::runtime_error("bad dimensions (B, C >= 1, 1 <= LOG_SF <= 24)");
    y.sf = 1u << y.log_sf;
    y.Bp = 1u << clog2(y.B); y.Cp = 1u << clog2(y.C);
    y.D = y.Bp * y.Cp; y.N = y.sf;
    y.logD = clog2(y.D); y.logN = y.log_sf; y.logG = clog2(y.Cp);
    y.n1 = y.logD >= y.logN ? y.logD - y.logN : 0;
    return y;
}
bool layout_ok(const Lay& y) { return y.Cp <= y.N && y.N <= y.D && y.D % y.N == 0; }

// the public table tLookupRange(-sf/2, sf): table[i] = i - sf/2 (zkllm-src/tlookup.cu:384-391)
std::vector<Fr> range_table(const Lay& y) {
    std::vector<Fr> t(y.N);
    for (uint32_t i = 0; i < y.N; i++) t[i] = fr_from_i64((int64_t)i - (int64_t)(y.sf >> 1));
    return t;
}
int do_prove(int argc, char** argv) {
    const ClaimFlags cf = claim_flags(argc, argv);
    argc = cf.base_argc;
    if (argc != 10 && argc != 11) throw std::invalid_argument("prove <obdir> <seed> <X-int64.bin> <B> <C> <LOG_SF> <gen.bin> <q.bin> [Xr-out]");
    const std::string obdir = argv[2], seed = argv[3];
    const Lay y = lay_of(argv[5], argv[6], argv[7]);
    const std::vector<uint8_t> g = read_file(argv[8]), q = read_file(argv[9]);
    if (g.size() != (size_t)y.Cp * G1B) throw std::runtime_error("generator size != C_pad");
    if (q.size() < G1B) throw std::runtime_error("q.bin holds no point");
    if (!layout_ok(y)) throw std::runtime_error("layout needs C_pad <= N <= D, N | D");
    std::vector<int64_t> X((size_t)y.B * y.C);
    {
        const std::vector<uint8_t> raw = read_file(argv[4]);
        if (raw.size() < X.size() * 8) throw std::runtime_error(std::string("short read / wrong dims: ") + argv[4]);
        memcpy(X.data(), raw.data(), X.size() * 8);
    }
    // rescaling_kernel (zkllm-src/rescaling.cu:8-21): rem in [-sf/2, sf/2), X = sf * Xr + rem
    std::vector<int64_t> Xr(X.size()), rem(X.size());
    const int64_t sf = y.sf, hsf = sf >> 1;
    for (size_t i = 0; i < X.size(); i++) {
        const int64_t t = (X[i] + hsf) % sf;
        rem[i] = (t < 0 ? t + sf : t) - hsf;
        Xr[i] = (X[i] - rem[i]) / sf;
    }
    if (argc == 11) {
        std::vector<int32_t> o(Xr.begin(), Xr.end());
        std::vector<uint8_t> b(o.size() * 4);
        memcpy(b.data(), o.data(), b.size());
        write_file(argv[10], b);
    }
    // multiplicities over the padded witness (the padding's zeros count too)
    std::vector<int64_t> cnt(y.N, 0);
    for (size_t i = 0; i < rem.size(); i++) cnt[(size_t)(rem[i] + hsf)]++;
    cnt[(size_t)hsf] += (int64_t)y.D - (int64_t)rem.size();

    Laps laps("rescale_prove");
    Ctx x;
    laps.lap("context");
    const std::vector<Fr> Xp = pad_matrix(X.data(), y.B, y.C, y.Bp, y.Cp), Xrp = pad_matrix(Xr.data(), y.B, y.C, y.Bp, y.Cp),
                          Rp = pad_matrix(rem.data(), y.B, y.C, y.Bp, y.Cp), Mp = pad_matrix(cnt.data(), y.N / y.Cp, y.Cp, y.N / y.Cp, y.Cp),
                          Tp = range_table(y);
    Dev gd(x, g.data(), g.size());
    Dev xd(x, Xp.data(), Xp.size() * FRB), xrd(x, Xrp.data(), Xrp.size() * FRB), rd(x, Rp.data(), Rp.size() * FRB), md(x, Mp.data(), Mp.size() * FRB),
        td(x, Tp.data(), Tp.size() * FRB);
    const std::vector<uint8_t> comX = commit_rows(x, gd, xd, y.Bp, y.Cp), comXr = commit_rows(x, gd, xrd, y.Bp, y.Cp),
                               comR = commit_rows(x, gd, rd, y.Bp, y.Cp), comM = commit_rows(x, gd, md, y.N / y.Cp, y.Cp);
    laps.lap("commitments");
    write_file(obdir + "/com_X.bin", comX);
    write_file(obdir + "/com_Xr.bin", comXr);
    write_file(obdir + "/com_rem.bin", comR);
    write_file(obdir + "/com_m.bin", comM);
    { std::vector<uint8_t> f; const uint32_t dm[3] = {y.B, y.C, y.log_sf}; put(f, dm, 12); write_file(obdir + "/dims.bin", f); }

    Transcript tr(seed);
    tr.absorb_u32("B", y.B); tr.absorb_u32("C", y.C); tr.absorb_u32("LOG_SF", y.log_sf);
    tr.absorb("com_X", comX.data(), comX.size());
    tr.absorb("com_Xr", comXr.data(), comXr.size());
    tr.absorb("com_rem", comR.data(), comR.size());
    tr.absorb("com_m", comM.data(), comM.size());
    const Fr beta = tr.challenge_fr();
    Dev ad(x, (size_t)y.D * FRB), bd(x, (size_t)y.N * FRB);
    x.ck(zkh_fr_inv_add(x.c, rd.p, y.D, beta.v, ad.p), "A = 1 / (rem + beta)");
    const std::vector<uint8_t> comA = commit_rows(x, gd, ad, y.Bp, y.Cp);
    write_file(obdir + "/com_A.bin", comA);
    tr.absorb("com_A", comA.data(), comA.size());
    const Fr alpha = tr.challenge_fr();
    const std::vector<Fr> u = tr.challenge_vec(y.logD);
    x.ck(zkh_fr_inv_add(x.c, td.p, y.N, beta.v, bd.p), "B = 1 / (T + beta)");
    Fr bm;
    x.ck(zkh_fr_dot(x.c, bd.p, md.p, y.N, bm.v), "sum B m");
    const Fr alpha_sq = fr_mul(alpha, alpha), Cc = fr_sub(alpha_sq, bm);
    std::vector<Fr> ev((size_t)4 * y.logD), ws(y.logD);
    Fr term[5];                                                     // A_f, S_f, B_f, T_f, m_f
    x.ck(zkh_fr_lookup_sumcheck(x.c, ad.p, rd.p, bd.p, td.p, md.p, y.logD, y.logN, alpha.v, beta.v, Cc.v, u.data(), tr.st, ev.data(), ws.data(), term),
         "lookup sumcheck");
    {
        std::vector<uint8_t> f;
        const uint32_t n = 4 * y.logD;
        put(f, &n, 4); put(f, ev.data(), ev.size() * FRB);
        put(f, term[0].v, FRB); put(f, term[1].v, FRB); put(f, term[4].v, FRB);
        write_file(obdir + "/lookup.bin", f);
    }
    tr.absorb_fr("A_f", term[0]); tr.absorb_fr("S_f", term[1]); tr.absorb_fr("m_f", term[4]);
    laps.lap("lookup");
    const std::vector<Fr> u_pt(ws.rbegin(), ws.rend()), u_m(ws.rbegin(), ws.rend() - y.n1);
    if (cf.on()) {
        // claim mode (zkob_rescale.cu:179-203): the three lookup terminals as claims (order A, rem, m), witnesses, final state
        const std::string witA = cf.accdir + "/wit_" + cf.obid + "_A.fr", witR = cf.accdir + "/wit_" + cf.obid + "_rem.fr",
                          witM = cf.accdir + "/wit_" + cf.obid + "_m.fr";
        write_file(witA, ad.host());
        save_scalars(witR, Rp); save_scalars(witM, Mp);
        const std::vector<Fr> none;
        claim_emit(cf.accdir, make_claim(cf.obid, "A", obdir + "/com_A.bin", y.Cp, y.Bp, u_pt, none, term[0]));
        witref_emit(cf.accdir, obdir + "/com_A.bin", witA);
        claim_emit(cf.accdir, make_claim(cf.obid, "rem", obdir + "/com_rem.bin", y.Cp, y.Bp, u_pt, none, term[1]));
        witref_emit(cf.accdir, obdir + "/com_rem.bin", witR);
        claim_emit(cf.accdir, make_claim(cf.obid, "m", obdir + "/com_m.bin", y.Cp, y.N / y.Cp, u_m, none, term[4]));
        witref_emit(cf.accdir, obdir + "/com_m.bin", witM);
        drvstate_emit(cf.accdir, cf.obid, tr.st);
        std::cout << "PROVED rescaling obligation (claim mode, 3 claims emitted) -> " << obdir << std::endl;
        return 0;
    }
    open_prove(x, ad, y.Bp, y.Cp, gd, q.data(), u_pt, obdir + "/ipa_A.bin", tr);
    open_prove(x, rd, y.Bp, y.Cp, gd, q.data(), u_pt, obdir + "/ipa_rem.bin", tr);
    open_prove(x, md, y.N / y.Cp, y.Cp, gd, q.data(), u_m, obdir + "/ipa_m.bin", tr);
    laps.lap("openings");
    std::cout << "PROVED rescaling obligation -> " << obdir << std::endl;
    return 0;
}

bool verify(Ctx& x, const std::string& obdir, const std::string& seed, const Lay& y, const std::vector<uint8_t>& g, const std::vector<uint8_t>& q,
            const ClaimFlags& cf) {
    if (g.size() != (size_t)y.Cp * G1B || !layout_ok(y)) { std::cout << "REJECT: bad layout params" << std::endl; return false; }
    {
        const std::vector<uint8_t> f = read_file(obdir + "/dims.bin");
        uint32_t dm[3];
        if (f.size() < 12) return false;
        memcpy(dm, f.data(), 12);
        if (dm[0] != y.B || dm[1] != y.C || dm[2] != y.log_sf) { std::cout << "REJECT: dims.bin mismatch" << std::endl; return false; }
    }
    const std::vector<uint8_t> comX = read_file(obdir + "/com_X.bin"), comXr = read_file(obdir + "/com_Xr.bin"), comR = read_file(obdir + "/com_rem.bin"),
                               comM = read_file(obdir + "/com_m.bin"), comA = read_file(obdir + "/com_A.bin");
    const size_t rowsB = (size_t)y.Bp * G1B;
    if (comX.size() != rowsB || comXr.size() != rowsB || comR.size() != rowsB || comA.size() != rowsB || comM.size() != (size_t)(y.N / y.Cp) * G1B) {
        std::cout << "REJECT: commitment row counts" << std::endl; return false;
    }
    Laps laps("rescale_verify");
    // (1) the homomorphic affine link, all rows at once
    {
        Dev dx(x, comX.data(), comX.size()), dxr(x, comXr.data(), comXr.size()), dr(x, comR.data(), comR.size());
        const Fr s = fr_u32(y.sf);
        uint32_t bad = 0;
        x.ck(zkh_g1_rows_check(x.c, dx.p, dxr.p, s.v, dr.p, y.Bp, &bad), "affine link");
        if (bad) { std::cout << "REJECT: affine link com_X != sf*com_Xr + com_rem (" << bad << " rows)" << std::endl; return false; }
    }
    laps.lap("affine_link");
    std::vector<Fr> ev((size_t)4 * y.logD);
    Fr A_f, S_f, m_f;
    {
        const std::vector<uint8_t> f = read_file(obdir + "/lookup.bin");
        uint32_t n = 0;
        if (f.size() >= 4) memcpy(&n, f.data(), 4);
        if (f.size() < 4 || n != 4 * y.logD) { std::cout << "REJECT: round count" << std::endl; return false; }
        if (f.size() != 4 + (size_t)(n + 3) * FRB) { std::cout << "REJECT: lookup.bin size" << std::endl; return false; }
        memcpy(ev.data(), &f[4], (size_t)n * FRB);
        memcpy(A_f.v, &f[4 + (size_t)n * FRB], FRB);
        memcpy(S_f.v, &f[4 + (size_t)(n + 1) * FRB], FRB);
        memcpy(m_f.v, &f[4 + (size_t)(n + 2) * FRB], FRB);
    }
    for (const Fr& e : ev) if (!fr_lt(e, FR_MOD)) { std::cout << "REJECT: non-canonical round evaluation" << std::endl; return false; }
    if (!fr_lt(A_f, FR_MOD) || !fr_lt(S_f, FR_MOD) || !fr_lt(m_f, FR_MOD)) { std::cout << "REJECT: non-canonical terminal" << std::endl; return false; }

    Transcript tr(seed);
    tr.absorb_u32("B", y.B); tr.absorb_u32("C", y.C); tr.absorb_u32("LOG_SF", y.log_sf);
    tr.absorb("com_X", comX.data(), comX.size());
    tr.absorb("com_Xr", comXr.data(), comXr.size());
    tr.absorb("com_rem", comR.data(), comR.size());
    tr.absorb("com_m", comM.data(), comM.size());
    const Fr beta = tr.challenge_fr();
    tr.absorb("com_A", comA.data(), comA.size());
    const Fr alpha = tr.challenge_fr();
    const std::vector<Fr> u = tr.challenge_vec(y.logD);

    // (2) the lookup rounds, (3) B_f and T_f from the public table, (4) the terminal identity
    std::vector<Fr> ws;
    {
        const std::vector<Fr> Tp = range_table(y);
        Dev td(x, Tp.data(), Tp.size() * FRB);
        if (!lookup_verify(x, tr, ev, A_f, S_f, m_f, alpha, beta, u, td, y.logD, y.logN, ws, laps)) return false;
    }
    tr.absorb_fr("A_f", A_f); tr.absorb_fr("S_f", S_f); tr.absorb_fr("m_f", m_f);

    // (5) the openings bind the terminals to the commitments
    const std::vector<Fr> u_pt(ws.rbegin(), ws.rend()), u_m(ws.rbegin(), ws.rend() - y.n1);
    if (cf.on()) {
        const std::vector<Fr> none;
        claim_emit(cf.accdir, make_claim(cf.obid, "A", obdir + "/com_A.bin", y.Cp, y.Bp, u_pt, none, A_f));
        claim_emit(cf.accdir, make_claim(cf.obid, "rem", obdir + "/com_rem.bin", y.Cp, y.Bp, u_pt, none, S_f));
        claim_emit(cf.accdir, make_claim(cf.obid, "m", obdir + "/com_m.bin", y.Cp, y.N / y.Cp, u_m, none, m_f));
        drvstate_emit(cf.accdir, cf.obid, tr.st);
        std::cout << "ACCEPT-conditional (3 claims emitted; final verdict gated on opening_batch)" << std::endl;
        return true;
    }
    Dev gd(x, g.data(), g.size());
    if (!open_check(x, comA, y.Cp, gd, q.data(), u_pt, A_f, obdir + "/ipa_A.bin", tr)) { std::cout << "REJECT: IPA opening of A_f vs com_A" << std::endl; return false; }
    if (!open_check(x, comR, y.Cp, gd, q.data(), u_pt, S_f, obdir + "/ipa_rem.bin", tr)) { std::cout << "REJECT: IPA opening of S_f vs com_rem" << std::endl; return false; }
    if (!open_check(x, comM, y.Cp, gd, q.data(), u_m, m_f, obdir + "/ipa_m.bin", tr)) { std::cout << "REJECT: IPA opening of m_f vs com_m" << std::endl; return false; }
    laps.lap("openings");
    std::cout << "ACCEPT" << std::endl;
    return true;
}

int do_verify(int argc, char** argv) {
    const ClaimFlags cf = claim_flags(argc, argv);
    argc = cf.base_argc;
    if (argc != 9) throw std::invalid_argument("verify <obdir> <seed> <B> <C> <LOG_SF> <gen.bin> <q.bin>");
    const Lay y = lay_of(argv[4], argv[5], argv[6]);
    const std::vector<uint8_t> g = read_file(argv[7]), q = read_file(argv[8]);
    if (q.size() < G1B) throw std::runtime_error("q.bin holds no point");
    Ctx x;
    return verify(x, argv[2], argv[3], y, g, q, cf) ? 0 : 1;
}

int run1(int argc, char** argv);

// prove -> verify on the reference's selftest shapes with generators made here, then changed files and a value out of range
int do_selftest() {
    static const uint32_t GEN[36] = {
        0xfd530c16u, 0x5cb38790u, 0x9976fff5u, 0x7817fc67u, 0x143ba1c1u, 0x154f95c7u, 0xf3d0e747u, 0xf0ae6acdu, 0x21dbf440u,
        0xedce6eccu, 0x9e0bfb75u, 0x12017741u, 0x0ce72271u, 0xbaac93d5u, 0x7918fd8eu, 0x8c22631au, 0x570725ceu, 0xdd595f13u,
        0x50405194u, 0x51ac5829u, 0xad0059c0u, 0x0e1c8c3fu, 0x5008a26au, 0x0bbc3efcu, 0x0002fffdu, 0x76090000u, 0xc40c0002u,
        0xebf4000bu, 0x53c758bau, 0x5f489857u, 0x70525745u, 0x77ce5853u, 0xa256ec6du, 0x5c071a97u, 0xfa80e493u, 0x15f65ec3u};
    char tmpl[] = "/tmp/zkob_rescale_selftest_XXXXXX";
    const char* dir = mkdtemp(tmpl);
    if (!dir) throw std::runtime_error("no temporary directory");
    const std::string D = dir;
    bool all = true;
    const uint32_t cases[3][3] = {{8, 4, 4}, {4, 16, 4}, {8, 6, 6}};
    const char* files[] = {"gen.bin", "q.bin", "X.i64", "com_X.bin", "com_Xr.bin", "com_rem.bin", "com_m.bin", "com_A.bin", "dims.bin", "lookup.bin",
                           "ipa_A.bin", "ipa_rem.bin", "ipa_m.bin"};
    for (const auto& cs : cases) {
        const uint32_t B = cs[0], C = cs[1], L = cs[2], Cp = 1u << clog2(C);
        uint64_t s = 0x9E3779B97F4A7C15ull * (B + 31 * C + 977 * L);
        auto next = [&]() { s = s * 6364136223846793005ull + 1442695040888963407ull; return (uint32_t)(s >> 33); };
        {
            Ctx x;
            Dev gd(x, GEN, sizeof GEN);
            std::vector<uint8_t> pts((size_t)(Cp + 1) * G1B);
            for (uint32_t i = 0; i < Cp + 1; i++) {
                const Fr k = fr_u32(2 * next() + 1);
                Dev kd(x, k.v, FRB);
                x.ck(zkh_g1_msm(x.c, gd.p, kd.p, 1, &pts[(size_t)i * G1B]), "generator");
            }
            write_file(D + "/gen.bin", std::vector<uint8_t>(pts.begin(), pts.begin() + (size_t)Cp * G1B));
            write_file(D + "/q.bin", std::vector<uint8_t>(pts.begin() + (size_t)Cp * G1B, pts.end()));
        }
        std::vector<int64_t> X((size_t)B * C);
        for (auto& v : X) v = (int64_t)(next() % 8191) - 4095;
        std::vector<uint8_t> xb(X.size() * 8);
        memcpy(xb.data(), X.data(), xb.size());
        write_file(D + "/X.i64", xb);
        const std::string sB = std::to_string(B), sC = std::to_string(C), sL = std::to_string(L), g = D + "/gen.bin", q = D + "/q.bin";
        auto call = [&](std::vector<std::string> a) {
            std::vector<char*> av;
            for (auto& t : a) av.push_back(const_cast<char*>(t.c_str()));
            return run1((int)av.size(), av.data());
        };
        auto ver = [&]() { return call({"zkob_rescale", "verify", D, "selftest:rescale", sB, sC, sL, g, q}); };
        bool ok = call({"zkob_rescale", "prove", D, "selftest:rescale", D + "/X.i64", sB, sC, sL, g, q}) == 0 && ver() == 0;
        struct { const char* file; long off; } forged[] = {{"/lookup.bin", 4 + 32}, {"/lookup.bin", -32}, {"/ipa_rem.bin", -32},
                                                           {"/com_A.bin", 24}, {"/com_rem.bin", 24}, {"/com_m.bin", 24}};
        bool rejected = true;
        for (const auto& f : forged) {
            std::vector<uint8_t> b = read_file(D + f.file);
            const size_t o = f.off >= 0 ? (size_t)f.off : b.size() - (size_t)(-f.off);
            b[o] += 1;
            write_file(D + f.file, b);
            rejected = rejected && ver() == 1;
            b[o] -= 1;
            write_file(D + f.file, b);
        }
        std::cout << "case " << B << "x" << C << " log_sf " << L << ": honest " << (ok ? "ACCEPT" : "FAIL") << ", six changed files "
                  << (rejected ? "REJECT" : "FAIL") << std::endl;
        all = all && ok && rejected;
    }
    for (const char* n : files) remove((D + "/" + n).c_str());
    remove(D.c_str());
    std::cout << (all ? "ZKOB-RESCALE SELFTEST: ALL PASS" : "ZKOB-RESCALE SELFTEST: FAIL") << std::endl;
    return all ? 0 : 1;
}

int run1(int argc, char** argv) {
    const std::string mode = argc > 1 ? argv[1] : "";
    try {
        if (mode == "selftest") return do_selftest();
        if (mode == "prove") return do_prove(argc, argv);
        if (mode == "verify") return do_verify(argc, argv);
    } catch (const std::invalid_argument& e) {
        std::cerr << "zkob_rescale: " << e.what() << std::endl;
        return 2;
    }
    std::cerr << "usage: zkob_rescale prove ... | verify ... | selftest | serve" << std::endl;
    return 2;
}

}  // namespace

int main(int argc, char** argv) {
    try {
        if (argc > 1 && std::string(argv[1]) == "serve") return serve_loop(argv[0], run1);
        return run1(argc, argv);
    } catch (const std::exception& e) {
        std::cerr << "zkob_rescale: " << e.what() << std::endl;
        return 3;
    }
}
