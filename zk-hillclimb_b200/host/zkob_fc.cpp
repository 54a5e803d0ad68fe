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
// With --claims <accdir> <obid> [<registered com_W>] (zkob_fc.cu:41-57) prove appends its three terminal claims, the witness
// tensors and its final transcript state to the accumulator directory instead of opening inline, and verify recomputes the
// claims into the verifier's accumulator and answers "ACCEPT-conditional".  The weight-privacy variants of the reference
// (--wpriv, --apriv, --hiding) are not built: those flags are refused with exit code 2.
//
// Everything heavy runs through the C ABI of libzkh (commitments, partial evaluations, the sumcheck with its transcript on
// the device, the arguments, fold chains); the host keeps the transcript between those calls and a few scalars.
#include "zkob_common.hpp"

using namespace zkob;

namespace {

struct Dims { uint32_t B, IN, OUT, lb, lj, lk, Bp, INp, OUTp; };
Dims dims_of(const char* b, const char* in, const char* out) {
    Dims d;
    d.B = (uint32_t)atoi(b); d.IN = (uint32_t)atoi(in); d.OUT = (uint32_t)atoi(out);
    if (!d.B || d.IN < 2 || !d.OUT) throw std::runtime_error("bad dimensions (B >= 1, IN >= 2, OUT >= 1)");
    d.lb = clog2(d.B); d.lj = clog2(d.IN); d.lk = clog2(d.OUT);
    d.Bp = 1u << d.lb; d.INp = 1u << d.lj; d.OUTp = 1u << d.lk;
    return d;
}
int do_commit(int argc, char** argv) {
    if (claim_flags(argc, argv).on()) throw std::invalid_argument("commit takes no --claims block");
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
    const ClaimFlags cf = claim_flags(argc, argv);
    if (cf.on() && cf.comref.empty()) throw std::invalid_argument("prove --claims needs <accdir> <obid> <registered-com_W>");
    argc = cf.base_argc;
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
    if (cf.on()) {
        // claim mode: the three terminal claims go to the accumulator at the program points of the inline openings (order W, X,
        // Y) with the witness tensors the batch program reads, then this transcript's final state (zkob_fc.cu:442-470)
        const std::string witW = cf.accdir + "/wit_" + cf.obid + "_W.fr", witX = cf.accdir + "/wit_" + cf.obid + "_X.fr",
                          witY = cf.accdir + "/wit_" + cf.obid + "_Y.fr";
        save_scalars(witW, Wp); save_scalars(witX, Xp); save_scalars(witY, Yp);
        claim_emit(cf.accdir, make_claim(cf.obid, "W", cf.comref, d.OUTp, d.INp, u_output, u_input, claim_W));
        witref_emit(cf.accdir, cf.comref, witW);
        claim_emit(cf.accdir, make_claim(cf.obid, "X", obdir + "/com_X.bin", d.INp, d.Bp, u_input, u_batch, claim_X));
        witref_emit(cf.accdir, obdir + "/com_X.bin", witX);
        claim_emit(cf.accdir, make_claim(cf.obid, "Y", obdir + "/com_Y.bin", d.OUTp, d.Bp, u_output, u_batch, claim));
        witref_emit(cf.accdir, obdir + "/com_Y.bin", witY);
        drvstate_emit(cf.accdir, cf.obid, tr.st);
        std::cout << "PROVED matmul obligation (claim mode, 3 claims emitted) -> " << obdir << std::endl;
        return 0;
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

bool verify(Ctx& x, const std::string& obdir, const std::string& seed, const Dims& d, const std::string& comW_path, const std::vector<uint8_t>& gi,
            const std::vector<uint8_t>& go, const std::vector<uint8_t>& q, const ClaimFlags& cf) {
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

    if (cf.on()) {
        // claim mode: the claims recomputed from this replay go to the verifier's accumulator; the verdict is conditional on the batch
        claim_emit(cf.accdir, make_claim(cf.obid, "W", comW_path, d.OUTp, d.INp, u_output, u_input, claim_W));
        claim_emit(cf.accdir, make_claim(cf.obid, "X", obdir + "/com_X.bin", d.INp, d.Bp, u_input, u_batch, claim_X));
        claim_emit(cf.accdir, make_claim(cf.obid, "Y", obdir + "/com_Y.bin", d.OUTp, d.Bp, u_output, u_batch, claim));
        drvstate_emit(cf.accdir, cf.obid, tr.st);
        std::cout << "ACCEPT-conditional (3 claims emitted; final verdict gated on opening_batch)" << std::endl;
        return true;
    }
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
    const ClaimFlags cf = claim_flags(argc, argv);
    argc = cf.base_argc;
    if (argc != 11) throw std::invalid_argument("verify <obdir> <seed> <B> <IN> <OUT> <com_W.bin> <gen_in> <gen_out> <q>");
    const Dims d = dims_of(argv[4], argv[5], argv[6]);
    const std::vector<uint8_t> gi = read_file(argv[8]), go = read_file(argv[9]), q = read_file(argv[10]);
    if (q.size() < G1B) throw std::runtime_error("q.bin holds no point");
    Ctx x;
    return verify(x, argv[2], argv[3], d, argv[7], gi, go, q, cf) ? 0 : 1;
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

}  // namespace

int main(int argc, char** argv) {
    try {
        if (argc > 1 && std::string(argv[1]) == "serve") return serve_loop(argv[0], run1);
        return run1(argc, argv);
    } catch (const std::exception& e) {
        std::cerr << "zkob_fc: " << e.what() << std::endl;
        return 3;
    }
}
