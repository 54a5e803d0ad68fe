// Driver for the gated-activation obligation (mlp.swiglu) of the reference's first proof stack, with the command line, the
// files and the exit codes of the reference's zkob_glu (zkllm-src/zkob_glu.cu:1-63, :84-278 prove, :281-497 verify):
//   (1) mapping lookup: every pair (G[i], S[i]) is a row of the public table {(x, f(x))}: the logUp lookup on the combined
//       witness G + r S against the combined table, the verifier forming com_G + r com_S homomorphically;
//   (2) Hadamard sumcheck: H = S .* U through the equality-weighted degree-3 sumcheck.
//
//   zkob_glu prove  <obdir> <seed> <G-int32.bin> <U-int32.bin> <B> <C> <low> <len> <mapped-int32.bin> <gen.bin> <q.bin>
//                   [H-int64-out.bin] [--claims <accdir> <obid>]
//   zkob_glu verify <obdir> <seed> <B> <C> <low> <len> <mapped-int32.bin> <gen.bin> <q.bin> [--claims <vaccdir> <obid>]
//   zkob_glu serve
//
// Files in <obdir> (byte for byte the reference's): dims.bin, com_G / com_S / com_U / com_H / com_m / com_A.bin, lookup.bin,
// hp.bin, ipa_A / ipa_comb / ipa_m / ipa_H / ipa_S / ipa_U.bin; in claim mode com_comb.bin and the accumulator's files instead
// of the six openings.  Exit 0 = success / ACCEPT, 1 = REJECT, anything else = failure.
//
// Transcript schedule (zkob_glu.cu:24-33): B, C, LOW, LEN, com_G, com_S, com_U, com_H, com_m -> r -> beta; com_A -> alpha -> u;
// lookup rounds; A_f, S_f, m_f; openings of A, comb, m; u_h; claim_H; Hadamard rounds; S_f2, U_f2; openings of H, S, U.
#include "zkob_common.hpp"

using namespace zkob;

namespace {

struct Lay { uint32_t B, C, len, Bp, Cp, D, N, logD, logN, n1; int32_t low; };
Lay lay_of(const char* b, const char* c, const char* low, const char* len) {
    Lay y;
    y.B = (uint32_t)atoi(b); y.C = (uint32_t)atoi(c); y.low = atoi(low); y.len = (uint32_t)atoi(len);
    if (!y.B || !y.C || y.len < 2) throw std::runtime_error("bad dimensions");
    y.Bp = 1u << clog2(y.B); y.Cp = 1u << clog2(y.C);
    y.D = y.Bp * y.Cp; y.N = y.len;
    y.logD = clog2(y.D); y.logN = clog2(y.N);
    y.n1 = y.logD >= y.logN ? y.logD - y.logN : 0;
    return y;
}
bool layout_ok(const Lay& y) { return y.Cp <= y.N && y.N <= y.D && y.D % y.N == 0; }
// the mapped values of the public table, with the layout rule that the pair (0, 0) is a row (load_mapped, zkob_glu.cu:66-77)
std::vector<int32_t> load_mapped(const std::string& path, const Lay& y) {
    const std::vector<int32_t> m = load_ints(path, y.len);
    if (y.len != (1u << clog2(y.len))) throw std::runtime_error("table len must be pow2");
    if (y.low > 0 || (int64_t)y.low + y.len <= 0) throw std::runtime_error("table must contain x=0");
    if (m[(size_t)(-(int64_t)y.low)] != 0) throw std::runtime_error("layout needs mapped(0) == 0");
    return m;
}
// table + r * mapped on the device (T_comb); the same shape serves comb = G + r S
void combine(Ctx& x, Dev& acc, const Dev& add, const Fr& r, uint64_t n) { x.ck(zkh_fr_axpy(x.c, acc.p, add.p, r.v, n), "combination"); }
void absorb_head(Transcript& tr, const Lay& y) {
    tr.absorb_u32("B", y.B); tr.absorb_u32("C", y.C); tr.absorb_u32("LOW", (uint32_t)y.low); tr.absorb_u32("LEN", y.len);
}

int do_prove(int argc, char** argv) {
    const ClaimFlags cf = claim_flags(argc, argv);
    argc = cf.base_argc;
    if (argc != 13 && argc != 14) throw std::invalid_argument("prove <obdir> <seed> <G> <U> <B> <C> <low> <len> <mapped> <gen.bin> <q.bin> [H-out]");
    const std::string obdir = argv[2], seed = argv[3];
    const Lay y = lay_of(argv[6], argv[7], argv[8], argv[9]);
    const std::vector<int32_t> G = load_ints(argv[4], (size_t)y.B * y.C), U = load_ints(argv[5], (size_t)y.B * y.C), mapped = load_mapped(argv[10], y);
    const std::vector<uint8_t> g = read_file(argv[11]), q = read_file(argv[12]);
    if (g.size() != (size_t)y.Cp * G1B) throw std::runtime_error("generator size != C_pad");
    if (q.size() < G1B) throw std::runtime_error("q.bin holds no point");
    if (!layout_ok(y)) throw std::runtime_error("layout needs C_pad <= N <= D, N | D");
    // S = f(G) from the table, H = S .* U, multiplicities over the padded witness (the padding's zeros are the row (0, 0))
    std::vector<int64_t> Gl(G.begin(), G.end()), Ul(U.begin(), U.end()), S(G.size()), H(G.size()), cnt(y.N, 0), tab(y.N), mp(mapped.begin(), mapped.end());
    for (size_t i = 0; i < G.size(); i++) {
        const int64_t k = (int64_t)G[i] - y.low;
        if (k < 0 || k >= (int64_t)y.len) throw std::runtime_error("a value of G lies outside the table");
        S[i] = mapped[(size_t)k];
        H[i] = S[i] * U[i];
        cnt[(size_t)k]++;
    }
    cnt[(size_t)(-(int64_t)y.low)] += (int64_t)y.D - (int64_t)G.size();
    for (uint32_t i = 0; i < y.N; i++) tab[i] = (int64_t)y.low + i;
    if (argc == 14) {                                              // the chain file: the unpadded B x C products as int64
        std::vector<uint8_t> b(H.size() * 8);
        memcpy(b.data(), H.data(), b.size());
        write_file(argv[13], b);
    }
    Ctx x;
    const std::vector<Fr> Gp = pad_matrix(Gl.data(), y.B, y.C, y.Bp, y.Cp), Sp = pad_matrix(S.data(), y.B, y.C, y.Bp, y.Cp),
                          Up = pad_matrix(Ul.data(), y.B, y.C, y.Bp, y.Cp), Hp = pad_matrix(H.data(), y.B, y.C, y.Bp, y.Cp), Mp = lift(cnt);
    Dev gd(x, g.data(), g.size());
    Dev dG(x, Gp.data(), Gp.size() * FRB), dS(x, Sp.data(), Sp.size() * FRB), dU(x, Up.data(), Up.size() * FRB), dH(x, Hp.data(), Hp.size() * FRB),
        dM(x, Mp.data(), Mp.size() * FRB);
    const std::vector<uint8_t> comG = commit_rows(x, gd, dG, y.Bp, y.Cp), comS = commit_rows(x, gd, dS, y.Bp, y.Cp), comU = commit_rows(x, gd, dU, y.Bp, y.Cp),
                               comH = commit_rows(x, gd, dH, y.Bp, y.Cp), comM = commit_rows(x, gd, dM, y.N / y.Cp, y.Cp);
    write_file(obdir + "/com_G.bin", comG); write_file(obdir + "/com_S.bin", comS); write_file(obdir + "/com_U.bin", comU);
    write_file(obdir + "/com_H.bin", comH); write_file(obdir + "/com_m.bin", comM);
    { std::vector<uint8_t> f; const int32_t dm[4] = {(int32_t)y.B, (int32_t)y.C, y.low, (int32_t)y.len}; put(f, dm, 16); write_file(obdir + "/dims.bin", f); }

    Transcript tr(seed);
    absorb_head(tr, y);
    tr.absorb("com_G", comG.data(), comG.size()); tr.absorb("com_S", comS.data(), comS.size()); tr.absorb("com_U", comU.data(), comU.size());
    tr.absorb("com_H", comH.data(), comH.size()); tr.absorb("com_m", comM.data(), comM.size());
    const Fr r = tr.challenge_fr(), beta = tr.challenge_fr();
    // combined witness and table
    const std::vector<Fr> Tp = lift(tab), Vp = lift(mp);
    Dev comb(x, Gp.data(), Gp.size() * FRB), tcomb(x, Tp.data(), Tp.size() * FRB), dV(x, Vp.data(), Vp.size() * FRB);
    combine(x, comb, dS, r, y.D);
    combine(x, tcomb, dV, r, y.N);
    Dev dA(x, (size_t)y.D * FRB), dB(x, (size_t)y.N * FRB);
    x.ck(zkh_fr_inv_add(x.c, comb.p, y.D, beta.v, dA.p), "A = 1 / (comb + beta)");
    const std::vector<uint8_t> comA = commit_rows(x, gd, dA, y.Bp, y.Cp);
    write_file(obdir + "/com_A.bin", comA);
    tr.absorb("com_A", comA.data(), comA.size());
    const Fr alpha = tr.challenge_fr();
    const std::vector<Fr> u = tr.challenge_vec(y.logD);
    x.ck(zkh_fr_inv_add(x.c, tcomb.p, y.N, beta.v, dB.p), "B = 1 / (T + beta)");
    Fr bm;
    x.ck(zkh_fr_dot(x.c, dB.p, dM.p, y.N, bm.v), "sum B m");
    const Fr Cc = fr_sub(fr_mul(alpha, alpha), bm);
    std::vector<Fr> ev((size_t)4 * y.logD), ws(y.logD);
    Fr term[5];                                                     // A_f, S_f, B_f, T_f, m_f
    x.ck(zkh_fr_lookup_sumcheck(x.c, dA.p, comb.p, dB.p, tcomb.p, dM.p, y.logD, y.logN, alpha.v, beta.v, Cc.v, u.data(), tr.st, ev.data(), ws.data(), term),
         "lookup sumcheck");
    {
        std::vector<uint8_t> f;
        const uint32_t n = 4 * y.logD;
        put(f, &n, 4); put(f, ev.data(), ev.size() * FRB);
        put(f, term[0].v, FRB); put(f, term[1].v, FRB); put(f, term[4].v, FRB);
        write_file(obdir + "/lookup.bin", f);
    }
    tr.absorb_fr("A_f", term[0]); tr.absorb_fr("S_f", term[1]); tr.absorb_fr("m_f", term[4]);
    const std::vector<Fr> u_pt(ws.rbegin(), ws.rend()), u_m(ws.rbegin(), ws.rend() - y.n1), none;
    if (cf.on()) {
        // the file that stands for the verifier's homomorphic com_G + r com_S, then the lookup's three claims (order A, comb, m)
        {
            Dev cg(x, comG.data(), comG.size()), cs(x, comS.data(), comS.size()), cc(x, comG.size());
            x.ck(zkh_g1_rows_lincomb(x.c, cs.p, r.v, cg.p, y.Bp, 0, cc.p), "com_G + r com_S");
            write_file(obdir + "/com_comb.bin", cc.host());
        }
        const std::string witA = cf.accdir + "/wit_" + cf.obid + "_A.fr", witC = cf.accdir + "/wit_" + cf.obid + "_comb.fr",
                          witM = cf.accdir + "/wit_" + cf.obid + "_m.fr";
        write_file(witA, dA.host()); write_file(witC, comb.host()); save_scalars(witM, Mp);
        claim_emit(cf.accdir, make_claim(cf.obid, "A", obdir + "/com_A.bin", y.Cp, y.Bp, u_pt, none, term[0]));
        witref_emit(cf.accdir, obdir + "/com_A.bin", witA);
        claim_emit(cf.accdir, make_claim(cf.obid, "comb", obdir + "/com_comb.bin", y.Cp, y.Bp, u_pt, none, term[1]));
        witref_emit(cf.accdir, obdir + "/com_comb.bin", witC);
        claim_emit(cf.accdir, make_claim(cf.obid, "m", obdir + "/com_m.bin", y.Cp, y.N / y.Cp, u_m, none, term[4]));
        witref_emit(cf.accdir, obdir + "/com_m.bin", witM);
    } else {
        open_prove(x, dA, y.Bp, y.Cp, gd, q.data(), u_pt, obdir + "/ipa_A.bin", tr);
        open_prove(x, comb, y.Bp, y.Cp, gd, q.data(), u_pt, obdir + "/ipa_comb.bin", tr);
        open_prove(x, dM, y.N / y.Cp, y.Cp, gd, q.data(), u_m, obdir + "/ipa_m.bin", tr);
    }
    // Hadamard part: H~(u_h) = sum_b eq(u_h, b) S(b) U(b)
    const std::vector<Fr> u_h = tr.challenge_vec(y.logD);
    Fr claim_H;
    x.ck(zkh_fr_mle_eval(x.c, dH.p, u_h.data(), y.logD, claim_H.v), "claim_H");
    tr.absorb_fr("claim_H", claim_H);
    Dev dE(x, (size_t)y.D * FRB);
    x.ck(zkh_fr_eq_build(x.c, u_h.data(), y.logD, dE.p), "eq table");
    std::vector<Fr> hev((size_t)4 * y.logD), wsh(y.logD);
    Fr fin[3];
    const void* cols[3] = {dE.p, dS.p, dU.p};
    const char* labels[4] = {"hp0", "hp1", "hp2", "hp3"};
    x.ck(zkh_fr_sumcheck(x.c, cols, 3, y.logD, labels, tr.st, hev.data(), wsh.data(), fin), "hadamard sumcheck");
    tr.absorb_fr("S_f2", fin[1]); tr.absorb_fr("U_f2", fin[2]);
    {
        std::vector<uint8_t> f;
        const uint32_t n = 4 * y.logD;
        put(f, claim_H.v, FRB); put(f, &n, 4); put(f, hev.data(), hev.size() * FRB); put(f, fin[1].v, FRB); put(f, fin[2].v, FRB);
        write_file(obdir + "/hp.bin", f);
    }
    const std::vector<Fr> u_pt2(wsh.rbegin(), wsh.rend());
    if (cf.on()) {
        const std::string witH = cf.accdir + "/wit_" + cf.obid + "_H.fr", witS = cf.accdir + "/wit_" + cf.obid + "_S.fr",
                          witU = cf.accdir + "/wit_" + cf.obid + "_U.fr";
        save_scalars(witH, Hp); save_scalars(witS, Sp); save_scalars(witU, Up);
        claim_emit(cf.accdir, make_claim(cf.obid, "H", obdir + "/com_H.bin", y.Cp, y.Bp, u_h, none, claim_H));
        witref_emit(cf.accdir, obdir + "/com_H.bin", witH);
        claim_emit(cf.accdir, make_claim(cf.obid, "S", obdir + "/com_S.bin", y.Cp, y.Bp, u_pt2, none, fin[1]));
        witref_emit(cf.accdir, obdir + "/com_S.bin", witS);
        claim_emit(cf.accdir, make_claim(cf.obid, "U", obdir + "/com_U.bin", y.Cp, y.Bp, u_pt2, none, fin[2]));
        witref_emit(cf.accdir, obdir + "/com_U.bin", witU);
        drvstate_emit(cf.accdir, cf.obid, tr.st);
        std::cout << "PROVED swiglu obligation (claim mode, 6 claims emitted) -> " << obdir << std::endl;
        return 0;
    }
    open_prove(x, dH, y.Bp, y.Cp, gd, q.data(), u_h, obdir + "/ipa_H.bin", tr);
    open_prove(x, dS, y.Bp, y.Cp, gd, q.data(), u_pt2, obdir + "/ipa_S.bin", tr);
    open_prove(x, dU, y.Bp, y.Cp, gd, q.data(), u_pt2, obdir + "/ipa_U.bin", tr);
    std::cout << "PROVED swiglu obligation -> " << obdir << std::endl;
    return 0;
}

// count, then `count` scalars, at offset o of f; false when the file is too short or the count is not `want`
bool read_evals(const std::vector<uint8_t>& f, size_t& o, uint32_t want, std::vector<Fr>& ev) {
    uint32_t n = 0;
    if (o + 4 > f.size()) return false;
    memcpy(&n, &f[o], 4);
    o += 4;
    if (n != want || o + (size_t)n * FRB > f.size()) return false;
    ev.resize(n);
    memcpy(ev.data(), &f[o], (size_t)n * FRB);
    o += (size_t)n * FRB;
    for (const Fr& e : ev) if (!fr_lt(e, FR_MOD)) return false;
    return true;
}
bool read_scalar(const std::vector<uint8_t>& f, size_t& o, Fr& v) {
    if (o + FRB > f.size()) return false;
    memcpy(v.v, &f[o], FRB);
    o += FRB;
    return fr_lt(v, FR_MOD);
}

bool verify(Ctx& x, const std::string& obdir, const std::string& seed, const Lay& y, const std::vector<int32_t>& mapped, const std::vector<uint8_t>& g,
            const std::vector<uint8_t>& q, const ClaimFlags& cf) {
    if (g.size() != (size_t)y.Cp * G1B || !layout_ok(y)) { std::cout << "REJECT: bad layout params" << std::endl; return false; }
    {
        const std::vector<uint8_t> f = read_file(obdir + "/dims.bin");
        int32_t dm[4];
        if (f.size() < 16) return false;
        memcpy(dm, f.data(), 16);
        if (dm[0] != (int32_t)y.B || dm[1] != (int32_t)y.C || dm[2] != y.low || dm[3] != (int32_t)y.len) { std::cout << "REJECT: dims.bin mismatch" << std::endl; return false; }
    }
    const std::vector<uint8_t> comG = read_file(obdir + "/com_G.bin"), comS = read_file(obdir + "/com_S.bin"), comU = read_file(obdir + "/com_U.bin"),
                               comH = read_file(obdir + "/com_H.bin"), comM = read_file(obdir + "/com_m.bin"), comA = read_file(obdir + "/com_A.bin");
    const size_t rowsB = (size_t)y.Bp * G1B;
    if (comG.size() != rowsB || comS.size() != rowsB || comU.size() != rowsB || comH.size() != rowsB || comA.size() != rowsB ||
        comM.size() != (size_t)(y.N / y.Cp) * G1B) { std::cout << "REJECT: commitment row counts" << std::endl; return false; }
    std::vector<Fr> ev, hev;
    Fr A_f, S_f, m_f, claim_H, S_f2, U_f2;
    {
        const std::vector<uint8_t> f = read_file(obdir + "/lookup.bin"), h = read_file(obdir + "/hp.bin");
        size_t o = 0, p = 0;
        const bool okl = read_evals(f, o, 4 * y.logD, ev) && read_scalar(f, o, A_f) && read_scalar(f, o, S_f) && read_scalar(f, o, m_f) && o == f.size();
        const bool okh = read_scalar(h, p, claim_H) && read_evals(h, p, 4 * y.logD, hev) && read_scalar(h, p, S_f2) && read_scalar(h, p, U_f2) && p == h.size();
        if (!okl || !okh) { std::cout << "REJECT: round count" << std::endl; return false; }
    }
    Laps laps("glu_verify");
    Transcript tr(seed);
    absorb_head(tr, y);
    tr.absorb("com_G", comG.data(), comG.size()); tr.absorb("com_S", comS.data(), comS.size()); tr.absorb("com_U", comU.data(), comU.size());
    tr.absorb("com_H", comH.data(), comH.size()); tr.absorb("com_m", comM.data(), comM.size());
    const Fr r = tr.challenge_fr(), beta = tr.challenge_fr();
    tr.absorb("com_A", comA.data(), comA.size());
    const Fr alpha = tr.challenge_fr();
    const std::vector<Fr> u = tr.challenge_vec(y.logD);
    // the combined commitment, formed homomorphically: com_G + r com_S
    std::vector<uint8_t> comC;
    {
        Dev cg(x, comG.data(), comG.size()), cs(x, comS.data(), comS.size()), cc(x, comG.size());
        x.ck(zkh_g1_rows_lincomb(x.c, cs.p, r.v, cg.p, y.Bp, 0, cc.p), "com_G + r com_S");
        comC = cc.host();
    }
    laps.lap("comb_loop");
    std::vector<Fr> ws;
    {
        std::vector<int64_t> tab(y.N), mp(mapped.begin(), mapped.end());
        for (uint32_t i = 0; i < y.N; i++) tab[i] = (int64_t)y.low + i;
        const std::vector<Fr> Tp = lift(tab), Vp = lift(mp);
        Dev tcomb(x, Tp.data(), Tp.size() * FRB), dV(x, Vp.data(), Vp.size() * FRB);
        combine(x, tcomb, dV, r, y.N);
        if (!lookup_verify(x, tr, ev, A_f, S_f, m_f, alpha, beta, u, tcomb, y.logD, y.logN, ws, laps)) return false;
    }
    tr.absorb_fr("A_f", A_f); tr.absorb_fr("S_f", S_f); tr.absorb_fr("m_f", m_f);
    const std::vector<Fr> u_pt(ws.rbegin(), ws.rend()), u_m(ws.rbegin(), ws.rend() - y.n1), none;
    Dev gd(x, g.data(), g.size());
    if (cf.on()) {
        // the comb claim opens against the prover's com_comb.bin: only after that file equals this verifier's own combination
        const std::vector<uint8_t> file = read_file(obdir + "/com_comb.bin");
        if (file.size() != rowsB) { std::cout << "REJECT: com_comb.bin row count" << std::endl; return false; }
        Dev cf_(x, file.data(), file.size()), cg(x, comG.data(), comG.size()), cs(x, comS.data(), comS.size());
        uint32_t bad = 0;
        x.ck(zkh_g1_rows_check(x.c, cf_.p, cs.p, r.v, cg.p, y.Bp, &bad), "com_comb.bin");
        if (bad) { std::cout << "REJECT: com_comb.bin != com_G + r*com_S (" << bad << " rows)" << std::endl; return false; }
    } else {
        if (!open_check(x, comA, y.Cp, gd, q.data(), u_pt, A_f, obdir + "/ipa_A.bin", tr)) { std::cout << "REJECT: IPA opening of A_f vs com_A" << std::endl; return false; }
        if (!open_check(x, comC, y.Cp, gd, q.data(), u_pt, S_f, obdir + "/ipa_comb.bin", tr)) { std::cout << "REJECT: IPA opening of S_f vs com_G + r*com_S" << std::endl; return false; }
        if (!open_check(x, comM, y.Cp, gd, q.data(), u_m, m_f, obdir + "/ipa_m.bin", tr)) { std::cout << "REJECT: IPA opening of m_f vs com_m" << std::endl; return false; }
    }
    laps.lap("lookup");
    // Hadamard part
    const std::vector<Fr> u_h = tr.challenge_vec(y.logD);
    tr.absorb_fr("claim_H", claim_H);
    const Fr inv2 = fr_inv(fr_u32(2)), inv6 = fr_inv(fr_u32(6));
    Fr curh = claim_H, eq_acc = fr_u32(1);
    std::vector<Fr> wsh;
    for (uint32_t k = 0; k < y.logD; k++) {
        const std::array<Fr, 4> e = {hev[4 * k], hev[4 * k + 1], hev[4 * k + 2], hev[4 * k + 3]};
        if (!fr_eq(curh, fr_add(e[0], e[1]))) { std::cout << "REJECT: hadamard round " << k << " p(0)+p(1) != claim" << std::endl; return false; }
        tr.absorb_fr("hp0", e[0]); tr.absorb_fr("hp1", e[1]); tr.absorb_fr("hp2", e[2]); tr.absorb_fr("hp3", e[3]);
        const Fr w = tr.challenge_fr();
        wsh.push_back(w);
        curh = lagrange4(e, w, inv6, inv2);
        eq_acc = fr_mul(eq_acc, eq1(u_h[y.logD - 1 - k], w));
    }
    if (!fr_eq(curh, fr_mul(eq_acc, fr_mul(S_f2, U_f2)))) { std::cout << "REJECT: hadamard terminal identity" << std::endl; return false; }
    tr.absorb_fr("S_f2", S_f2); tr.absorb_fr("U_f2", U_f2);
    const std::vector<Fr> u_pt2(wsh.rbegin(), wsh.rend());
    if (cf.on()) {
        claim_emit(cf.accdir, make_claim(cf.obid, "A", obdir + "/com_A.bin", y.Cp, y.Bp, u_pt, none, A_f));
        claim_emit(cf.accdir, make_claim(cf.obid, "comb", obdir + "/com_comb.bin", y.Cp, y.Bp, u_pt, none, S_f));
        claim_emit(cf.accdir, make_claim(cf.obid, "m", obdir + "/com_m.bin", y.Cp, y.N / y.Cp, u_m, none, m_f));
        claim_emit(cf.accdir, make_claim(cf.obid, "H", obdir + "/com_H.bin", y.Cp, y.Bp, u_h, none, claim_H));
        claim_emit(cf.accdir, make_claim(cf.obid, "S", obdir + "/com_S.bin", y.Cp, y.Bp, u_pt2, none, S_f2));
        claim_emit(cf.accdir, make_claim(cf.obid, "U", obdir + "/com_U.bin", y.Cp, y.Bp, u_pt2, none, U_f2));
        drvstate_emit(cf.accdir, cf.obid, tr.st);
        std::cout << "ACCEPT-conditional (6 claims emitted; final verdict gated on opening_batch)" << std::endl;
        return true;
    }
    if (!open_check(x, comH, y.Cp, gd, q.data(), u_h, claim_H, obdir + "/ipa_H.bin", tr)) { std::cout << "REJECT: IPA opening of claim_H vs com_H" << std::endl; return false; }
    if (!open_check(x, comS, y.Cp, gd, q.data(), u_pt2, S_f2, obdir + "/ipa_S.bin", tr)) { std::cout << "REJECT: IPA opening of S_f2 vs com_S" << std::endl; return false; }
    if (!open_check(x, comU, y.Cp, gd, q.data(), u_pt2, U_f2, obdir + "/ipa_U.bin", tr)) { std::cout << "REJECT: IPA opening of U_f2 vs com_U" << std::endl; return false; }
    laps.lap("hadamard");
    std::cout << "ACCEPT" << std::endl;
    return true;
}

int do_verify(int argc, char** argv) {
    const ClaimFlags cf = claim_flags(argc, argv);
    argc = cf.base_argc;
    if (argc != 11) throw std::invalid_argument("verify <obdir> <seed> <B> <C> <low> <len> <mapped> <gen.bin> <q.bin>");
    const Lay y = lay_of(argv[4], argv[5], argv[6], argv[7]);
    const std::vector<int32_t> mapped = load_mapped(argv[8], y);
    const std::vector<uint8_t> g = read_file(argv[9]), q = read_file(argv[10]);
    if (q.size() < G1B) throw std::runtime_error("q.bin holds no point");
    Ctx x;
    return verify(x, argv[2], argv[3], y, mapped, g, q, cf) ? 0 : 1;
}

int run1(int argc, char** argv) {
    const std::string mode = argc > 1 ? argv[1] : "";
    try {
        if (mode == "prove") return do_prove(argc, argv);
        if (mode == "verify") return do_verify(argc, argv);
    } catch (const std::invalid_argument& e) {
        std::cerr << "zkob_glu: " << e.what() << std::endl;
        return 2;
    }
    std::cerr << "usage: zkob_glu prove ... [--claims <accdir> <obid>] | verify ... [--claims <vaccdir> <obid>] | serve" << std::endl;
    return 2;
}

}  // namespace

int main(int argc, char** argv) {
    try {
        if (argc > 1 && std::string(argv[1]) == "serve") return serve_loop(argv[0], run1);
        return run1(argc, argv);
    } catch (const std::exception& e) {
        std::cerr << "zkob_glu: " << e.what() << std::endl;
        return 3;
    }
}
