// Driver for the RMS-norm obligation of the reference's first proof stack, with the command line, the files and the exit codes of the
// reference's zkob_rmsnorm (zkllm-src/zkob_rmsnorm.cu:1-70, :123-586 prove, :593-975 verify).  It binds the inverse-RMS advice R (B
// values) to X (B x C int32) within +-1: with M[s] = sum_j X[s, j]^2 + C_eps the exact R satisfies (R-1)^2 M <= 2^64 C <= (R+1)^2 M.
//  1. limb range lookup: P1 = 2^64 C - (R-1)^2 M and P2 = (R+1)^2 M - 2^64 C, both in [0, 2^80), as five 16-bit limbs each in the
//     rows of L (max(16, 65536 / B) rows of B values, committed with gen_B), logUp against 0 .. 65535;
//  2. affine links, no openings: com_P1 == sum_i 2^(16 i) com_L[i], com_P2 == sum_i 2^(16 i) com_L[5 + i];
//  3. sum of squares: M~(u_b) - C_eps = sum eq . X . X (Hadamard sumcheck with the row-broadcast eq table, S_f2 == U_f2);
//  4. bracket quartics: 2^64 C - P1~(u_b2) over (eq, R-1, R-1, M) and P2~(u_b2) + 2^64 C over (eq, R+1, R+1, M); R opens at the
//     two terminal points expecting A_f + 1 and A_f - 1;
//  5. outer product W = R x g through val_W == val_R val_g (g against the REGISTERED commitment);
//  6. W_ = rescale(W, 2^16) committed here (its proof is a separate zkob_rescale run); 7. Hadamard Y = W_ .* X.
//
//   zkob_rmsnorm prove  <obdir> <seed> <X-int32> <R-int32> <g-int32> <B> <C> <C_eps-u64> <gen_C> <gen_B> <q.bin> [W-i64-out Y-i64-out]
//                       [--claims <accdir> <obid> <registered-com_g-path>]
//   zkob_rmsnorm verify <obdir> <seed> <B> <C> <C_eps> <com_g-path> <gen_C> <gen_B> <q.bin> [--claims <vaccdir> <obid>]
//   zkob_rmsnorm serve
//
// Files in <obdir> (byte for byte the reference's): dims.bin, com_{X,g,R,M,P1,P2,L,m_L,W,Wr,Y,A_L}.bin, lookup.bin, hpss.bin, qp1.bin,
// qp2.bin, outer.bin, hp.bin and 17 openings ipa_*.bin.  The weight-privacy mode (--wpriv) is refused.
// Exit 0 = success / ACCEPT, 1 = REJECT, anything else = failure.
#include "zkob_common.hpp"

using namespace zkob;

namespace {

typedef unsigned __int128 u128;
typedef __int128 i128;
constexpr uint32_t LOOKUP_N = 65536;

struct Lay { uint32_t B, C, Bp, Cp, D, logD, logB, logC, N, n_rows, DL, logDL, n1, logN; uint64_t C_eps; };
Lay lay_of(const char* b, const char* c, const char* ceps) {
    Lay y;
    y.B = (uint32_t)atoi(b); y.C = (uint32_t)atoi(c); y.C_eps = strtoull(ceps, nullptr, 10);
    if (!y.B || !y.C) throw std::runtime_error("bad dimensions");
    y.Bp = 1u << clog2(y.B); y.Cp = 1u << clog2(y.C);
    y.D = y.Bp * y.Cp; y.logD = clog2(y.D); y.logB = clog2(y.Bp); y.logC = clog2(y.Cp);
    y.N = LOOKUP_N; y.logN = 16;
    y.n_rows = std::max(16u, y.N / y.Bp); y.DL = y.n_rows * y.Bp;
    y.logDL = clog2(y.DL); y.n1 = clog2(y.DL / y.N);
    return y;
}
std::string layout_error(const Lay& y, size_t genC, size_t genB) {
    if (y.B != y.Bp) return "B must equal B_pad (power of two)";
    if (y.C >= (1u << 16)) return "C must be < 2^16";
    if (genC != (size_t)y.Cp * G1B) return "gen_C size != C_pad";
    if (genB != (size_t)y.Bp * G1B) return "gen_B size != B_pad";
    if (y.Bp > y.N || y.N > y.DL || y.DL % y.N) return "limb lookup layout needs B_pad <= N <= D_L, N | D_L";
    if (y.logB < 1) return "B must be at least 2";
    return "";
}
Fr fr_from_u128(u128 v) {
    Fr r{};
    for (int i = 0; i < 4; i++) r.v[i] = (uint32_t)(v >> (32 * i));
    return r;
}
Fr fr_from_u64(uint64_t v) { return fr_from_u128(v); }
void absorb_head(Transcript& tr, const Lay& y) {
    tr.absorb_u32("B", y.B); tr.absorb_u32("C", y.C); tr.absorb_u32("C_eps_lo", (uint32_t)y.C_eps); tr.absorb_u32("C_eps_hi", (uint32_t)(y.C_eps >> 32));
}
void write_pf(const std::string& path, const Fr& claim, const std::vector<Fr>& hev, const Fr& a, const Fr& b, const Fr* c = nullptr) {
    std::vector<uint8_t> f;
    const uint32_t n = (uint32_t)hev.size();
    put(f, claim.v, FRB); put(f, &n, 4); put(f, hev.data(), hev.size() * FRB); put(f, a.v, FRB); put(f, b.v, FRB);
    if (c) put(f, c->v, FRB);
    write_file(path, f);
}
// eq(u_b) broadcast along the rows of the padded grid (k_bcast_rows)
void bcast_eq(Ctx& x, const std::vector<Fr>& u_b, const Lay& y, Dev& out) {
    Dev e(x, (size_t)y.Bp * FRB);
    x.ck(zkh_fr_eq_build(x.c, u_b.data(), y.logB, e.p), "eq table");
    const std::vector<uint8_t> raw = e.host();
    std::vector<Fr> w((size_t)y.D);
    for (uint32_t i = 0; i < y.Bp; i++) {
        Fr v;
        memcpy(v.v, &raw[(size_t)i * FRB], FRB);
        for (uint32_t j = 0; j < y.Cp; j++) w[(size_t)i * y.Cp + j] = v;
    }
    x.ck(zkh_upload(x.c, out.p, w.data(), w.size() * FRB), "upload");
}
std::vector<std::string> qlabels(const char* tag) {
    std::vector<std::string> l;
    for (int i = 0; i < 5; i++) l.push_back(std::string(tag) + "p" + std::to_string(i));
    return l;
}

struct Sum { Fr claim, fin[4]; std::vector<Fr> ws, ev; };
// a product sumcheck over nc columns (3: Hadamard, labels hp0..hp3; 4: quartic, labels <tag>p0..p4)
Sum sumcheck(Ctx& x, Transcript& tr, const Fr& claim, const std::vector<const void*>& cols, uint32_t logn, const char* qtag) {
    Sum s;
    s.claim = claim;
    const int nc = (int)cols.size();
    s.ev.resize((size_t)(nc + 1) * logn);
    s.ws.resize(logn);
    std::vector<std::string> names = qtag ? qlabels(qtag) : std::vector<std::string>{"hp0", "hp1", "hp2", "hp3"};
    std::vector<const char*> labels;
    for (const std::string& n : names) labels.push_back(n.c_str());
    x.ck(zkh_fr_sumcheck(x.c, cols.data(), nc, logn, labels.data(), tr.st, s.ev.data(), s.ws.data(), s.fin), "sumcheck");
    return s;
}

int do_prove(int argc, char** argv) {
    const ClaimFlags cf = claim_flags(argc, argv);
    argc = cf.base_argc;
    if (argc != 13 && argc != 15)
        throw std::invalid_argument("prove <obdir> <seed> <X-int32> <R-int32> <g-int32> <B> <C> <C_eps-u64> <gen_C> <gen_B> <q.bin> [W-i64-out Y-i64-out]");
    if (cf.on() && cf.comref.empty()) throw std::runtime_error("prove --claims needs <accdir> <obid> <registered-com_g>");
    const std::string obdir = argv[2], seed = argv[3];
    const Lay y = lay_of(argv[7], argv[8], argv[9]);
    const uint32_t B = y.B, C = y.C, Cp = y.Cp, D = y.D, N = y.N, n_rows = y.n_rows, DL = y.DL;
    const std::vector<int32_t> Xh = load_ints(argv[4], (size_t)B * C), Rh = load_ints(argv[5], B), gh = load_ints(argv[6], C);
    const std::vector<uint8_t> genC = read_file(argv[10]), genB = read_file(argv[11]), q = read_file(argv[12]);
    if (q.size() < G1B) throw std::runtime_error("q.bin holds no point");
    const std::string le = layout_error(y, genC.size(), genB.size());
    if (!le.empty()) throw std::runtime_error(le);

    // the bracket arithmetic in 128-bit integers
    const u128 U1 = 1;
    const i128 c64C = ((i128)C) << 64;
    std::vector<Fr> Mf(B), P1f(B), P2f(B);
    std::vector<int64_t> Lh((size_t)DL, 0), cnt(N, 0), Rl(Rh.begin(), Rh.end()), T1h(B), T2h(B);
    for (uint32_t s = 0; s < B; s++) {
        u128 M = y.C_eps;
        for (uint32_t j = 0; j < C; j++) M += (u128)((int64_t)Xh[(size_t)s * C + j] * (int64_t)Xh[(size_t)s * C + j]);
        if (M >= (U1 << 62)) throw std::runtime_error("M >= 2^62");
        Mf[s] = fr_from_u128(M);
        const i128 r = Rh[s];
        const i128 V1 = c64C - (r - 1) * (r - 1) * (i128)M, V2 = (r + 1) * (r + 1) * (i128)M - c64C;
        if (V1 < 0 || V2 < 0) throw std::runtime_error("advice R out of +-1 tolerance (bracket violated)");
        if ((u128)V1 >= (U1 << 80) || (u128)V2 >= (U1 << 80)) throw std::runtime_error("bracket residual >= 2^80");
        for (uint32_t i = 0; i < 5; i++) {
            Lh[(size_t)i * B + s] = (int64_t)(((u128)V1 >> (16 * i)) & 0xFFFF);
            Lh[(size_t)(5 + i) * B + s] = (int64_t)(((u128)V2 >> (16 * i)) & 0xFFFF);
        }
        P1f[s] = fr_from_u128((u128)V1);
        P2f[s] = fr_from_u128((u128)V2);
        T1h[s] = Rh[s] - 1; T2h[s] = Rh[s] + 1;
    }
    for (size_t k = 0; k < DL; k++) cnt[(size_t)Lh[k]]++;
    // W = R x g, its rescaling by 2^16 (rescaling_kernel: remainder in [-2^15, 2^15)), Y = W_ .* X
    std::vector<int64_t> Wh((size_t)B * C), Wrh((size_t)B * C), Yh((size_t)B * C), Xl(Xh.begin(), Xh.end()), gl(gh.begin(), gh.end());
    const int64_t sf = 1 << 16, hsf = sf >> 1;
    for (uint32_t s = 0; s < B; s++)
        for (uint32_t j = 0; j < C; j++) {
            const size_t k = (size_t)s * C + j;
            Wh[k] = (int64_t)Rh[s] * (int64_t)gh[j];
            const int64_t t = (Wh[k] + hsf) % sf, rem = (t < 0 ? t + sf : t) - hsf;
            Wrh[k] = (Wh[k] - rem) / sf;
            Yh[k] = Wrh[k] * Xl[k];
        }
    if (argc == 15) {
        std::vector<uint8_t> b(Wh.size() * 8);
        memcpy(b.data(), Wh.data(), b.size());
        write_file(argv[13], b);
        memcpy(b.data(), Yh.data(), b.size());
        write_file(argv[14], b);
    }
    std::vector<int64_t> tab(N);
    for (uint32_t i = 0; i < N; i++) tab[i] = i;

    Ctx x;
    Dev gC(x, genC.data(), genC.size()), gB(x, genB.data(), genB.size());
    const std::vector<Fr> Xp = pad_matrix(Xl.data(), B, C, B, Cp), gp = pad_matrix(gl.data(), 1, C, 1, Cp), Rf = lift(Rl), T1f = lift(T1h), T2f = lift(T2h),
                          Lf = lift(Lh), mLf = lift(cnt), Wp = pad_matrix(Wh.data(), B, C, B, Cp), Wrp = pad_matrix(Wrh.data(), B, C, B, Cp),
                          Yp = pad_matrix(Yh.data(), B, C, B, Cp), Tp = lift(tab), none;
    Dev dX(x, Xp.data(), Xp.size() * FRB), dg(x, gp.data(), gp.size() * FRB), dR(x, Rf.data(), Rf.size() * FRB), dT1(x, T1f.data(), T1f.size() * FRB),
        dT2(x, T2f.data(), T2f.size() * FRB), dM(x, Mf.data(), Mf.size() * FRB), dP1(x, P1f.data(), P1f.size() * FRB), dP2(x, P2f.data(), P2f.size() * FRB),
        dL(x, Lf.data(), Lf.size() * FRB), dmL(x, mLf.data(), mLf.size() * FRB), dW(x, Wp.data(), Wp.size() * FRB), dWr(x, Wrp.data(), Wrp.size() * FRB),
        dY(x, Yp.data(), Yp.size() * FRB), dTab(x, Tp.data(), Tp.size() * FRB);
    const std::vector<uint8_t> comX = commit_rows(x, gC, dX, B, Cp), comg = commit_rows(x, gC, dg, 1, Cp), comR = commit_rows(x, gB, dR, 1, B),
                               comM = commit_rows(x, gB, dM, 1, B), comP1 = commit_rows(x, gB, dP1, 1, B), comP2 = commit_rows(x, gB, dP2, 1, B),
                               comL = commit_rows(x, gB, dL, n_rows, B), commL = commit_rows(x, gB, dmL, N / B, B), comW = commit_rows(x, gC, dW, B, Cp),
                               comWr = commit_rows(x, gC, dWr, B, Cp), comY = commit_rows(x, gC, dY, B, Cp);
    const struct { const char* name; const std::vector<uint8_t>* com; const char* label; } heads[11] = {
        {"com_X", &comX, "com_X"}, {"com_g", &comg, "com_g"}, {"com_R", &comR, "com_R"}, {"com_M", &comM, "com_M"}, {"com_P1", &comP1, "com_P1"},
        {"com_P2", &comP2, "com_P2"}, {"com_L", &comL, "com_L"}, {"com_m_L", &commL, "com_m_L"}, {"com_W", &comW, "com_W"}, {"com_Wr", &comWr, "com_W_"},
        {"com_Y", &comY, "com_Y"}};
    for (const auto& h : heads) write_file(obdir + "/" + h.name + ".bin", *h.com);
    { std::vector<uint8_t> f; const uint32_t dm[2] = {B, C}; put(f, dm, 8); put(f, &y.C_eps, 8); write_file(obdir + "/dims.bin", f); }

    Transcript tr(seed);
    absorb_head(tr, y);
    for (const auto& h : heads) tr.absorb(h.label, h.com->data(), h.com->size());
    const Fr beta = tr.challenge_fr();
    auto claim = [&](const char* tensor, const std::string& comref, uint32_t domain, uint32_t rows, const std::vector<Fr>& pt, const Fr& eval) {
        claim_emit(cf.accdir, make_claim(cf.obid, tensor, comref, domain, rows, pt, none, eval));
    };
    auto wref = [&](const char* tag, const std::string& comref, const std::vector<uint8_t>& scalars) {
        const std::string wit = cf.accdir + "/wit_" + cf.obid + "_" + tag + ".fr";
        write_file(wit, scalars);
        witref_emit(cf.accdir, comref, wit);
    };
    const uint8_t* Q = q.data();

    // (1) the limb range lookup
    {
        Dev dA(x, (size_t)DL * FRB), dBv(x, (size_t)N * FRB);
        x.ck(zkh_fr_inv_add(x.c, dL.p, DL, beta.v, dA.p), "A = 1 / (L + beta)");
        const std::vector<uint8_t> comA = commit_rows(x, gB, dA, n_rows, B);
        write_file(obdir + "/com_A_L.bin", comA);
        tr.absorb("com_A_L", comA.data(), comA.size());
        const Fr alpha = tr.challenge_fr();
        const std::vector<Fr> u = tr.challenge_vec(y.logDL);
        x.ck(zkh_fr_inv_add(x.c, dTab.p, N, beta.v, dBv.p), "B = 1 / (T + beta)");
        Fr bm;
        x.ck(zkh_fr_dot(x.c, dBv.p, dmL.p, N, bm.v), "sum B m");
        const Fr Cc = fr_sub(fr_mul(alpha, alpha), bm);
        std::vector<Fr> ev((size_t)4 * y.logDL), ws(y.logDL);
        Fr term[5];
        x.ck(zkh_fr_lookup_sumcheck(x.c, dA.p, dL.p, dBv.p, dTab.p, dmL.p, y.logDL, y.logN, alpha.v, beta.v, Cc.v, u.data(), tr.st, ev.data(), ws.data(), term),
             "limb lookup sumcheck");
        {
            std::vector<uint8_t> f;
            const uint32_t n = 4 * y.logDL;
            put(f, &n, 4); put(f, ev.data(), ev.size() * FRB); put(f, term[0].v, FRB); put(f, term[1].v, FRB); put(f, term[4].v, FRB);
            write_file(obdir + "/lookup.bin", f);
        }
        tr.absorb_fr("A_f", term[0]); tr.absorb_fr("S_f", term[1]); tr.absorb_fr("m_f", term[4]);
        const std::vector<Fr> u_pt(ws.rbegin(), ws.rend()), u_m(ws.rbegin(), ws.rend() - y.n1);
        if (cf.on()) {
            claim("AL", obdir + "/com_A_L.bin", B, n_rows, u_pt, term[0]);
            wref("AL", obdir + "/com_A_L.bin", dA.host());
            claim("L", obdir + "/com_L.bin", B, n_rows, u_pt, term[1]);
            wref("L", obdir + "/com_L.bin", dL.host());
            claim("mL", obdir + "/com_m_L.bin", B, N / B, u_m, term[4]);
            wref("mL", obdir + "/com_m_L.bin", dmL.host());
        } else {
            open_prove(x, dA, n_rows, B, gB, Q, u_pt, obdir + "/ipa_AL.bin", tr);
            open_prove(x, dL, n_rows, B, gB, Q, u_pt, obdir + "/ipa_L.bin", tr);
            open_prove(x, dmL, N / B, B, gB, Q, u_m, obdir + "/ipa_mL.bin", tr);
        }
    }
    // (3) the sum of squares
    {
        const std::vector<Fr> u_b = tr.challenge_vec(y.logB);
        Fr ev_M;
        x.ck(zkh_fr_mle_eval(x.c, dM.p, u_b.data(), y.logB, ev_M.v), "ev_M");
        tr.absorb_fr("ev_M", ev_M);
        Dev dE(x, (size_t)D * FRB);
        bcast_eq(x, u_b, y, dE);
        const Sum s = sumcheck(x, tr, ev_M, {dE.p, dX.p, dX.p}, y.logD, nullptr);
        tr.absorb_fr("S_f2", s.fin[1]); tr.absorb_fr("U_f2", s.fin[2]);
        write_pf(obdir + "/hpss.bin", ev_M, s.ev, s.fin[1], s.fin[2]);
        const std::vector<Fr> u_ss(s.ws.rbegin(), s.ws.rend());
        if (cf.on()) {
            claim("X_ss", obdir + "/com_X.bin", Cp, B, u_ss, s.fin[1]);
            wref("X", obdir + "/com_X.bin", dX.host());
            claim("M", obdir + "/com_M.bin", B, 1, u_b, ev_M);
            wref("M", obdir + "/com_M.bin", dM.host());
        } else {
            open_prove(x, dX, B, Cp, gC, Q, u_ss, obdir + "/ipa_X_ss.bin", tr);
            open_prove(x, dM, 1, B, gB, Q, u_b, obdir + "/ipa_M.bin", tr);
        }
    }
    // (4) the bracket quartics
    {
        const std::vector<Fr> u_b2 = tr.challenge_vec(y.logB);
        Fr ev_P1, ev_P2;
        x.ck(zkh_fr_mle_eval(x.c, dP1.p, u_b2.data(), y.logB, ev_P1.v), "ev_P1");
        x.ck(zkh_fr_mle_eval(x.c, dP2.p, u_b2.data(), y.logB, ev_P2.v), "ev_P2");
        tr.absorb_fr("ev_P1", ev_P1); tr.absorb_fr("ev_P2", ev_P2);
        Dev dE2(x, (size_t)B * FRB);
        x.ck(zkh_fr_eq_build(x.c, u_b2.data(), y.logB, dE2.p), "eq table");
        const Sum q1 = sumcheck(x, tr, ev_P1, {dE2.p, dT1.p, dT1.p, dM.p}, y.logB, "q1");
        const Sum q2 = sumcheck(x, tr, ev_P2, {dE2.p, dT2.p, dT2.p, dM.p}, y.logB, "q2");
        tr.absorb_fr("q1A_f", q1.fin[1]); tr.absorb_fr("q1B_f", q1.fin[2]); tr.absorb_fr("q1C_f", q1.fin[3]);
        tr.absorb_fr("q2A_f", q2.fin[1]); tr.absorb_fr("q2B_f", q2.fin[2]); tr.absorb_fr("q2C_f", q2.fin[3]);
        write_pf(obdir + "/qp1.bin", ev_P1, q1.ev, q1.fin[1], q1.fin[2], &q1.fin[3]);
        write_pf(obdir + "/qp2.bin", ev_P2, q2.ev, q2.fin[1], q2.fin[2], &q2.fin[3]);
        const std::vector<Fr> pt1(q1.ws.rbegin(), q1.ws.rend()), pt2(q2.ws.rbegin(), q2.ws.rend());
        const Fr one = fr_u32(1), R1 = fr_add(q1.fin[1], one), R2 = fr_sub(q2.fin[1], one);
        if (cf.on()) {
            claim("P1", obdir + "/com_P1.bin", B, 1, u_b2, ev_P1);
            wref("P1", obdir + "/com_P1.bin", dP1.host());
            claim("P2", obdir + "/com_P2.bin", B, 1, u_b2, ev_P2);
            wref("P2", obdir + "/com_P2.bin", dP2.host());
            claim("R_q1", obdir + "/com_R.bin", B, 1, pt1, R1);
            wref("R", obdir + "/com_R.bin", dR.host());
            claim("M_q1", obdir + "/com_M.bin", B, 1, pt1, q1.fin[3]);
            claim("R_q2", obdir + "/com_R.bin", B, 1, pt2, R2);
            claim("M_q2", obdir + "/com_M.bin", B, 1, pt2, q2.fin[3]);
        } else {
            open_prove(x, dP1, 1, B, gB, Q, u_b2, obdir + "/ipa_P1.bin", tr);
            open_prove(x, dP2, 1, B, gB, Q, u_b2, obdir + "/ipa_P2.bin", tr);
            open_prove(x, dR, 1, B, gB, Q, pt1, obdir + "/ipa_R_q1.bin", tr);
            open_prove(x, dM, 1, B, gB, Q, pt1, obdir + "/ipa_M_q1.bin", tr);
            open_prove(x, dR, 1, B, gB, Q, pt2, obdir + "/ipa_R_q2.bin", tr);
            open_prove(x, dM, 1, B, gB, Q, pt2, obdir + "/ipa_M_q2.bin", tr);
        }
    }
    // (5) the outer product W = R x g
    {
        const std::vector<Fr> u_b3 = tr.challenge_vec(y.logB), u_c3 = tr.challenge_vec(y.logC);
        std::vector<Fr> u_pt3(u_c3);
        u_pt3.insert(u_pt3.end(), u_b3.begin(), u_b3.end());
        Fr val_R, val_g, val_W;
        x.ck(zkh_fr_mle_eval(x.c, dR.p, u_b3.data(), y.logB, val_R.v), "val_R");
        if (y.logC) x.ck(zkh_fr_mle_eval(x.c, dg.p, u_c3.data(), y.logC, val_g.v), "val_g");
        else val_g = gp[0];
        x.ck(zkh_fr_mle_eval(x.c, dW.p, u_pt3.data(), y.logD, val_W.v), "val_W");
        if (!fr_eq(val_W, fr_mul(val_R, val_g))) throw std::runtime_error("outer product val_W != val_R*val_g (convention bug)");
        tr.absorb_fr("val_R", val_R); tr.absorb_fr("val_g", val_g); tr.absorb_fr("val_W", val_W);
        { std::vector<uint8_t> f; put(f, val_R.v, FRB); put(f, val_g.v, FRB); put(f, val_W.v, FRB); write_file(obdir + "/outer.bin", f); }
        if (cf.on()) {
            claim("R_o", obdir + "/com_R.bin", B, 1, u_b3, val_R);
            claim("g", cf.comref, Cp, 1, u_c3, val_g);              // against the REGISTERED commitment of g
            wref("g", cf.comref, dg.host());
            claim("W", obdir + "/com_W.bin", Cp, B, u_pt3, val_W);
            wref("W", obdir + "/com_W.bin", dW.host());
        } else {
            open_prove(x, dR, 1, B, gB, Q, u_b3, obdir + "/ipa_R_o.bin", tr);
            open_prove(x, dg, 1, Cp, gC, Q, u_c3, obdir + "/ipa_g.bin", tr);
            open_prove(x, dW, B, Cp, gC, Q, u_pt3, obdir + "/ipa_W.bin", tr);
        }
    }
    // (7) Hadamard Y = W_ .* X
    const std::vector<Fr> u_h = tr.challenge_vec(y.logD);
    Fr claim_Y;
    x.ck(zkh_fr_mle_eval(x.c, dY.p, u_h.data(), y.logD, claim_Y.v), "claim_Y");
    tr.absorb_fr("claim_Y", claim_Y);
    Dev dEh(x, (size_t)D * FRB);
    x.ck(zkh_fr_eq_build(x.c, u_h.data(), y.logD, dEh.p), "eq table");
    const Sum h = sumcheck(x, tr, claim_Y, {dEh.p, dWr.p, dX.p}, y.logD, nullptr);
    tr.absorb_fr("S_f2h", h.fin[1]); tr.absorb_fr("U_f2h", h.fin[2]);
    write_pf(obdir + "/hp.bin", claim_Y, h.ev, h.fin[1], h.fin[2]);
    const std::vector<Fr> u_pth(h.ws.rbegin(), h.ws.rend());
    if (cf.on()) {
        claim("Y", obdir + "/com_Y.bin", Cp, B, u_h, claim_Y);
        wref("Y", obdir + "/com_Y.bin", dY.host());
        claim("Wr", obdir + "/com_Wr.bin", Cp, B, u_pth, h.fin[1]);
        wref("Wr", obdir + "/com_Wr.bin", dWr.host());
        claim("X_h", obdir + "/com_X.bin", Cp, B, u_pth, h.fin[2]);
        drvstate_emit(cf.accdir, cf.obid, tr.st);
        std::cout << "PROVED rmsnorm obligation (claim mode, 17 claims emitted) -> " << obdir << std::endl;
        return 0;
    }
    open_prove(x, dY, B, Cp, gC, Q, u_h, obdir + "/ipa_Y.bin", tr);
    open_prove(x, dWr, B, Cp, gC, Q, u_pth, obdir + "/ipa_Wr.bin", tr);
    open_prove(x, dX, B, Cp, gC, Q, u_pth, obdir + "/ipa_X_h.bin", tr);
    std::cout << "PROVED rmsnorm obligation -> " << obdir << std::endl;
    return 0;
}

// claim, count, evaluations, then `nterm` terminals (read_hp / read_qp); false on a wrong size, count or a non-canonical scalar
struct Pf { Fr claim, fin[3]; std::vector<Fr> ev; };
bool read_pf(const std::string& path, uint32_t want, int nterm, Pf& p) {
    const std::vector<uint8_t> f = read_file(path);
    if (f.size() != FRB + 4 + (size_t)want * FRB + (size_t)nterm * FRB) return false;
    uint32_t n;
    memcpy(p.claim.v, &f[0], FRB);
    memcpy(&n, &f[FRB], 4);
    if (n != want) return false;
    p.ev.resize(n);
    memcpy(p.ev.data(), &f[FRB + 4], (size_t)n * FRB);
    for (int t = 0; t < nterm; t++) {
        memcpy(p.fin[t].v, &f[FRB + 4 + (size_t)(n + t) * FRB], FRB);
        if (!fr_lt(p.fin[t], FR_MOD)) return false;
    }
    for (const Fr& e : p.ev) if (!fr_lt(e, FR_MOD)) return false;
    return fr_lt(p.claim, FR_MOD);
}
// sum_{i<5} 2^(16 i) com_L[first + i] compared with the one-row commitment `com` as group elements
bool affine_link(Ctx& x, const std::vector<uint8_t>& comL, uint32_t first, const std::vector<uint8_t>& com) {
    std::vector<Fr> sc(8, fr_u32(0));
    for (uint32_t i = 0; i < 5; i++) { sc[i] = fr_u32(0); sc[i].v[i / 2] = (i & 1) ? 65536u : 1u; }
    Dev pts(x, &comL[(size_t)first * G1B], 8 * G1B), sd(x, sc.data(), sc.size() * FRB);
    uint8_t acc[G1B];
    x.ck(zkh_g1_msm(x.c, pts.p, sd.p, 8, acc), "limb combination");
    const uint8_t zero[G1B] = {0};
    const Fr one = fr_u32(1);
    Dev lhs(x, com.data(), G1B), a(x, acc, G1B), b(x, zero, G1B);
    uint32_t bad = 0;
    x.ck(zkh_g1_rows_check(x.c, lhs.p, a.p, one.v, b.p, 1, &bad), "affine link");
    return bad == 0;
}

bool verify(Ctx& x, const std::string& obdir, const std::string& seed, const Lay& y, const std::string& com_g_path, const std::vector<uint8_t>& genC,
            const std::vector<uint8_t>& genB, const std::vector<uint8_t>& q, const ClaimFlags& cf) {
    if (!layout_error(y, genC.size(), genB.size()).empty()) return rj("bad layout params");
    const uint32_t B = y.B, C = y.C, Cp = y.Cp, N = y.N, n_rows = y.n_rows, logB = y.logB, logD = y.logD;
    {
        const std::vector<uint8_t> f = read_file(obdir + "/dims.bin");
        if (f.size() < 16) return rj("dims.bin short read");
        uint32_t dm[2];
        uint64_t e;
        memcpy(dm, &f[0], 8); memcpy(&e, &f[8], 8);
        if (dm[0] != B || dm[1] != C || e != y.C_eps) return rj("dims.bin mismatch");
    }
    auto com = [&](const char* n) { return read_file(obdir + "/" + n + ".bin"); };
    const std::vector<uint8_t> comX = com("com_X"), comg = read_file(com_g_path), comR = com("com_R"), comM = com("com_M"), comP1 = com("com_P1"),
                               comP2 = com("com_P2"), comL = com("com_L"), commL = com("com_m_L"), comW = com("com_W"), comWr = com("com_Wr"), comY = com("com_Y"),
                               comAL = com("com_A_L");
    const size_t rB = (size_t)B * G1B;
    if (comX.size() != rB || comW.size() != rB || comWr.size() != rB || comY.size() != rB || comg.size() != G1B || comR.size() != G1B || comM.size() != G1B ||
        comP1.size() != G1B || comP2.size() != G1B || comL.size() != (size_t)n_rows * G1B || comAL.size() != (size_t)n_rows * G1B ||
        commL.size() != (size_t)(N / B) * G1B)
        return rj("commitment row counts");
    Pf ss, qp1, qp2, hp;
    std::vector<Fr> lev;
    Fr A_f, S_f, m_f, val_R, val_g, val_W;
    {
        const std::vector<uint8_t> f = read_file(obdir + "/lookup.bin");
        const uint32_t want = 4 * y.logDL;
        uint32_t n = 0;
        if (f.size() >= 4) memcpy(&n, f.data(), 4);
        if (f.size() != 4 + (size_t)want * FRB + 3 * FRB || n != want) return rj("limb lookup round count");
        lev.resize(n);
        memcpy(lev.data(), &f[4], (size_t)n * FRB);
        memcpy(A_f.v, &f[4 + (size_t)n * FRB], FRB); memcpy(S_f.v, &f[4 + (size_t)(n + 1) * FRB], FRB); memcpy(m_f.v, &f[4 + (size_t)(n + 2) * FRB], FRB);
        for (const Fr& e : lev) if (!fr_lt(e, FR_MOD)) return rj("limb lookup round count");
        if (!fr_lt(A_f, FR_MOD) || !fr_lt(S_f, FR_MOD) || !fr_lt(m_f, FR_MOD)) return rj("limb lookup round count");
    }
    if (!read_pf(obdir + "/hpss.bin", 4 * logD, 2, ss)) return rj("SS round count");
    if (!read_pf(obdir + "/qp1.bin", 5 * logB, 3, qp1) || !read_pf(obdir + "/qp2.bin", 5 * logB, 3, qp2)) return rj("quartic round count");
    if (!read_pf(obdir + "/hp.bin", 4 * logD, 2, hp)) return rj("hadamard round count");
    {
        const std::vector<uint8_t> f = read_file(obdir + "/outer.bin");
        if (f.size() < 3 * FRB) return rj("outer.bin short read");
        memcpy(val_R.v, &f[0], FRB); memcpy(val_g.v, &f[FRB], FRB); memcpy(val_W.v, &f[2 * FRB], FRB);
        if (!fr_lt(val_R, FR_MOD) || !fr_lt(val_g, FR_MOD) || !fr_lt(val_W, FR_MOD)) return rj("non-canonical outer.bin");
    }
    Laps laps("rmsnorm_verify");
    // (2) the homomorphic affine limb links
    if (!affine_link(x, comL, 0, comP1)) return rj("affine link P1 != sum 2^16i * com_L_row[i]");
    if (!affine_link(x, comL, 5, comP2)) return rj("affine link P2 != sum 2^16i * com_L_row[5+i]");

    Transcript tr(seed);
    absorb_head(tr, y);
    const struct { const char* label; const std::vector<uint8_t>* c; } heads[11] = {
        {"com_X", &comX}, {"com_g", &comg}, {"com_R", &comR}, {"com_M", &comM}, {"com_P1", &comP1}, {"com_P2", &comP2}, {"com_L", &comL}, {"com_m_L", &commL},
        {"com_W", &comW}, {"com_W_", &comWr}, {"com_Y", &comY}};
    for (const auto& h : heads) tr.absorb(h.label, h.c->data(), h.c->size());
    const Fr beta = tr.challenge_fr();
    tr.absorb("com_A_L", comAL.data(), comAL.size());
    const Fr alpha = tr.challenge_fr();
    const std::vector<Fr> u_L = tr.challenge_vec(y.logDL), none;
    Dev gC(x, genC.data(), genC.size()), gB(x, genB.data(), genB.size());
    const uint8_t* Q = q.data();
    // (1) the limb lookup
    std::vector<Fr> wsl;
    {
        std::vector<int64_t> tab(N);
        for (uint32_t i = 0; i < N; i++) tab[i] = i;
        const std::vector<Fr> Tp = lift(tab);
        Dev td(x, Tp.data(), Tp.size() * FRB);
        if (!lookup_verify(x, tr, lev, A_f, S_f, m_f, alpha, beta, u_L, td, y.logDL, y.logN, wsl, laps, "limb lookup")) return false;
    }
    tr.absorb_fr("A_f", A_f); tr.absorb_fr("S_f", S_f); tr.absorb_fr("m_f", m_f);
    const std::vector<Fr> u_ptL(wsl.rbegin(), wsl.rend()), u_mL(wsl.rbegin(), wsl.rend() - y.n1);
    if (!cf.on()) {
        if (!open_check(x, comAL, B, gB, Q, u_ptL, A_f, obdir + "/ipa_AL.bin", tr)) return rj("IPA opening of A_f vs com_A_L");
        if (!open_check(x, comL, B, gB, Q, u_ptL, S_f, obdir + "/ipa_L.bin", tr)) return rj("IPA opening of S_f vs com_L");
        if (!open_check(x, commL, B, gB, Q, u_mL, m_f, obdir + "/ipa_mL.bin", tr)) return rj("IPA opening of m_f vs com_m_L");
    }
    const Fr inv2 = fr_inv(fr_u32(2)), inv6 = fr_inv(fr_u32(6)), inv4 = fr_inv(fr_u32(4)), inv24 = fr_inv(fr_u32(24)), one = fr_u32(1);
    // (3) the sum of squares: the eq factor only over the row rounds (the row bits are the high bits)
    const std::vector<Fr> u_b = tr.challenge_vec(logB);
    tr.absorb_fr("ev_M", ss.claim);
    std::vector<Fr> ws_ss;
    {
        Fr cur = fr_sub(ss.claim, fr_from_u64(y.C_eps)), eq_acc = one;
        for (uint32_t k = 0; k < logD; k++) {
            const std::array<Fr, 4> e = {ss.ev[4 * k], ss.ev[4 * k + 1], ss.ev[4 * k + 2], ss.ev[4 * k + 3]};
            if (!fr_eq(cur, fr_add(e[0], e[1]))) return rj("SS round " + std::to_string(k) + " p(0)+p(1) != claim");
            tr.absorb_fr("hp0", e[0]); tr.absorb_fr("hp1", e[1]); tr.absorb_fr("hp2", e[2]); tr.absorb_fr("hp3", e[3]);
            const Fr w = tr.challenge_fr();
            ws_ss.push_back(w);
            cur = lagrange4(e, w, inv6, inv2);
            if (k < logB) eq_acc = fr_mul(eq_acc, eq1(u_b[logB - 1 - k], w));
        }
        if (!fr_eq(ss.fin[0], ss.fin[1])) return rj("SS S_f2 != U_f2");
        if (!fr_eq(cur, fr_mul(eq_acc, fr_mul(ss.fin[0], ss.fin[1])))) return rj("SS terminal identity");
    }
    tr.absorb_fr("S_f2", ss.fin[0]); tr.absorb_fr("U_f2", ss.fin[1]);
    const std::vector<Fr> u_ss(ws_ss.rbegin(), ws_ss.rend());
    if (!cf.on()) {
        if (!open_check(x, comX, Cp, gC, Q, u_ss, ss.fin[0], obdir + "/ipa_X_ss.bin", tr)) return rj("IPA opening of X (SS) vs com_X");
        if (!open_check(x, comM, B, gB, Q, u_b, ss.claim, obdir + "/ipa_M.bin", tr)) return rj("IPA opening of ev_M vs com_M");
    }
    // (4) the bracket quartics
    const std::vector<Fr> u_b2 = tr.challenge_vec(logB);
    tr.absorb_fr("ev_P1", qp1.claim); tr.absorb_fr("ev_P2", qp2.claim);
    Fr c64C{};
    c64C.v[2] = C;                                                  // 2^64 C
    std::vector<Fr> ws_q1, ws_q2;
    auto quartic = [&](const Pf& qp, Fr cur, const char* tag, std::vector<Fr>& ws) {
        Fr eqa = one;
        const std::vector<std::string> names = qlabels(tag);
        for (uint32_t k = 0; k < logB; k++) {
            const std::array<Fr, 5> e = {qp.ev[5 * k], qp.ev[5 * k + 1], qp.ev[5 * k + 2], qp.ev[5 * k + 3], qp.ev[5 * k + 4]};
            if (!fr_eq(cur, fr_add(e[0], e[1]))) return rj(std::string(tag) + " round " + std::to_string(k) + " p(0)+p(1) != claim");
            for (int i = 0; i < 5; i++) tr.absorb_fr(names[i].c_str(), e[i]);
            const Fr w = tr.challenge_fr();
            ws.push_back(w);
            cur = lagrange5(e, w, inv24, inv6, inv4);
            eqa = fr_mul(eqa, eq1(u_b2[logB - 1 - k], w));
        }
        if (!fr_eq(qp.fin[0], qp.fin[1])) return rj(std::string(tag) + " A_f != B_f");
        if (!fr_eq(cur, fr_mul(eqa, fr_mul(fr_mul(qp.fin[0], qp.fin[1]), qp.fin[2])))) return rj(std::string(tag) + " terminal identity");
        return true;
    };
    if (!quartic(qp1, fr_sub(c64C, qp1.claim), "q1", ws_q1)) return false;
    if (!quartic(qp2, fr_add(qp2.claim, c64C), "q2", ws_q2)) return false;
    tr.absorb_fr("q1A_f", qp1.fin[0]); tr.absorb_fr("q1B_f", qp1.fin[1]); tr.absorb_fr("q1C_f", qp1.fin[2]);
    tr.absorb_fr("q2A_f", qp2.fin[0]); tr.absorb_fr("q2B_f", qp2.fin[1]); tr.absorb_fr("q2C_f", qp2.fin[2]);
    const std::vector<Fr> pt1(ws_q1.rbegin(), ws_q1.rend()), pt2(ws_q2.rbegin(), ws_q2.rend());
    const Fr R1 = fr_add(qp1.fin[0], one), R2 = fr_sub(qp2.fin[0], one);
    if (!cf.on()) {
        if (!open_check(x, comP1, B, gB, Q, u_b2, qp1.claim, obdir + "/ipa_P1.bin", tr)) return rj("IPA opening of ev_P1 vs com_P1");
        if (!open_check(x, comP2, B, gB, Q, u_b2, qp2.claim, obdir + "/ipa_P2.bin", tr)) return rj("IPA opening of ev_P2 vs com_P2");
        if (!open_check(x, comR, B, gB, Q, pt1, R1, obdir + "/ipa_R_q1.bin", tr)) return rj("IPA opening of R@pt1 (expect q1.A_f + 1) vs com_R");
        if (!open_check(x, comM, B, gB, Q, pt1, qp1.fin[2], obdir + "/ipa_M_q1.bin", tr)) return rj("IPA opening of M@pt1 vs com_M");
        if (!open_check(x, comR, B, gB, Q, pt2, R2, obdir + "/ipa_R_q2.bin", tr)) return rj("IPA opening of R@pt2 (expect q2.A_f - 1) vs com_R");
        if (!open_check(x, comM, B, gB, Q, pt2, qp2.fin[2], obdir + "/ipa_M_q2.bin", tr)) return rj("IPA opening of M@pt2 vs com_M");
    }
    // (5) the outer product
    const std::vector<Fr> u_b3 = tr.challenge_vec(logB), u_c3 = tr.challenge_vec(y.logC);
    tr.absorb_fr("val_R", val_R); tr.absorb_fr("val_g", val_g); tr.absorb_fr("val_W", val_W);
    if (!fr_eq(val_W, fr_mul(val_R, val_g))) return rj("outer product check val_W != val_R * val_g");
    std::vector<Fr> u_pt3(u_c3);
    u_pt3.insert(u_pt3.end(), u_b3.begin(), u_b3.end());
    if (!cf.on()) {
        if (!open_check(x, comR, B, gB, Q, u_b3, val_R, obdir + "/ipa_R_o.bin", tr)) return rj("IPA opening of val_R vs com_R");
        if (!open_check(x, comg, Cp, gC, Q, u_c3, val_g, obdir + "/ipa_g.bin", tr)) return rj("IPA opening of val_g vs registered com_g");
        if (!open_check(x, comW, Cp, gC, Q, u_pt3, val_W, obdir + "/ipa_W.bin", tr)) return rj("IPA opening of val_W vs com_W");
    }
    // (7) Hadamard Y = W_ .* X
    const std::vector<Fr> u_h = tr.challenge_vec(logD);
    tr.absorb_fr("claim_Y", hp.claim);
    std::vector<Fr> wsh;
    {
        Fr cur = hp.claim, eq_h = one;
        for (uint32_t k = 0; k < logD; k++) {
            const std::array<Fr, 4> e = {hp.ev[4 * k], hp.ev[4 * k + 1], hp.ev[4 * k + 2], hp.ev[4 * k + 3]};
            if (!fr_eq(cur, fr_add(e[0], e[1]))) return rj("hadamard round " + std::to_string(k) + " p(0)+p(1) != claim");
            tr.absorb_fr("hp0", e[0]); tr.absorb_fr("hp1", e[1]); tr.absorb_fr("hp2", e[2]); tr.absorb_fr("hp3", e[3]);
            const Fr w = tr.challenge_fr();
            wsh.push_back(w);
            cur = lagrange4(e, w, inv6, inv2);
            eq_h = fr_mul(eq_h, eq1(u_h[logD - 1 - k], w));
        }
        if (!fr_eq(cur, fr_mul(eq_h, fr_mul(hp.fin[0], hp.fin[1])))) return rj("hadamard terminal identity");
    }
    tr.absorb_fr("S_f2h", hp.fin[0]); tr.absorb_fr("U_f2h", hp.fin[1]);
    const std::vector<Fr> u_pth(wsh.rbegin(), wsh.rend());
    if (cf.on()) {
        auto claim = [&](const char* tensor, const std::string& comref, uint32_t domain, uint32_t rows, const std::vector<Fr>& pt, const Fr& eval) {
            claim_emit(cf.accdir, make_claim(cf.obid, tensor, comref, domain, rows, pt, none, eval));
        };
        claim("AL", obdir + "/com_A_L.bin", B, n_rows, u_ptL, A_f);
        claim("L", obdir + "/com_L.bin", B, n_rows, u_ptL, S_f);
        claim("mL", obdir + "/com_m_L.bin", B, N / B, u_mL, m_f);
        claim("X_ss", obdir + "/com_X.bin", Cp, B, u_ss, ss.fin[0]);
        claim("M", obdir + "/com_M.bin", B, 1, u_b, ss.claim);
        claim("P1", obdir + "/com_P1.bin", B, 1, u_b2, qp1.claim);
        claim("P2", obdir + "/com_P2.bin", B, 1, u_b2, qp2.claim);
        claim("R_q1", obdir + "/com_R.bin", B, 1, pt1, R1);
        claim("M_q1", obdir + "/com_M.bin", B, 1, pt1, qp1.fin[2]);
        claim("R_q2", obdir + "/com_R.bin", B, 1, pt2, R2);
        claim("M_q2", obdir + "/com_M.bin", B, 1, pt2, qp2.fin[2]);
        claim("R_o", obdir + "/com_R.bin", B, 1, u_b3, val_R);
        claim("g", com_g_path, Cp, 1, u_c3, val_g);
        claim("W", obdir + "/com_W.bin", Cp, B, u_pt3, val_W);
        claim("Y", obdir + "/com_Y.bin", Cp, B, u_h, hp.claim);
        claim("Wr", obdir + "/com_Wr.bin", Cp, B, u_pth, hp.fin[0]);
        claim("X_h", obdir + "/com_X.bin", Cp, B, u_pth, hp.fin[1]);
        drvstate_emit(cf.accdir, cf.obid, tr.st);
        std::cout << "ACCEPT-conditional (17 claims emitted; final verdict gated on opening_batch)" << std::endl;
        return true;
    }
    if (!open_check(x, comY, Cp, gC, Q, u_h, hp.claim, obdir + "/ipa_Y.bin", tr)) return rj("IPA opening of claim_Y vs com_Y");
    if (!open_check(x, comWr, Cp, gC, Q, u_pth, hp.fin[0], obdir + "/ipa_Wr.bin", tr)) return rj("IPA opening of W_ terminal vs com_W_");
    if (!open_check(x, comX, Cp, gC, Q, u_pth, hp.fin[1], obdir + "/ipa_X_h.bin", tr)) return rj("IPA opening of X (hadamard) vs com_X");
    std::cout << "ACCEPT" << std::endl;
    return true;
}

int do_verify(int argc, char** argv) {
    const ClaimFlags cf = claim_flags(argc, argv);
    argc = cf.base_argc;
    if (argc != 11) throw std::invalid_argument("verify <obdir> <seed> <B> <C> <C_eps> <com_g-path> <gen_C> <gen_B> <q.bin>");
    const Lay y = lay_of(argv[4], argv[5], argv[6]);
    const std::vector<uint8_t> genC = read_file(argv[8]), genB = read_file(argv[9]), q = read_file(argv[10]);
    if (q.size() < G1B) throw std::runtime_error("q.bin holds no point");
    if (!layout_error(y, genC.size(), genB.size()).empty()) return rj("bad layout params") ? 0 : 1;
    Ctx x;
    return verify(x, argv[2], argv[3], y, argv[7], genC, genB, q, cf) ? 0 : 1;
}

int run1(int argc, char** argv) {
    const std::string mode = argc > 1 ? argv[1] : "";
    try {
        if (mode == "prove") return do_prove(argc, argv);
        if (mode == "verify") return do_verify(argc, argv);
    } catch (const std::invalid_argument& e) {
        std::cerr << "zkob_rmsnorm: " << e.what() << std::endl;
        return 2;
    }
    std::cerr << "usage: zkob_rmsnorm prove ... [--claims <accdir> <obid> <registered-com_g>] | verify ... [--claims <vaccdir> <obid>] | serve" << std::endl;
    return 2;
}

}  // namespace

int main(int argc, char** argv) {
    try {
        if (argc > 1 && std::string(argv[1]) == "serve") return serve_loop(argv[0], run1);
        return run1(argc, argv);
    } catch (const std::exception& e) {
        std::cerr << "zkob_rmsnorm: " << e.what() << std::endl;
        return 3;
    }
}
