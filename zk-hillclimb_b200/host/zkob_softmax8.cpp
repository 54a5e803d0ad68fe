// Driver for the temperature-8 causal softmax obligation (layer.attn.softmax.h{hh} of the faithful-architecture chain) of the
// reference's first proof stack, with the command line, the files and the exit codes of the reference's zkob_softmax8
// (zkllm-src/zkob_softmax8.cu:1-76, :153-706 prove, :746-1235 verify).  Beside the score grid z (B x NCOL int32, B == NCOL) it takes
// the per-row allowed maximum mx (B int32, one committed row) and binds
//   (R0) Dm[i, j] = mask (z - mx[i]) + (1 - mask) SENT, SENT = LOW8 + LEN8 - 1 the table's last row (mapped to 0): cD1 = the MLE of
//        mask .* z and cD2 = the MLE of mask .* bcast(mx) at u_d by two Hadamard sumchecks (the broadcast never committed: its
//        terminal opens com_mx at the row bits), Dm~(u_d) opened against com_Dm, Dm~(u_d) == cD1 - cD2 + SENT (1 - sum eq(u_d) mask);
//   (R1) E = X_E8[Dm - LOW8]: the mapping lookup on Dm + r E, the verifier forming com_Dm + r com_E; E is 0 at masked positions BY
//        THE TABLE, so the mask leaves every later weight;
//   (R2) S[i] = sum_j E[i, j]: a Hadamard sumcheck with the pure row-broadcast eq weight;
//   (R3) P = round_half_up(2^16 E / S) through the bracket r1 = 2^17 E + S - 2 P S in [0, 2S): c1 = E~(u_r), c2 = (P .* bcast(S))~(u_r),
//        the four limb planes of L at (u_r, plane bits), S at the row bits of u_r, the limb range lookup, the two bracket identities.
//
//   zkob_softmax8 prove  <obdir> <seed> <z-int32.bin> <mx-int32.bin> <B> <NCOL> <LOW8> <LEN8> <expmap8-int32.bin> <LEN_R8> <gen.bin>
//                        <q.bin> [P-int32-out.bin] [--claims <accdir> <obid>]
//   zkob_softmax8 verify <obdir> <seed> <B> <NCOL> <LOW8> <LEN8> <expmap8-int32.bin> <LEN_R8> <gen.bin> <q.bin> [--claims <vaccdir> <obid>]
//   zkob_softmax8 serve
//
// Files in <obdir> (byte for byte the reference's): dims.bin, com_{z,mx,Dm,E,P,S,L,m_E8,m_L,A_E8,A_L}.bin, lookup_E8.bin, lookup_L.bin,
// hp_cD1.bin, hp_cD2.bin, vdm.bin, hp_rs.bin, hp_v1.bin, hp_v2.bin, lvals.bin and 19 openings ipa_*.bin (claim mode: com_comb.bin and no
// openings).  Exit 0 = success / ACCEPT, 1 = REJECT, anything else = failure.
#include "zkob_common.hpp"

using namespace zkob;

namespace {

constexpr uint32_t LOG_OUT = 16;                                    // P at scale 2^16
constexpr int64_t ENV = 1LL << 19;                                  // the honest envelope of z and mx

struct Lay { uint32_t B, NCOL, LEN_E, LEN_R, D, DL, logB, logC, logD, logDL, logNE, logNR, n1E, n1L; int32_t LOW_E; };
Lay lay_of(const char* b, const char* ncol, const char* low, const char* lenE, const char* lenR) {
    Lay y;
    y.B = (uint32_t)atoi(b); y.NCOL = (uint32_t)atoi(ncol); y.LOW_E = atoi(low);
    y.LEN_E = (uint32_t)strtoul(lenE, nullptr, 10); y.LEN_R = (uint32_t)strtoul(lenR, nullptr, 10);
    if (!y.B || !y.NCOL || !y.LEN_E || !y.LEN_R) throw std::runtime_error("bad dimensions");
    y.D = y.B * y.NCOL; y.DL = 4 * y.D;
    y.logB = clog2(y.B); y.logC = clog2(y.NCOL); y.logD = y.logB + y.logC; y.logDL = y.logD + 2;
    y.logNE = clog2(y.LEN_E); y.logNR = clog2(y.LEN_R);
    y.n1E = y.logD >= y.logNE ? y.logD - y.logNE : 0;
    y.n1L = y.logDL >= y.logNR ? y.logDL - y.logNR : 0;
    return y;
}
std::string layout_error(const Lay& y, size_t gen) {
    if (y.B != y.NCOL) return "B != NCOL";
    if (y.B != (1u << y.logB)) return "B not a power of two";
    if (gen != (size_t)y.NCOL * G1B) return "generator size != NCOL";
    if (y.LEN_E != (1u << y.logNE) || y.LEN_R != (1u << y.logNR)) return "table lengths must be pow2";
    if (y.NCOL > y.LEN_E || y.LEN_E > y.D || y.D % y.LEN_E) return "exp lookup layout needs NCOL <= LEN8 <= D, LEN8 | D";
    if (y.NCOL > y.LEN_R || y.LEN_R > y.DL || y.DL % y.LEN_R) return "limb lookup layout needs NCOL <= LEN_R8 <= 4D, LEN_R8 | 4D";
    return "";
}
std::vector<int32_t> load_expmap(const std::string& path, uint32_t len) {
    if (len != (1u << clog2(len))) throw std::runtime_error("LEN8 must be pow2");
    const std::vector<uint8_t> raw = read_file(path);
    if (raw.size() < (size_t)len * 4) throw std::runtime_error("expmap8 table: short read");
    std::vector<int32_t> v(len);
    memcpy(v.data(), raw.data(), (size_t)len * 4);
    return v;
}
void absorb_head(Transcript& tr, const Lay& y) {
    tr.absorb_u32("B", y.B); tr.absorb_u32("NCOL", y.NCOL); tr.absorb_u32("LOW8", (uint32_t)y.LOW_E); tr.absorb_u32("LEN8", y.LEN_E);
    tr.absorb_u32("LEN_R8", y.LEN_R); tr.absorb_u32("LOG_OUT", LOG_OUT); tr.absorb_u32("SENT", (uint32_t)(int32_t)((int64_t)y.LOW_E + y.LEN_E - 1));
}
void write_lookup(const std::string& path, const std::vector<Fr>& ev, const Fr* term) {
    std::vector<uint8_t> f;
    const uint32_t n = (uint32_t)ev.size();
    put(f, &n, 4); put(f, ev.data(), ev.size() * FRB);
    put(f, term[0].v, FRB); put(f, term[1].v, FRB); put(f, term[4].v, FRB);
    write_file(path, f);
}
// the public causal mask as 0 / 1 scalars, and the row broadcast of a B-vector
std::vector<Fr> mask_grid(const Lay& y) {
    std::vector<Fr> m((size_t)y.D, fr_u32(0));
    for (uint32_t i = 0; i < y.B; i++)
        for (uint32_t j = 0; j <= i && j < y.NCOL; j++) m[(size_t)i * y.NCOL + j] = fr_u32(1);
    return m;
}
// W_rs = bcast_rows(eq(u_b)): row i carries eq(u_b)[i] in every column
void rowsum_weights(Ctx& x, const std::vector<Fr>& u_b, const Lay& y, Dev& out) {
    Dev e(x, (size_t)y.B * FRB);
    x.ck(zkh_fr_eq_build(x.c, u_b.data(), y.logB, e.p), "eq table");
    const std::vector<uint8_t> raw = e.host();
    std::vector<Fr> w((size_t)y.D, fr_u32(0));
    for (uint32_t i = 0; i < y.B; i++) {
        Fr v;
        memcpy(v.v, &raw[(size_t)i * FRB], FRB);
        for (uint32_t j = 0; j < y.NCOL; j++) w[(size_t)i * y.NCOL + j] = v;
    }
    x.ck(zkh_upload(x.c, out.p, w.data(), w.size() * FRB), "upload");
}
std::vector<Fr> plane_point(const std::vector<Fr>& u_r, uint32_t p) {
    std::vector<Fr> pt(u_r);
    pt.push_back(fr_u32(p & 1)); pt.push_back(fr_u32(p >> 1));
    return pt;
}
const char* const PLANE_FILE[4] = {"/ipa_L00.bin", "/ipa_L10.bin", "/ipa_L01.bin", "/ipa_L11.bin"};
const char* const PLANE_NAME[4] = {"L00", "L10", "L01", "L11"};
const char* const PLANE_LABEL[4] = {"v00", "v10", "v01", "v11"};

struct Had { Fr claim, S_f2, U_f2; std::vector<Fr> ws; };
// the Hadamard sumcheck over (E, S, U) with the claim already absorbed; the terminals absorbed and the file written
Had hadamard(Ctx& x, Transcript& tr, const Fr& claim, const Dev& dE, const Dev& dS, const Dev& dU, uint32_t logn, const std::string& path) {
    Had h;
    h.claim = claim;
    std::vector<Fr> hev((size_t)4 * logn);
    h.ws.resize(logn);
    Fr fin[3];
    const void* cols[3] = {dE.p, dS.p, dU.p};
    const char* labels[4] = {"hp0", "hp1", "hp2", "hp3"};
    x.ck(zkh_fr_sumcheck(x.c, cols, 3, logn, labels, tr.st, hev.data(), h.ws.data(), fin), "hadamard sumcheck");
    h.S_f2 = fin[1]; h.U_f2 = fin[2];
    tr.absorb_fr("S_f2", h.S_f2); tr.absorb_fr("U_f2", h.U_f2);
    write_hp(path, h.claim, hev, h.S_f2, h.U_f2);
    return h;
}

int do_prove(int argc, char** argv) {
    const ClaimFlags cf = claim_flags(argc, argv);
    argc = cf.base_argc;
    if (argc != 14 && argc != 15)
        throw std::invalid_argument("prove <obdir> <seed> <z-int32> <mx-int32> <B> <NCOL> <LOW8> <LEN8> <expmap8-int32> <LEN_R8> <gen> <q.bin> [P-int32-out]");
    const std::string obdir = argv[2], seed = argv[3];
    const Lay y = lay_of(argv[6], argv[7], argv[8], argv[9], argv[11]);
    const uint32_t B = y.B, NCOL = y.NCOL, D = y.D, DL = y.DL, LEN_E = y.LEN_E, LEN_R = y.LEN_R;
    const std::vector<int32_t> zh = load_ints(argv[4], (size_t)D), mxh = load_ints(argv[5], (size_t)B), maph = load_expmap(argv[10], LEN_E);
    const std::vector<uint8_t> gen = read_file(argv[12]), q = read_file(argv[13]);
    if (q.size() < G1B) throw std::runtime_error("q.bin holds no point");
    const std::string le = layout_error(y, gen.size());
    if (!le.empty()) throw std::runtime_error(le);
    const int64_t LENR2 = (int64_t)LEN_R * (int64_t)LEN_R, SENT = (int64_t)y.LOW_E + (int64_t)LEN_E - 1;
    if (maph[LEN_E - 1] != 0) throw std::runtime_error("table sentinel (last entry) != 0");

    // the host integer chain: Dm, E, S, P, the four limb planes, the multiplicities of both lookups
    std::vector<int64_t> zl(zh.begin(), zh.end()), mxl(mxh.begin(), mxh.end()), Dmh(D), Eh(D), Sh(B), Ph(D), Lh(DL), cntE(LEN_E, 0), cntL(LEN_R, 0);
    for (uint32_t i = 0; i < B; i++) {
        if (mxl[i] <= -ENV || mxl[i] >= ENV) throw std::runtime_error("mx outside the +-2^19 envelope");
        for (uint32_t j = 0; j < NCOL; j++) {
            const size_t idx = (size_t)i * NCOL + j;
            const int64_t z = zh[idx];
            if (z <= -ENV || z >= ENV) throw std::runtime_error("z_ outside the +-2^19 envelope");
            if (j <= i) {
                const int64_t diff = z - mxl[i];
                if (diff > 0) throw std::runtime_error("allowed diff > 0 (mx below the allowed row max)");
                if (diff < (int64_t)y.LOW_E) throw std::runtime_error("allowed diff below LOW8 (design 6.7 corner)");
                Dmh[idx] = diff;
            } else {
                Dmh[idx] = SENT;
            }
        }
    }
    for (size_t k = 0; k < D; k++) {
        Eh[k] = maph[(size_t)(Dmh[k] - y.LOW_E)];
        cntE[(size_t)(Dmh[k] - y.LOW_E)]++;
    }
    for (uint32_t i = 0; i < B; i++) {
        int64_t s = 0;
        for (uint32_t j = 0; j < NCOL; j++) s += Eh[(size_t)i * NCOL + j];
        if (s < 1) throw std::runtime_error("S[i] < 1 (table floor violated)");
        Sh[i] = s;
    }
    for (uint32_t i = 0; i < B; i++)
        for (uint32_t j = 0; j < NCOL; j++) {
            const size_t idx = (size_t)i * NCOL + j;
            const int64_t S = Sh[i], num = Eh[idx] * (int64_t)(1 << (LOG_OUT + 1)) + S;
            const int64_t P = num / (2 * S), r1 = num - 2 * P * S;
            if (r1 < 0 || r1 >= 2 * S) throw std::runtime_error("r1 out of [0, 2S) (P not per spec)");
            if (r1 >= LENR2 || 2 * S - 1 - r1 >= LENR2) throw std::runtime_error("bracket residual >= LEN_R8^2");
            const int64_t r2 = 2 * S - 1 - r1;
            Ph[idx] = P;
            Lh[idx] = r1 % LEN_R; Lh[(size_t)D + idx] = r1 / LEN_R;
            Lh[2 * (size_t)D + idx] = r2 % LEN_R; Lh[3 * (size_t)D + idx] = r2 / LEN_R;
        }
    for (size_t k = 0; k < DL; k++) cntL[(size_t)Lh[k]]++;
    if (argc == 15) {                                               // the chain file: B x NCOL int32, scale 2^16
        std::vector<int32_t> pi(D);
        for (size_t k = 0; k < D; k++) pi[k] = (int32_t)Ph[k];
        std::vector<uint8_t> b((size_t)D * 4);
        memcpy(b.data(), pi.data(), b.size());
        write_file(argv[14], b);
    }
    std::vector<int64_t> Sbh(D), mxbh(D), tabE(LEN_E), mapl(maph.begin(), maph.end()), tabR(LEN_R);
    for (uint32_t i = 0; i < B; i++)
        for (uint32_t j = 0; j < NCOL; j++) { Sbh[(size_t)i * NCOL + j] = Sh[i]; mxbh[(size_t)i * NCOL + j] = mxl[i]; }
    for (uint32_t i = 0; i < LEN_E; i++) tabE[i] = (int64_t)y.LOW_E + i;
    for (uint32_t i = 0; i < LEN_R; i++) tabR[i] = i;

    Ctx x;
    Dev gd(x, gen.data(), gen.size());
    const std::vector<Fr> zf = lift(zl), mxf = lift(mxl), Dmf = lift(Dmh), mxbf = lift(mxbh), Ef = lift(Eh), Sf = lift(Sh), Pf = lift(Ph), Lf = lift(Lh),
                          mEf = lift(cntE), mLf = lift(cntL), Sbf = lift(Sbh), MKf = mask_grid(y), ones((size_t)D, fr_u32(1)), none;
    Dev dmx(x, mxf.data(), mxf.size() * FRB), dDm(x, Dmf.data(), Dmf.size() * FRB), dmxb(x, mxbf.data(), mxbf.size() * FRB);
    Dev dz(x, zf.data(), zf.size() * FRB), dE(x, Ef.data(), Ef.size() * FRB), dS(x, Sf.data(), Sf.size() * FRB), dP(x, Pf.data(), Pf.size() * FRB),
        dL(x, Lf.data(), Lf.size() * FRB), dmE(x, mEf.data(), mEf.size() * FRB), dmL(x, mLf.data(), mLf.size() * FRB), dSb(x, Sbf.data(), Sbf.size() * FRB),
        dMK(x, MKf.data(), MKf.size() * FRB), dOnes(x, ones.data(), ones.size() * FRB);
    const std::vector<uint8_t> comz = commit_rows(x, gd, dz, B, NCOL), commx = commit_rows(x, gd, dmx, 1, NCOL), comDm = commit_rows(x, gd, dDm, B, NCOL),
                               comE = commit_rows(x, gd, dE, B, NCOL), comP = commit_rows(x, gd, dP, B, NCOL),
                               comS = commit_rows(x, gd, dS, 1, NCOL), comL = commit_rows(x, gd, dL, 4 * B, NCOL),
                               commE = commit_rows(x, gd, dmE, LEN_E / NCOL, NCOL), commL = commit_rows(x, gd, dmL, LEN_R / NCOL, NCOL);
    write_file(obdir + "/com_z.bin", comz); write_file(obdir + "/com_mx.bin", commx); write_file(obdir + "/com_Dm.bin", comDm);
    write_file(obdir + "/com_E.bin", comE); write_file(obdir + "/com_P.bin", comP);
    write_file(obdir + "/com_S.bin", comS); write_file(obdir + "/com_L.bin", comL); write_file(obdir + "/com_m_E8.bin", commE);
    write_file(obdir + "/com_m_L.bin", commL);
    {
        std::vector<uint8_t> f;
        const uint32_t d0[2] = {B, NCOL}, d1[3] = {LEN_E, LEN_R, LOG_OUT};
        const int32_t se = (int32_t)SENT;
        put(f, d0, 8); put(f, &y.LOW_E, 4); put(f, d1, 12); put(f, &se, 4);
        write_file(obdir + "/dims.bin", f);
    }
    Transcript tr(seed);
    absorb_head(tr, y);
    tr.absorb("com_z", comz.data(), comz.size()); tr.absorb("com_mx", commx.data(), commx.size()); tr.absorb("com_Dm", comDm.data(), comDm.size());
    tr.absorb("com_E", comE.data(), comE.size()); tr.absorb("com_P", comP.data(), comP.size());
    tr.absorb("com_S", comS.data(), comS.size()); tr.absorb("com_L", comL.data(), comL.size()); tr.absorb("com_m_E8", commE.data(), commE.size());
    tr.absorb("com_m_L", commL.data(), commL.size());
    const Fr r = tr.challenge_fr(), beta_E = tr.challenge_fr();
    auto claim = [&](const char* tensor, const std::string& comref, uint32_t rows, const std::vector<Fr>& pt, const Fr& eval) {
        claim_emit(cf.accdir, make_claim(cf.obid, tensor, comref, NCOL, rows, pt, none, eval));
    };
    auto wref = [&](const char* tag, const std::string& comref, const std::vector<uint8_t>& scalars) {
        const std::string wit = cf.accdir + "/wit_" + cf.obid + "_" + tag + ".fr";
        write_file(wit, scalars);
        witref_emit(cf.accdir, comref, wit);
    };

    // obligation 1: the exp mapping lookup on Dm + r E against table + r mapped
    {
        const std::vector<Fr> Tp = lift(tabE), Vp = lift(mapl);
        Dev comb(x, Dmf.data(), Dmf.size() * FRB), tcomb(x, Tp.data(), Tp.size() * FRB), dV(x, Vp.data(), Vp.size() * FRB);
        x.ck(zkh_fr_axpy(x.c, comb.p, dE.p, r.v, D), "Dm + r E");
        x.ck(zkh_fr_axpy(x.c, tcomb.p, dV.p, r.v, LEN_E), "table + r mapped");
        Dev dA(x, (size_t)D * FRB), dB(x, (size_t)LEN_E * FRB);
        x.ck(zkh_fr_inv_add(x.c, comb.p, D, beta_E.v, dA.p), "A = 1 / (comb + beta)");
        const std::vector<uint8_t> comA = commit_rows(x, gd, dA, B, NCOL);
        write_file(obdir + "/com_A_E8.bin", comA);
        tr.absorb("com_A_E8", comA.data(), comA.size());
        const Fr alpha = tr.challenge_fr();
        const std::vector<Fr> u = tr.challenge_vec(y.logD);
        x.ck(zkh_fr_inv_add(x.c, tcomb.p, LEN_E, beta_E.v, dB.p), "B = 1 / (T + beta)");
        Fr bm;
        x.ck(zkh_fr_dot(x.c, dB.p, dmE.p, LEN_E, bm.v), "sum B m");
        const Fr Cc = fr_sub(fr_mul(alpha, alpha), bm);
        std::vector<Fr> ev((size_t)4 * y.logD), ws(y.logD);
        Fr term[5];
        x.ck(zkh_fr_lookup_sumcheck(x.c, dA.p, comb.p, dB.p, tcomb.p, dmE.p, y.logD, y.logNE, alpha.v, beta_E.v, Cc.v, u.data(), tr.st, ev.data(), ws.data(), term),
             "exp lookup sumcheck");
        write_lookup(obdir + "/lookup_E8.bin", ev, term);
        tr.absorb_fr("A_f", term[0]); tr.absorb_fr("S_f", term[1]); tr.absorb_fr("m_f", term[4]);
        const std::vector<Fr> u_pt(ws.rbegin(), ws.rend()), u_m(ws.rbegin(), ws.rend() - y.n1E);
        if (cf.on()) {
            Dev cz(x, comDm.data(), comDm.size()), ce(x, comE.data(), comE.size()), cc(x, comDm.size());
            x.ck(zkh_g1_rows_lincomb(x.c, ce.p, r.v, cz.p, B, 0, cc.p), "com_Dm + r com_E");
            write_file(obdir + "/com_comb.bin", cc.host());
            claim("A_E8", obdir + "/com_A_E8.bin", B, u_pt, term[0]);
            wref("A_E8", obdir + "/com_A_E8.bin", dA.host());
            claim("comb", obdir + "/com_comb.bin", B, u_pt, term[1]);
            wref("comb", obdir + "/com_comb.bin", comb.host());
            claim("m_E8", obdir + "/com_m_E8.bin", LEN_E / NCOL, u_m, term[4]);
            wref("m_E8", obdir + "/com_m_E8.bin", dmE.host());
        } else {
            open_prove(x, dA, B, NCOL, gd, q.data(), u_pt, obdir + "/ipa_A_E8.bin", tr);
            open_prove(x, comb, B, NCOL, gd, q.data(), u_pt, obdir + "/ipa_comb.bin", tr);
            open_prove(x, dmE, LEN_E / NCOL, NCOL, gd, q.data(), u_m, obdir + "/ipa_m_E8.bin", tr);
        }
    }
    // obligation 2: the Dm-binding block at u_d: cD1 on z, cD2 on the broadcast of mx, both with the weight eq(u_d) .* mask
    {
        const std::vector<Fr> u_d = tr.challenge_vec(y.logD);
        Dev dW(x, (size_t)D * FRB);
        x.ck(zkh_fr_eq_build(x.c, u_d.data(), y.logD, dW.p), "eq table");
        x.ck(zkh_fr_mul(x.c, dW.p, dW.p, dMK.p, D), "eq .* mask");
        Fr cD1, cD2, vDm;
        x.ck(zkh_fr_dot(x.c, dW.p, dz.p, D, cD1.v), "cD1");
        tr.absorb_fr("cD1", cD1);
        const Had h1 = hadamard(x, tr, cD1, dW, dz, dOnes, y.logD, obdir + "/hp_cD1.bin");
        const std::vector<Fr> pt_cd1(h1.ws.rbegin(), h1.ws.rend());
        if (cf.on()) {
            claim("z_cD1", obdir + "/com_z.bin", B, pt_cd1, h1.S_f2);
            wref("z", obdir + "/com_z.bin", dz.host());
        } else {
            open_prove(x, dz, B, NCOL, gd, q.data(), pt_cd1, obdir + "/ipa_z_cD1.bin", tr);
        }
        x.ck(zkh_fr_dot(x.c, dW.p, dmxb.p, D, cD2.v), "cD2");
        tr.absorb_fr("cD2", cD2);
        const Had h2 = hadamard(x, tr, cD2, dW, dmxb, dOnes, y.logD, obdir + "/hp_cD2.bin");
        const std::vector<Fr> pt_cd2(h2.ws.rbegin(), h2.ws.rend()), pt_cd2_rows(pt_cd2.begin() + y.logC, pt_cd2.end());
        if (cf.on()) {                                              // the broadcast is pinned to com_mx at the row bits
            claim("mx_cD2", obdir + "/com_mx.bin", 1, pt_cd2_rows, h2.S_f2);
            wref("mx", obdir + "/com_mx.bin", dmx.host());
        } else {
            open_prove(x, dmx, 1, NCOL, gd, q.data(), pt_cd2_rows, obdir + "/ipa_mx_cD2.bin", tr);
        }
        x.ck(zkh_fr_mle_eval(x.c, dDm.p, u_d.data(), y.logD, vDm.v), "vDm");
        tr.absorb_fr("vDm", vDm);
        { std::vector<uint8_t> f; put(f, vDm.v, FRB); write_file(obdir + "/vdm.bin", f); }
        if (cf.on()) {
            claim("Dm", obdir + "/com_Dm.bin", B, u_d, vDm);
            wref("Dm", obdir + "/com_Dm.bin", dDm.host());
        } else {
            open_prove(x, dDm, B, NCOL, gd, q.data(), u_d, obdir + "/ipa_Dm.bin", tr);
        }
    }
    // obligation 3: the limb range lookup of L against 0 .. LEN_R8 - 1
    {
        const Fr beta = tr.challenge_fr();
        const std::vector<Fr> Tp = lift(tabR);
        Dev tab(x, Tp.data(), Tp.size() * FRB), dA(x, (size_t)DL * FRB), dB(x, (size_t)LEN_R * FRB);
        x.ck(zkh_fr_inv_add(x.c, dL.p, DL, beta.v, dA.p), "A = 1 / (L + beta)");
        const std::vector<uint8_t> comA = commit_rows(x, gd, dA, 4 * B, NCOL);
        write_file(obdir + "/com_A_L.bin", comA);
        tr.absorb("com_A_L", comA.data(), comA.size());
        const Fr alpha = tr.challenge_fr();
        const std::vector<Fr> u = tr.challenge_vec(y.logDL);
        x.ck(zkh_fr_inv_add(x.c, tab.p, LEN_R, beta.v, dB.p), "B = 1 / (T + beta)");
        Fr bm;
        x.ck(zkh_fr_dot(x.c, dB.p, dmL.p, LEN_R, bm.v), "sum B m");
        const Fr Cc = fr_sub(fr_mul(alpha, alpha), bm);
        std::vector<Fr> ev((size_t)4 * y.logDL), ws(y.logDL);
        Fr term[5];
        x.ck(zkh_fr_lookup_sumcheck(x.c, dA.p, dL.p, dB.p, tab.p, dmL.p, y.logDL, y.logNR, alpha.v, beta.v, Cc.v, u.data(), tr.st, ev.data(), ws.data(), term),
             "limb lookup sumcheck");
        write_lookup(obdir + "/lookup_L.bin", ev, term);
        tr.absorb_fr("A_f", term[0]); tr.absorb_fr("S_f", term[1]); tr.absorb_fr("m_f", term[4]);
        const std::vector<Fr> u_pt(ws.rbegin(), ws.rend()), u_m(ws.rbegin(), ws.rend() - y.n1L);
        if (cf.on()) {
            claim("A_L", obdir + "/com_A_L.bin", 4 * B, u_pt, term[0]);
            wref("A_L", obdir + "/com_A_L.bin", dA.host());
            claim("L_lk", obdir + "/com_L.bin", 4 * B, u_pt, term[1]);
            wref("L", obdir + "/com_L.bin", dL.host());
            claim("m_L", obdir + "/com_m_L.bin", LEN_R / NCOL, u_m, term[4]);
            wref("m_L", obdir + "/com_m_L.bin", dmL.host());
        } else {
            open_prove(x, dA, 4 * B, NCOL, gd, q.data(), u_pt, obdir + "/ipa_A_L.bin", tr);
            open_prove(x, dL, 4 * B, NCOL, gd, q.data(), u_pt, obdir + "/ipa_L_lk.bin", tr);
            open_prove(x, dmL, LEN_R / NCOL, NCOL, gd, q.data(), u_m, obdir + "/ipa_m_L.bin", tr);
        }
    }
    // obligation 4: the row sums, S~(u_b) = sum_b bcast_rows(eq(u_b))(b) E(b)
    {
        const std::vector<Fr> u_b = tr.challenge_vec(y.logB);
        Fr ev_S;
        x.ck(zkh_fr_mle_eval(x.c, dS.p, u_b.data(), y.logB, ev_S.v), "ev_S");
        tr.absorb_fr("ev_S", ev_S);
        Dev dW(x, (size_t)D * FRB);
        rowsum_weights(x, u_b, y, dW);
        const Had h = hadamard(x, tr, ev_S, dW, dE, dOnes, y.logD, obdir + "/hp_rs.bin");
        const std::vector<Fr> pt(h.ws.rbegin(), h.ws.rend());
        if (cf.on()) {
            claim("E_rs", obdir + "/com_E.bin", B, pt, h.S_f2);
            wref("E", obdir + "/com_E.bin", dE.host());
            claim("S_rs", obdir + "/com_S.bin", 1, u_b, ev_S);
            wref("S", obdir + "/com_S.bin", dS.host());
        } else {
            open_prove(x, dE, B, NCOL, gd, q.data(), pt, obdir + "/ipa_E_rs.bin", tr);
            open_prove(x, dS, 1, NCOL, gd, q.data(), u_b, obdir + "/ipa_S_rs.bin", tr);
        }
    }
    // obligations 5 and 6: c1 = E~(u_r), c2 = (P .* bcast(S))~(u_r)
    const std::vector<Fr> u_r = tr.challenge_vec(y.logD), ur_row(u_r.begin() + y.logC, u_r.end());
    Dev dEq(x, (size_t)D * FRB);
    x.ck(zkh_fr_eq_build(x.c, u_r.data(), y.logD, dEq.p), "eq table");
    {
        Fr c1;
        x.ck(zkh_fr_mle_eval(x.c, dE.p, u_r.data(), y.logD, c1.v), "c1");
        tr.absorb_fr("c1", c1);
        const Had h = hadamard(x, tr, c1, dEq, dE, dOnes, y.logD, obdir + "/hp_v1.bin");
        const std::vector<Fr> pt1(h.ws.rbegin(), h.ws.rend());
        if (cf.on()) claim("E_v1", obdir + "/com_E.bin", B, pt1, h.S_f2);
        else open_prove(x, dE, B, NCOL, gd, q.data(), pt1, obdir + "/ipa_E_v1.bin", tr);
    }
    {
        Dev dPS(x, (size_t)D * FRB);
        x.ck(zkh_fr_mul(x.c, dPS.p, dP.p, dSb.p, D), "P .* bcast(S)");
        Fr c2;
        x.ck(zkh_fr_dot(x.c, dEq.p, dPS.p, D, c2.v), "c2");
        tr.absorb_fr("c2", c2);
        const Had h = hadamard(x, tr, c2, dEq, dP, dSb, y.logD, obdir + "/hp_v2.bin");
        const std::vector<Fr> pt2(h.ws.rbegin(), h.ws.rend()), pt2_rows(pt2.begin() + y.logC, pt2.end());
        if (cf.on()) {
            claim("P_v2", obdir + "/com_P.bin", B, pt2, h.S_f2);
            wref("P", obdir + "/com_P.bin", dP.host());
            claim("S_v2", obdir + "/com_S.bin", 1, pt2_rows, h.U_f2);
        } else {
            open_prove(x, dP, B, NCOL, gd, q.data(), pt2, obdir + "/ipa_P_v2.bin", tr);
            open_prove(x, dS, 1, NCOL, gd, q.data(), pt2_rows, obdir + "/ipa_S_v2.bin", tr);
        }
    }
    // obligation 7: the four limb planes of L at (u_r, plane bits), and S at the row bits of u_r
    Fr lv[5];
    for (uint32_t p = 0; p < 4; p++) {
        const std::vector<Fr> pt = plane_point(u_r, p);
        x.ck(zkh_fr_mle_eval(x.c, dL.p, pt.data(), y.logDL, lv[p].v), "plane evaluation");
        tr.absorb_fr(PLANE_LABEL[p], lv[p]);
    }
    for (uint32_t p = 0; p < 4; p++) {
        const std::vector<Fr> pt = plane_point(u_r, p);
        if (cf.on()) claim(PLANE_NAME[p], obdir + "/com_L.bin", 4 * B, pt, lv[p]);
        else open_prove(x, dL, 4 * B, NCOL, gd, q.data(), pt, obdir + PLANE_FILE[p], tr);
    }
    x.ck(zkh_fr_mle_eval(x.c, dS.p, ur_row.data(), y.logB, lv[4].v), "S_id");
    tr.absorb_fr("S_id", lv[4]);
    { std::vector<uint8_t> f; put(f, lv, 5 * FRB); write_file(obdir + "/lvals.bin", f); }
    if (cf.on()) {
        claim("S_id", obdir + "/com_S.bin", 1, ur_row, lv[4]);
        drvstate_emit(cf.accdir, cf.obid, tr.st);
        std::cout << "PROVED softmax8 obligation (claim mode, 19 claims emitted) -> " << obdir << std::endl;
        return 0;
    }
    open_prove(x, dS, 1, NCOL, gd, q.data(), ur_row, obdir + "/ipa_S_id.bin", tr);
    std::cout << "PROVED softmax8 obligation -> " << obdir << std::endl;
    return 0;
}

struct Lk { Fr A_f, S_f, m_f; std::vector<Fr> ev; };
bool read_lookup(const std::string& path, uint32_t want, Lk& p) {
    const std::vector<uint8_t> f = read_file(path);
    if (f.size() != 4 + (size_t)want * FRB + 3 * FRB) return false;
    uint32_t n;
    memcpy(&n, &f[0], 4);
    if (n != want) return false;
    p.ev.resize(n);
    memcpy(p.ev.data(), &f[4], (size_t)n * FRB);
    memcpy(p.A_f.v, &f[4 + (size_t)n * FRB], FRB);
    memcpy(p.S_f.v, &f[4 + (size_t)(n + 1) * FRB], FRB);
    memcpy(p.m_f.v, &f[4 + (size_t)(n + 2) * FRB], FRB);
    for (const Fr& e : p.ev) if (!fr_lt(e, FR_MOD)) return false;
    return fr_lt(p.A_f, FR_MOD) && fr_lt(p.S_f, FR_MOD) && fr_lt(p.m_f, FR_MOD);
}

// the round checks of one Hadamard sumcheck; cur = the claim the terminal must meet, ws the challenges, eq_acc the product of eq(u, w)
// in the reference's order when u is given
bool hadamard_rounds(Transcript& tr, const Hp& hp, uint32_t logn, const char* tag, const Fr& inv2, const Fr& inv6, std::vector<Fr>& ws, Fr& cur,
                     const std::vector<Fr>* u = nullptr, Fr* eq_acc = nullptr) {
    cur = hp.claim;
    for (uint32_t k = 0; k < logn; k++) {
        const std::array<Fr, 4> e = {hp.ev[4 * k], hp.ev[4 * k + 1], hp.ev[4 * k + 2], hp.ev[4 * k + 3]};
        if (!fr_eq(cur, fr_add(e[0], e[1]))) return rj(std::string(tag) + " round " + std::to_string(k) + " p(0)+p(1) != claim");
        tr.absorb_fr("hp0", e[0]); tr.absorb_fr("hp1", e[1]); tr.absorb_fr("hp2", e[2]); tr.absorb_fr("hp3", e[3]);
        const Fr w = tr.challenge_fr();
        ws.push_back(w);
        cur = lagrange4(e, w, inv6, inv2);
        if (u) *eq_acc = fr_mul(*eq_acc, eq1((*u)[logn - 1 - k], w));
    }
    return true;
}

bool verify(Ctx& x, const std::string& obdir, const std::string& seed, const Lay& y, const std::vector<int32_t>& maph, const std::vector<uint8_t>& gen,
            const std::vector<uint8_t>& q, const ClaimFlags& cf) {
    if (!layout_error(y, gen.size()).empty()) return rj("bad layout params");
    const uint32_t B = y.B, NCOL = y.NCOL, D = y.D, LEN_E = y.LEN_E, LEN_R = y.LEN_R;
    if (maph[LEN_E - 1] != 0) return rj("table sentinel (last entry) != 0");
    const int64_t SENT = (int64_t)y.LOW_E + (int64_t)LEN_E - 1;
    {
        const std::vector<uint8_t> f = read_file(obdir + "/dims.bin");
        if (f.size() < 28) return rj("dims.bin short read");
        uint32_t d0[2], d1[3];
        int32_t lo, se;
        memcpy(d0, &f[0], 8); memcpy(&lo, &f[8], 4); memcpy(d1, &f[12], 12); memcpy(&se, &f[24], 4);
        if (d0[0] != B || d0[1] != NCOL || lo != y.LOW_E || d1[0] != LEN_E || d1[1] != LEN_R || d1[2] != LOG_OUT || se != (int32_t)SENT) return rj("dims.bin mismatch");
    }
    const std::vector<uint8_t> comz = read_file(obdir + "/com_z.bin"), commx = read_file(obdir + "/com_mx.bin"), comDm = read_file(obdir + "/com_Dm.bin"),
                               comE = read_file(obdir + "/com_E.bin"), comP = read_file(obdir + "/com_P.bin"),
                               comS = read_file(obdir + "/com_S.bin"), comL = read_file(obdir + "/com_L.bin"), commE = read_file(obdir + "/com_m_E8.bin"),
                               commL = read_file(obdir + "/com_m_L.bin"), comAE = read_file(obdir + "/com_A_E8.bin"), comAL = read_file(obdir + "/com_A_L.bin");
    const size_t rB = (size_t)B * G1B;
    if (comz.size() != rB || commx.size() != G1B || comDm.size() != rB || comE.size() != rB || comP.size() != rB || comS.size() != G1B || comL.size() != 4 * rB || comAE.size() != rB || comAL.size() != 4 * rB ||
        commE.size() != (size_t)(LEN_E / NCOL) * G1B || commL.size() != (size_t)(LEN_R / NCOL) * G1B)
        return rj("commitment row counts");
    Lk pfE, pfL;
    Hp hp_cd1, hp_cd2, hp_rs, hp_v1, hp_v2;
    Fr lv[5], vDm;
    {
        const std::vector<uint8_t> f = read_file(obdir + "/vdm.bin");
        if (f.size() < FRB) return rj("vdm.bin short read");
        memcpy(vDm.v, f.data(), FRB);
        if (!fr_lt(vDm, FR_MOD)) return rj("non-canonical vdm");
    }
    if (!read_lookup(obdir + "/lookup_E8.bin", 4 * y.logD, pfE)) return rj("exp lookup round count");
    if (!read_lookup(obdir + "/lookup_L.bin", 4 * y.logDL, pfL)) return rj("limb lookup round count");
    if (!read_hp(obdir + "/hp_cD1.bin", 4 * y.logD, hp_cd1) || !read_hp(obdir + "/hp_cD2.bin", 4 * y.logD, hp_cd2) || !read_hp(obdir + "/hp_rs.bin", 4 * y.logD, hp_rs) || !read_hp(obdir + "/hp_v1.bin", 4 * y.logD, hp_v1) || !read_hp(obdir + "/hp_v2.bin", 4 * y.logD, hp_v2))
        return rj("hadamard round count");
    {
        const std::vector<uint8_t> f = read_file(obdir + "/lvals.bin");
        if (f.size() < 5 * FRB) return rj("lvals.bin short read");
        memcpy(lv, f.data(), 5 * FRB);
        for (const Fr& v : lv) if (!fr_lt(v, FR_MOD)) return rj("non-canonical lvals");
    }
    Laps laps("softmax8_verify");
    const std::vector<Fr> MKf = mask_grid(y), none;
    Dev dMK(x, MKf.data(), MKf.size() * FRB), gd(x, gen.data(), gen.size());

    Transcript tr(seed);
    absorb_head(tr, y);
    tr.absorb("com_z", comz.data(), comz.size()); tr.absorb("com_mx", commx.data(), commx.size()); tr.absorb("com_Dm", comDm.data(), comDm.size());
    tr.absorb("com_E", comE.data(), comE.size()); tr.absorb("com_P", comP.data(), comP.size());
    tr.absorb("com_S", comS.data(), comS.size()); tr.absorb("com_L", comL.data(), comL.size()); tr.absorb("com_m_E8", commE.data(), commE.size());
    tr.absorb("com_m_L", commL.data(), commL.size());
    const Fr r = tr.challenge_fr(), beta_E = tr.challenge_fr();
    tr.absorb("com_A_E8", comAE.data(), comAE.size());
    const Fr alpha_E = tr.challenge_fr();
    const std::vector<Fr> u_E = tr.challenge_vec(y.logD);
    std::vector<uint8_t> comC;                                      // com_Dm + r com_E, formed homomorphically
    {
        Dev cz(x, comDm.data(), comDm.size()), ce(x, comE.data(), comE.size()), cc(x, comDm.size());
        x.ck(zkh_g1_rows_lincomb(x.c, ce.p, r.v, cz.p, B, 0, cc.p), "com_Dm + r com_E");
        comC = cc.host();
    }
    const Fr inv2 = fr_inv(fr_u32(2)), inv6 = fr_inv(fr_u32(6));

    // obligation 1: the exp lookup
    std::vector<Fr> ws_E;
    {
        std::vector<int64_t> tab(LEN_E), mp(maph.begin(), maph.end());
        for (uint32_t i = 0; i < LEN_E; i++) tab[i] = (int64_t)y.LOW_E + i;
        const std::vector<Fr> Tp = lift(tab), Vp = lift(mp);
        Dev tcomb(x, Tp.data(), Tp.size() * FRB), dV(x, Vp.data(), Vp.size() * FRB);
        x.ck(zkh_fr_axpy(x.c, tcomb.p, dV.p, r.v, LEN_E), "table + r mapped");
        if (!lookup_verify(x, tr, pfE.ev, pfE.A_f, pfE.S_f, pfE.m_f, alpha_E, beta_E, u_E, tcomb, y.logD, y.logNE, ws_E, laps, "exp lookup")) return false;
    }
    tr.absorb_fr("A_f", pfE.A_f); tr.absorb_fr("S_f", pfE.S_f); tr.absorb_fr("m_f", pfE.m_f);
    const std::vector<Fr> u_ptE(ws_E.rbegin(), ws_E.rend()), u_mE(ws_E.rbegin(), ws_E.rend() - y.n1E);
    if (cf.on()) {
        const std::vector<uint8_t> file = read_file(obdir + "/com_comb.bin");
        if (file.size() != rB) return rj("com_comb.bin row count");
        Dev cf_(x, file.data(), file.size()), cz(x, comDm.data(), comDm.size()), ce(x, comE.data(), comE.size());
        uint32_t bad = 0;
        x.ck(zkh_g1_rows_check(x.c, cf_.p, ce.p, r.v, cz.p, B, &bad), "com_comb.bin");
        if (bad) return rj("com_comb.bin != com_Dm + r*com_E (" + std::to_string(bad) + " rows)");
    } else {
        if (!open_check(x, comAE, NCOL, gd, q.data(), u_ptE, pfE.A_f, obdir + "/ipa_A_E8.bin", tr)) return rj("IPA opening of A_f vs com_A_E8");
        if (!open_check(x, comC, NCOL, gd, q.data(), u_ptE, pfE.S_f, obdir + "/ipa_comb.bin", tr)) return rj("IPA opening of S_f vs com_Dm + r*com_E");
        if (!open_check(x, commE, NCOL, gd, q.data(), u_mE, pfE.m_f, obdir + "/ipa_m_E8.bin", tr)) return rj("IPA opening of m_f vs com_m_E8");
    }
    // obligation 2, verifier side: the Dm-binding block, the verifier's own weight eq(u_d) .* mask folded over each leg's challenges
    const std::vector<Fr> u_d = tr.challenge_vec(y.logD);
    std::vector<Fr> ws_cd1, ws_cd2, ws_rs, ws_v1, ws_v2;
    Fr cur, k_MK;
    auto masked_leg = [&](const Hp& hp, const char* tag, std::vector<Fr>& ws, bool want_k) {
        tr.absorb_fr(tag, hp.claim);
        if (!hadamard_rounds(tr, hp, y.logD, tag, inv2, inv6, ws, cur)) return false;
        if (!fr_eq(hp.U_f2, fr_u32(1))) return rj(std::string(tag) + " U_f2 != 1");
        Dev dW(x, (size_t)D * FRB);
        x.ck(zkh_fr_eq_build(x.c, u_d.data(), y.logD, dW.p), "eq table");
        if (want_k) x.ck(zkh_fr_dot(x.c, dW.p, dMK.p, D, k_MK.v), "k_MK");       // sum_b eq(u_d, b) mask(b), for the Dm identity
        x.ck(zkh_fr_mul(x.c, dW.p, dW.p, dMK.p, D), "eq .* mask");
        const Fr W_f = fold_public(x, dW, D, ws);
        if (!fr_eq(cur, fr_mul(W_f, fr_mul(hp.S_f2, hp.U_f2)))) return rj(std::string(tag) + " terminal identity");
        tr.absorb_fr("S_f2", hp.S_f2); tr.absorb_fr("U_f2", hp.U_f2);
        return true;
    };
    if (!masked_leg(hp_cd1, "cD1", ws_cd1, true)) return false;
    const std::vector<Fr> pt_cd1(ws_cd1.rbegin(), ws_cd1.rend());
    if (!cf.on() && !open_check(x, comz, NCOL, gd, q.data(), pt_cd1, hp_cd1.S_f2, obdir + "/ipa_z_cD1.bin", tr)) return rj("IPA opening of cD1 terminal vs com_z");
    if (!masked_leg(hp_cd2, "cD2", ws_cd2, false)) return false;
    const std::vector<Fr> pt_cd2(ws_cd2.rbegin(), ws_cd2.rend()), pt_cd2_rows(pt_cd2.begin() + y.logC, pt_cd2.end());
    if (!cf.on() && !open_check(x, commx, NCOL, gd, q.data(), pt_cd2_rows, hp_cd2.S_f2, obdir + "/ipa_mx_cD2.bin", tr)) return rj("IPA opening of cD2 terminal vs com_mx");
    tr.absorb_fr("vDm", vDm);
    if (!cf.on() && !open_check(x, comDm, NCOL, gd, q.data(), u_d, vDm, obdir + "/ipa_Dm.bin", tr)) return rj("IPA opening of vDm vs com_Dm");
    // obligation 3: the limb lookup
    const Fr beta_L = tr.challenge_fr();
    tr.absorb("com_A_L", comAL.data(), comAL.size());
    const Fr alpha_L = tr.challenge_fr();
    const std::vector<Fr> u_L = tr.challenge_vec(y.logDL);
    std::vector<Fr> ws_L;
    {
        std::vector<int64_t> tab(LEN_R);
        for (uint32_t i = 0; i < LEN_R; i++) tab[i] = i;
        const std::vector<Fr> Tp = lift(tab);
        Dev td(x, Tp.data(), Tp.size() * FRB);
        if (!lookup_verify(x, tr, pfL.ev, pfL.A_f, pfL.S_f, pfL.m_f, alpha_L, beta_L, u_L, td, y.logDL, y.logNR, ws_L, laps, "limb lookup")) return false;
    }
    tr.absorb_fr("A_f", pfL.A_f); tr.absorb_fr("S_f", pfL.S_f); tr.absorb_fr("m_f", pfL.m_f);
    const std::vector<Fr> u_ptL(ws_L.rbegin(), ws_L.rend()), u_mL(ws_L.rbegin(), ws_L.rend() - y.n1L);
    if (!cf.on()) {
        if (!open_check(x, comAL, NCOL, gd, q.data(), u_ptL, pfL.A_f, obdir + "/ipa_A_L.bin", tr)) return rj("IPA opening of A_f vs com_A_L");
        if (!open_check(x, comL, NCOL, gd, q.data(), u_ptL, pfL.S_f, obdir + "/ipa_L_lk.bin", tr)) return rj("IPA opening of S_f vs com_L");
        if (!open_check(x, commL, NCOL, gd, q.data(), u_mL, pfL.m_f, obdir + "/ipa_m_L.bin", tr)) return rj("IPA opening of m_f vs com_m_L");
    }
    // obligation 4: the row sums; the broadcast eq weight folds to the product of eq factors over the row rounds (the row bits are the high bits)
    const std::vector<Fr> u_b = tr.challenge_vec(y.logB);
    tr.absorb_fr("ev_S", hp_rs.claim);
    if (!hadamard_rounds(tr, hp_rs, y.logD, "row-sum", inv2, inv6, ws_rs, cur)) return false;
    {
        Fr eq_acc = fr_u32(1);
        for (uint32_t k = 0; k < y.logB; k++) eq_acc = fr_mul(eq_acc, eq1(u_b[y.logB - 1 - k], ws_rs[k]));
        if (!fr_eq(hp_rs.U_f2, fr_u32(1))) return rj("row-sum U_f2 != 1");
        if (!fr_eq(cur, fr_mul(eq_acc, fr_mul(hp_rs.S_f2, hp_rs.U_f2)))) return rj("row-sum terminal identity");
    }
    tr.absorb_fr("S_f2", hp_rs.S_f2); tr.absorb_fr("U_f2", hp_rs.U_f2);
    const std::vector<Fr> pt_rs(ws_rs.rbegin(), ws_rs.rend());
    if (!cf.on()) {
        if (!open_check(x, comE, NCOL, gd, q.data(), pt_rs, hp_rs.S_f2, obdir + "/ipa_E_rs.bin", tr)) return rj("IPA opening of E (row-sum) vs com_E");
        if (!open_check(x, comS, NCOL, gd, q.data(), u_b, hp_rs.claim, obdir + "/ipa_S_rs.bin", tr)) return rj("IPA opening of ev_S vs com_S");
    }
    // obligation 5: V1, a pure eq weight
    const std::vector<Fr> u_r = tr.challenge_vec(y.logD), ur_row(u_r.begin() + y.logC, u_r.end());
    tr.absorb_fr("c1", hp_v1.claim);
    {
        Fr eq_v1 = fr_u32(1);
        if (!hadamard_rounds(tr, hp_v1, y.logD, "V1", inv2, inv6, ws_v1, cur, &u_r, &eq_v1)) return false;
        if (!fr_eq(hp_v1.U_f2, fr_u32(1))) return rj("V1 U_f2 != 1");
        if (!fr_eq(cur, fr_mul(eq_v1, fr_mul(hp_v1.S_f2, hp_v1.U_f2)))) return rj("V1 terminal identity");
    }
    tr.absorb_fr("S_f2", hp_v1.S_f2); tr.absorb_fr("U_f2", hp_v1.U_f2);
    const std::vector<Fr> pt1(ws_v1.rbegin(), ws_v1.rend());
    if (!cf.on() && !open_check(x, comE, NCOL, gd, q.data(), pt1, hp_v1.S_f2, obdir + "/ipa_E_v1.bin", tr)) return rj("IPA opening of E (V1) vs com_E");
    // obligation 6: V2, a pure eq weight
    tr.absorb_fr("c2", hp_v2.claim);
    Fr eq_acc = fr_u32(1);
    if (!hadamard_rounds(tr, hp_v2, y.logD, "V2", inv2, inv6, ws_v2, cur, &u_r, &eq_acc)) return false;
    if (!fr_eq(cur, fr_mul(eq_acc, fr_mul(hp_v2.S_f2, hp_v2.U_f2)))) return rj("V2 terminal identity");
    tr.absorb_fr("S_f2", hp_v2.S_f2); tr.absorb_fr("U_f2", hp_v2.U_f2);
    const std::vector<Fr> pt2(ws_v2.rbegin(), ws_v2.rend()), pt2_rows(pt2.begin() + y.logC, pt2.end());
    if (!cf.on()) {
        if (!open_check(x, comP, NCOL, gd, q.data(), pt2, hp_v2.S_f2, obdir + "/ipa_P_v2.bin", tr)) return rj("IPA opening of P (V2) vs com_P");
        // the never-committed broadcast is pinned to com_S: its MLE at pt2 is the row vector's MLE at the row bits of pt2
        if (!open_check(x, comS, NCOL, gd, q.data(), pt2_rows, hp_v2.U_f2, obdir + "/ipa_S_v2.bin", tr)) return rj("IPA opening of V2 U_f2 vs com_S");
    }
    // obligation 7: the limb planes, S_id, the bracket identities and the Dm identity
    for (uint32_t p = 0; p < 4; p++) tr.absorb_fr(PLANE_LABEL[p], lv[p]);
    if (!cf.on())
        for (uint32_t p = 0; p < 4; p++)
            if (!open_check(x, comL, NCOL, gd, q.data(), plane_point(u_r, p), lv[p], obdir + PLANE_FILE[p], tr))
                return rj(std::string("IPA opening of ") + PLANE_NAME[p] + " vs com_L");
    tr.absorb_fr("S_id", lv[4]);
    if (!cf.on() && !open_check(x, comS, NCOL, gd, q.data(), ur_row, lv[4], obdir + "/ipa_S_id.bin", tr)) return rj("IPA opening of S_id vs com_S");
    const Fr F_LENR = fr_u32(LEN_R), F_2P17 = fr_u32(1u << (LOG_OUT + 1));
    const Fr rt1 = fr_add(lv[0], fr_mul(F_LENR, lv[1])), rt2 = fr_add(lv[2], fr_mul(F_LENR, lv[3]));
    if (!fr_eq(fr_sub(fr_add(fr_mul(F_2P17, hp_v1.claim), lv[4]), fr_mul(fr_u32(2), hp_v2.claim)), rt1)) return rj("bracket r1 identity (I1)");
    if (!fr_eq(fr_add(fr_add(rt1, rt2), fr_u32(1)), fr_mul(fr_u32(2), lv[4]))) return rj("bracket sum identity (I2)");
    // Dm~(u_d) == cD1 - cD2 + SENT (1 - k_MK)
    if (!fr_eq(vDm, fr_add(fr_sub(hp_cd1.claim, hp_cd2.claim), fr_mul(fr_from_i64(SENT), fr_sub(fr_u32(1), k_MK))))) return rj("Dm identity");
    if (cf.on()) {
        auto claim = [&](const char* tensor, const std::string& comref, uint32_t rows, const std::vector<Fr>& pt, const Fr& eval) {
            claim_emit(cf.accdir, make_claim(cf.obid, tensor, comref, NCOL, rows, pt, none, eval));
        };
        claim("A_E8", obdir + "/com_A_E8.bin", B, u_ptE, pfE.A_f);
        claim("comb", obdir + "/com_comb.bin", B, u_ptE, pfE.S_f);
        claim("m_E8", obdir + "/com_m_E8.bin", LEN_E / NCOL, u_mE, pfE.m_f);
        claim("z_cD1", obdir + "/com_z.bin", B, pt_cd1, hp_cd1.S_f2);
        claim("mx_cD2", obdir + "/com_mx.bin", 1, pt_cd2_rows, hp_cd2.S_f2);
        claim("Dm", obdir + "/com_Dm.bin", B, u_d, vDm);
        claim("A_L", obdir + "/com_A_L.bin", 4 * B, u_ptL, pfL.A_f);
        claim("L_lk", obdir + "/com_L.bin", 4 * B, u_ptL, pfL.S_f);
        claim("m_L", obdir + "/com_m_L.bin", LEN_R / NCOL, u_mL, pfL.m_f);
        claim("E_rs", obdir + "/com_E.bin", B, pt_rs, hp_rs.S_f2);
        claim("S_rs", obdir + "/com_S.bin", 1, u_b, hp_rs.claim);
        claim("E_v1", obdir + "/com_E.bin", B, pt1, hp_v1.S_f2);
        claim("P_v2", obdir + "/com_P.bin", B, pt2, hp_v2.S_f2);
        claim("S_v2", obdir + "/com_S.bin", 1, pt2_rows, hp_v2.U_f2);
        for (uint32_t p = 0; p < 4; p++) claim(PLANE_NAME[p], obdir + "/com_L.bin", 4 * B, plane_point(u_r, p), lv[p]);
        claim("S_id", obdir + "/com_S.bin", 1, ur_row, lv[4]);
        drvstate_emit(cf.accdir, cf.obid, tr.st);
        std::cout << "ACCEPT-conditional (19 claims emitted; final verdict gated on opening_batch)" << std::endl;
        return true;
    }
    std::cout << "ACCEPT" << std::endl;
    return true;
}

int do_verify(int argc, char** argv) {
    const ClaimFlags cf = claim_flags(argc, argv);
    argc = cf.base_argc;
    if (argc != 12) throw std::invalid_argument("verify <obdir> <seed> <B> <NCOL> <LOW8> <LEN8> <expmap8-int32> <LEN_R8> <gen> <q.bin>");
    const Lay y = lay_of(argv[4], argv[5], argv[6], argv[7], argv[9]);
    const std::vector<int32_t> maph = load_expmap(argv[8], y.LEN_E);
    const std::vector<uint8_t> gen = read_file(argv[10]), q = read_file(argv[11]);
    if (q.size() < G1B) throw std::runtime_error("q.bin holds no point");
    if (!layout_error(y, gen.size()).empty()) return rj("bad layout params") ? 0 : 1;
    if (maph[y.LEN_E - 1] != 0) return rj("table sentinel (last entry) != 0") ? 0 : 1;
    Ctx x;
    return verify(x, argv[2], argv[3], y, maph, gen, q, cf) ? 0 : 1;
}

int run1(int argc, char** argv) {
    const std::string mode = argc > 1 ? argv[1] : "";
    try {
        if (mode == "prove") return do_prove(argc, argv);
        if (mode == "verify") return do_verify(argc, argv);
    } catch (const std::invalid_argument& e) {
        std::cerr << "zkob_softmax8: " << e.what() << std::endl;
        return 2;
    }
    std::cerr << "usage: zkob_softmax8 prove ... [--claims <accdir> <obid>] | verify ... [--claims <vaccdir> <obid>] | serve" << std::endl;
    return 2;
}

}  // namespace

int main(int argc, char** argv) {
    try {
        if (argc > 1 && std::string(argv[1]) == "serve") return serve_loop(argv[0], run1);
        return run1(argc, argv);
    } catch (const std::exception& e) {
        std::cerr << "zkob_softmax8: " << e.what() << std::endl;
        return 3;
    }
}
