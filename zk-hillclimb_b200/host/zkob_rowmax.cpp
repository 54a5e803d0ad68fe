// Driver for the row-maximum obligation of the reference's first proof stack, with the command line, the files and the exit codes of
// the reference's zkob_rowmax (zkllm-src/zkob_rowmax.cu:1-66, :403-1020 prove, :1046-1484 verify).  It proves that the committed
// row of B scalars mx holds mx[i] = max over the allowed columns of row i of the committed B x NCOL int32 grid z, with a committed
// one-hot selector S:
//   BIN     0 = sum eq(u_bin) S (S - 1), the verifier requiring U_f2 == S_f2 - 1;
//   SUM     1 = sum [bcast(eq(u_s)) . AL] S,   MASK  0 = sum [bcast(eq(u_m)) . (1 - AL)] S;
//   ATT     mx~(u_a) = sum bcast(eq(u_a)) S z (attainment);
//   DOM     Df = AL (bcast(mx) - z) >= 0: c1 and c2 (the weight eq(u_r) . AL on z and on the never-committed broadcast of mx, the
//           latter terminal opened against com_mx at the row bits), the NPL limb planes of L opened at (u_r, plane bit), the
//           identity c2 - c1 == v0 [+ LEN_R v1] and the range lookup of the limbs;
//   T-BIND  (vpad with target columns t*) 1 = sum W_t S, W_t[i, t*[i]] = eq(u_t)[i].
// The constant claims (0, 1, 0, 1) are protocol constants: imposed by the verifier, required of the files, never absorbed.
// The allowed set AL is public: causal (j <= i, B == NCOL, V = 0) or vpad (j < V).
//
//   zkob_rowmax prove  <obdir> <seed> <z-int32.bin> <B> <NCOL> <MODE> <V> <LEN_R> <NPL> <gen_grid.bin> <gen_mx.bin> <q.bin>
//                      [mx-int32-out.bin|-] [tstar-int32.bin] [--claims <accdir> <obid>]
//   zkob_rowmax verify <obdir> <seed> <B> <NCOL> <MODE> <V> <LEN_R> <NPL> <gen_grid.bin> <gen_mx.bin> <q.bin> [tstar-int32.bin]
//                      [--claims <vaccdir> <obid>]
//   zkob_rowmax serve
//
// Files in <obdir> (byte for byte the reference's): dims.bin, com_{z,S,mx,L,m_L,A_L}.bin, lookup_L.bin, hp_{bin,sum,mask,att,c1,c2}.bin
// [hp_tbind.bin], lvals.bin and 12 to 14 openings ipa_*.bin.  Exit 0 = success / ACCEPT, 1 = REJECT, anything else = failure.
#include "zkob_common.hpp"

#include <climits>

using namespace zkob;

namespace {

struct Lay { uint32_t B, NCOL, MODE, V, LEN_R, NPL, D, DL, logB, logC, logD, logDL, logN, n1; };
uint32_t parse_mode(const char* s) {
    if (!strcmp(s, "causal")) return 0;
    if (!strcmp(s, "vpad")) return 1;
    throw std::runtime_error("MODE must be 'causal' or 'vpad'");
}
Lay lay_of(const char* b, const char* ncol, const char* mode, const char* v, const char* lenr, const char* npl) {
    Lay y;
    y.B = (uint32_t)strtoul(b, nullptr, 10); y.NCOL = (uint32_t)strtoul(ncol, nullptr, 10); y.MODE = parse_mode(mode);
    y.V = (uint32_t)strtoul(v, nullptr, 10); y.LEN_R = (uint32_t)strtoul(lenr, nullptr, 10); y.NPL = (uint32_t)strtoul(npl, nullptr, 10);
    if (!y.B || !y.NCOL || !y.LEN_R) throw std::runtime_error("bad dimensions");
    y.D = y.B * y.NCOL; y.DL = y.NPL * y.D;
    y.logB = clog2(y.B); y.logC = clog2(y.NCOL); y.logD = y.logB + y.logC; y.logDL = y.logD + (y.NPL == 2 ? 1 : 0);
    y.logN = clog2(y.LEN_R); y.n1 = y.logDL >= y.logN ? y.logDL - y.logN : 0;
    return y;
}
std::string layout_error(const Lay& y, size_t gen, size_t genmx) {
    if (y.B != (1u << y.logB)) return "B not a power of two";
    if (y.NCOL != (1u << y.logC)) return "NCOL not a power of two";
    if (y.LEN_R != (1u << y.logN)) return "LEN_R not a power of two";
    if (y.NPL != 1 && y.NPL != 2) return "NPL must be 1 or 2";
    if (y.MODE == 0) {
        if (y.B != y.NCOL) return "causal requires B == NCOL";
        if (y.V != 0) return "causal requires V == 0";
    } else if (y.V == 0 || y.V > y.NCOL) {
        return "vpad requires 0 < V <= NCOL";
    }
    if (gen != (size_t)y.NCOL * G1B) return "gen_grid size != NCOL";
    if (genmx != (size_t)y.B * G1B) return "gen_mx size != B";
    const uint64_t DL = (uint64_t)y.NPL * y.B * y.NCOL;
    if (y.NCOL > y.LEN_R || y.LEN_R > DL || DL % y.LEN_R) return "limb lookup layout needs NCOL <= LEN_R <= NPL*D, LEN_R | NPL*D";
    return "";
}
std::string tstar_error(const Lay& y, const std::vector<int32_t>* t) {
    if (!t) return "";
    if (y.MODE == 0) return "t* supplied in causal mode";
    if (t->size() != y.B) return "t* size != B";
    for (int32_t v : *t) if (v < 0 || (uint32_t)v >= y.V) return "t* token out of [0, V)";
    return "";
}
bool allowed(const Lay& y, uint32_t i, uint32_t j) { return y.MODE == 0 ? j <= i : j < y.V; }
void absorb_head(Transcript& tr, const Lay& y, const std::vector<int32_t>* tstar) {
    tr.absorb_u32("B", y.B); tr.absorb_u32("NCOL", y.NCOL); tr.absorb_u32("MODE", y.MODE); tr.absorb_u32("V", y.V);
    tr.absorb_u32("LEN_R", y.LEN_R); tr.absorb_u32("NPL", y.NPL);
    if (y.MODE == 1 && tstar) tr.absorb("TSTAR", tstar->data(), (size_t)y.B * 4);
}
// bcast_rows(eq(u)) restricted to the allowed set (sel = 1), to its complement (sel = 0), or unrestricted (sel = 2)
void row_weights(Ctx& x, const std::vector<Fr>& u, const Lay& y, int sel, Dev& out) {
    Dev e(x, (size_t)y.B * FRB);
    x.ck(zkh_fr_eq_build(x.c, u.data(), y.logB, e.p), "eq table");
    const std::vector<uint8_t> raw = e.host();
    std::vector<Fr> w((size_t)y.D, fr_u32(0));
    for (uint32_t i = 0; i < y.B; i++) {
        Fr v;
        memcpy(v.v, &raw[(size_t)i * FRB], FRB);
        for (uint32_t j = 0; j < y.NCOL; j++)
            if (sel == 2 || (int)allowed(y, i, j) == sel) w[(size_t)i * y.NCOL + j] = v;
    }
    x.ck(zkh_upload(x.c, out.p, w.data(), w.size() * FRB), "upload");
}
// W_t[i, t*[i]] = eq(u_t)[i]
void tbind_weights(Ctx& x, const std::vector<Fr>& u, const Lay& y, const std::vector<int32_t>& tstar, Dev& out) {
    Dev e(x, (size_t)y.B * FRB);
    x.ck(zkh_fr_eq_build(x.c, u.data(), y.logB, e.p), "eq table");
    const std::vector<uint8_t> raw = e.host();
    std::vector<Fr> w((size_t)y.D, fr_u32(0));
    for (uint32_t i = 0; i < y.B; i++) memcpy(w[(size_t)i * y.NCOL + (uint32_t)tstar[i]].v, &raw[(size_t)i * FRB], FRB);
    x.ck(zkh_upload(x.c, out.p, w.data(), w.size() * FRB), "upload");
}
std::vector<Fr> mask_grid(const Lay& y) {
    std::vector<Fr> m((size_t)y.D, fr_u32(0));
    for (uint32_t i = 0; i < y.B; i++)
        for (uint32_t j = 0; j < y.NCOL; j++)
            if (allowed(y, i, j)) m[(size_t)i * y.NCOL + j] = fr_u32(1);
    return m;
}
std::vector<Fr> plane_point(const std::vector<Fr>& u_r, uint32_t p) {
    std::vector<Fr> pt(u_r);
    pt.push_back(fr_u32(p));
    return pt;
}

struct Had { Fr claim, S_f2, U_f2; std::vector<Fr> ws; };
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
    if (argc < 14 || argc > 16)
        throw std::invalid_argument("prove <obdir> <seed> <z-int32> <B> <NCOL> <MODE> <V> <LEN_R> <NPL> <gen_grid> <gen_mx> <q.bin> [mx-int32-out|-] [tstar-int32]");
    const std::string obdir = argv[2], seed = argv[3];
    const Lay y = lay_of(argv[5], argv[6], argv[7], argv[8], argv[9], argv[10]);
    const uint32_t B = y.B, NCOL = y.NCOL, D = y.D, DL = y.DL, LEN_R = y.LEN_R, NPL = y.NPL;
    const size_t cols_in = y.MODE == 1 ? (size_t)y.V : (size_t)NCOL;
    const std::vector<int32_t> zin = load_ints(argv[4], (size_t)B * cols_in);
    const std::vector<uint8_t> gen = read_file(argv[11]), genmx = read_file(argv[12]), q = read_file(argv[13]);
    if (q.size() < G1B) throw std::runtime_error("q.bin holds no point");
    std::string mx_out = argc >= 15 ? argv[14] : "";
    if (mx_out == "-") mx_out = "";
    std::vector<int32_t> tst;
    if (argc == 16) tst = load_ints(argv[15], B);
    const std::vector<int32_t>* tstar = argc == 16 ? &tst : nullptr;
    std::string le = layout_error(y, gen.size(), genmx.size());
    if (le.empty()) le = tstar_error(y, tstar);
    if (!le.empty()) throw std::runtime_error(le);
    const int64_t LIMIT = NPL == 1 ? (int64_t)LEN_R : (int64_t)LEN_R * (int64_t)LEN_R;

    // the host chain: the padded grid, the row maxima with the lowest attaining column, the one-hot selector, the limbs of Df
    std::vector<int64_t> zh((size_t)D, 0), mxh(B), Sh((size_t)D, 0), Uh((size_t)D), Lh((size_t)DL, 0), mxbh((size_t)D), cnt(LEN_R, 0);
    for (uint32_t i = 0; i < B; i++)
        for (uint32_t j = 0; j < cols_in; j++) {
            const int64_t v = zin[(size_t)i * cols_in + j];
            if (y.MODE == 1 && std::llabs(v) >= (1LL << 25)) throw std::runtime_error("vpad |z| >= 2^25 (envelope guard)");
            zh[(size_t)i * NCOL + j] = v;
        }
    for (uint32_t i = 0; i < B; i++) {
        int64_t best = LLONG_MIN;
        uint32_t bj = 0;
        for (uint32_t j = 0; j < NCOL; j++)
            if (allowed(y, i, j) && zh[(size_t)i * NCOL + j] > best) { best = zh[(size_t)i * NCOL + j]; bj = j; }
        mxh[i] = best;
        Sh[(size_t)i * NCOL + bj] = 1;
    }
    for (size_t k = 0; k < D; k++) Uh[k] = Sh[k] - 1;
    for (uint32_t i = 0; i < B; i++)
        for (uint32_t j = 0; j < NCOL; j++) {
            const size_t idx = (size_t)i * NCOL + j;
            mxbh[idx] = mxh[i];
            if (!allowed(y, i, j)) continue;
            const int64_t df = mxh[i] - zh[idx];
            if (df < 0) throw std::runtime_error("Df < 0 (witness bug)");
            if (df >= LIMIT) throw std::runtime_error("allowed Df >= LEN_R^NPL");
            if (NPL == 1) Lh[idx] = df;
            else { Lh[idx] = df % LEN_R; Lh[(size_t)D + idx] = df / LEN_R; }
        }
    for (size_t k = 0; k < DL; k++) cnt[(size_t)Lh[k]]++;
    if (!mx_out.empty()) {                                          // the chain file: B int32
        std::vector<int32_t> mi(mxh.begin(), mxh.end());
        std::vector<uint8_t> b((size_t)B * 4);
        memcpy(b.data(), mi.data(), b.size());
        write_file(mx_out, b);
    }
    std::vector<int64_t> tab(LEN_R);
    for (uint32_t i = 0; i < LEN_R; i++) tab[i] = i;

    Ctx x;
    Dev gd(x, gen.data(), gen.size()), gmx(x, genmx.data(), genmx.size());
    const std::vector<Fr> zf = lift(zh), Sf = lift(Sh), Uf = lift(Uh), mxf = lift(mxh), mxbf = lift(mxbh), Lf = lift(Lh), mLf = lift(cnt), Tp = lift(tab),
                          ALf = mask_grid(y), ones((size_t)D, fr_u32(1)), none;
    Dev dz(x, zf.data(), zf.size() * FRB), dS(x, Sf.data(), Sf.size() * FRB), dU(x, Uf.data(), Uf.size() * FRB), dmx(x, mxf.data(), mxf.size() * FRB),
        dmxb(x, mxbf.data(), mxbf.size() * FRB), dL(x, Lf.data(), Lf.size() * FRB), dmL(x, mLf.data(), mLf.size() * FRB), dTab(x, Tp.data(), Tp.size() * FRB),
        dAL(x, ALf.data(), ALf.size() * FRB), dOnes(x, ones.data(), ones.size() * FRB);
    const std::vector<uint8_t> comz = commit_rows(x, gd, dz, B, NCOL), comS = commit_rows(x, gd, dS, B, NCOL), commx = commit_rows(x, gmx, dmx, 1, B),
                               comL = commit_rows(x, gd, dL, NPL * B, NCOL), commL = commit_rows(x, gd, dmL, LEN_R / NCOL, NCOL);
    write_file(obdir + "/com_z.bin", comz); write_file(obdir + "/com_S.bin", comS); write_file(obdir + "/com_mx.bin", commx);
    write_file(obdir + "/com_L.bin", comL); write_file(obdir + "/com_m_L.bin", commL);
    { std::vector<uint8_t> f; const uint32_t dm[6] = {B, NCOL, y.MODE, y.V, LEN_R, NPL}; put(f, dm, 24); write_file(obdir + "/dims.bin", f); }

    Transcript tr(seed);
    absorb_head(tr, y, tstar);
    tr.absorb("com_z", comz.data(), comz.size()); tr.absorb("com_S", comS.data(), comS.size()); tr.absorb("com_mx", commx.data(), commx.size());
    tr.absorb("com_L", comL.data(), comL.size()); tr.absorb("com_m_L", commL.data(), commL.size());
    auto claim = [&](const char* tensor, const std::string& comref, uint32_t domain, uint32_t rows, const std::vector<Fr>& pt, const Fr& eval) {
        claim_emit(cf.accdir, make_claim(cf.obid, tensor, comref, domain, rows, pt, none, eval));
    };
    auto wref = [&](const char* tag, const std::string& comref, const std::vector<uint8_t>& scalars) {
        const std::string wit = cf.accdir + "/wit_" + cf.obid + "_" + tag + ".fr";
        write_file(wit, scalars);
        witref_emit(cf.accdir, comref, wit);
    };
    const uint8_t* Q = q.data();
    const std::string cS = obdir + "/com_S.bin", cz = obdir + "/com_z.bin", cmx = obdir + "/com_mx.bin", cL = obdir + "/com_L.bin";
    // the limb range lookup
    {
        const Fr beta = tr.challenge_fr();
        Dev dA(x, (size_t)DL * FRB), dBv(x, (size_t)LEN_R * FRB);
        x.ck(zkh_fr_inv_add(x.c, dL.p, DL, beta.v, dA.p), "A = 1 / (L + beta)");
        const std::vector<uint8_t> comA = commit_rows(x, gd, dA, NPL * B, NCOL);
        write_file(obdir + "/com_A_L.bin", comA);
        tr.absorb("com_A_L", comA.data(), comA.size());
        const Fr alpha = tr.challenge_fr();
        const std::vector<Fr> u = tr.challenge_vec(y.logDL);
        x.ck(zkh_fr_inv_add(x.c, dTab.p, LEN_R, beta.v, dBv.p), "B = 1 / (T + beta)");
        Fr bm;
        x.ck(zkh_fr_dot(x.c, dBv.p, dmL.p, LEN_R, bm.v), "sum B m");
        const Fr Cc = fr_sub(fr_mul(alpha, alpha), bm);
        std::vector<Fr> ev((size_t)4 * y.logDL), ws(y.logDL);
        Fr term[5];
        x.ck(zkh_fr_lookup_sumcheck(x.c, dA.p, dL.p, dBv.p, dTab.p, dmL.p, y.logDL, y.logN, alpha.v, beta.v, Cc.v, u.data(), tr.st, ev.data(), ws.data(), term),
             "limb lookup sumcheck");
        {
            std::vector<uint8_t> f;
            const uint32_t n = 4 * y.logDL;
            put(f, &n, 4); put(f, ev.data(), ev.size() * FRB); put(f, term[0].v, FRB); put(f, term[1].v, FRB); put(f, term[4].v, FRB);
            write_file(obdir + "/lookup_L.bin", f);
        }
        tr.absorb_fr("A_f", term[0]); tr.absorb_fr("S_f", term[1]); tr.absorb_fr("m_f", term[4]);
        const std::vector<Fr> u_pt(ws.rbegin(), ws.rend()), u_m(ws.rbegin(), ws.rend() - y.n1);
        if (cf.on()) {
            claim("A_L", obdir + "/com_A_L.bin", NCOL, NPL * B, u_pt, term[0]);
            wref("A_L", obdir + "/com_A_L.bin", dA.host());
            claim("L_lk", cL, NCOL, NPL * B, u_pt, term[1]);
            wref("L", cL, dL.host());
            claim("m_L", obdir + "/com_m_L.bin", NCOL, LEN_R / NCOL, u_m, term[4]);
            wref("m_L", obdir + "/com_m_L.bin", dmL.host());
        } else {
            open_prove(x, dA, NPL * B, NCOL, gd, Q, u_pt, obdir + "/ipa_A_L.bin", tr);
            open_prove(x, dL, NPL * B, NCOL, gd, Q, u_pt, obdir + "/ipa_L_lk.bin", tr);
            open_prove(x, dmL, LEN_R / NCOL, NCOL, gd, Q, u_m, obdir + "/ipa_m_L.bin", tr);
        }
    }
    Dev dW(x, (size_t)D * FRB);
    const Fr zero = fr_u32(0), one = fr_u32(1);
    {   // BIN
        const std::vector<Fr> u_bin = tr.challenge_vec(y.logD);
        x.ck(zkh_fr_eq_build(x.c, u_bin.data(), y.logD, dW.p), "eq table");
        const Had h = hadamard(x, tr, zero, dW, dS, dU, y.logD, obdir + "/hp_bin.bin");
        const std::vector<Fr> pt(h.ws.rbegin(), h.ws.rend());
        if (cf.on()) { claim("S_bin", cS, NCOL, B, pt, h.S_f2); wref("S", cS, dS.host()); }
        else open_prove(x, dS, B, NCOL, gd, Q, pt, obdir + "/ipa_S_bin.bin", tr);
    }
    {   // SUM
        const std::vector<Fr> u_s = tr.challenge_vec(y.logB);
        row_weights(x, u_s, y, 1, dW);
        const Had h = hadamard(x, tr, one, dW, dS, dOnes, y.logD, obdir + "/hp_sum.bin");
        const std::vector<Fr> pt(h.ws.rbegin(), h.ws.rend());
        if (cf.on()) claim("S_sum", cS, NCOL, B, pt, h.S_f2);
        else open_prove(x, dS, B, NCOL, gd, Q, pt, obdir + "/ipa_S_sum.bin", tr);
    }
    {   // MASK
        const std::vector<Fr> u_m = tr.challenge_vec(y.logB);
        row_weights(x, u_m, y, 0, dW);
        const Had h = hadamard(x, tr, zero, dW, dS, dOnes, y.logD, obdir + "/hp_mask.bin");
        const std::vector<Fr> pt(h.ws.rbegin(), h.ws.rend());
        if (cf.on()) claim("S_mask", cS, NCOL, B, pt, h.S_f2);
        else open_prove(x, dS, B, NCOL, gd, Q, pt, obdir + "/ipa_S_mask.bin", tr);
    }
    {   // ATT
        const std::vector<Fr> u_a = tr.challenge_vec(y.logB);
        Fr ev_mx;
        x.ck(zkh_fr_mle_eval(x.c, dmx.p, u_a.data(), y.logB, ev_mx.v), "ev_mx");
        tr.absorb_fr("ev_mx", ev_mx);
        row_weights(x, u_a, y, 2, dW);
        const Had h = hadamard(x, tr, ev_mx, dW, dS, dz, y.logD, obdir + "/hp_att.bin");
        const std::vector<Fr> pt(h.ws.rbegin(), h.ws.rend());
        if (cf.on()) {
            claim("S_att", cS, NCOL, B, pt, h.S_f2);
            claim("z_att", cz, NCOL, B, pt, h.U_f2);
            wref("z", cz, dz.host());
            claim("mx_att", cmx, B, 1, u_a, ev_mx);
            wref("mx", cmx, dmx.host());
        } else {
            open_prove(x, dS, B, NCOL, gd, Q, pt, obdir + "/ipa_S_att.bin", tr);
            open_prove(x, dz, B, NCOL, gd, Q, pt, obdir + "/ipa_z_att.bin", tr);
            open_prove(x, dmx, 1, B, gmx, Q, u_a, obdir + "/ipa_mx_att.bin", tr);
        }
    }
    // DOM: c1 on z, c2 on the broadcast of mx, both with the weight eq(u_r) . AL
    const std::vector<Fr> u_r = tr.challenge_vec(y.logD);
    x.ck(zkh_fr_eq_build(x.c, u_r.data(), y.logD, dW.p), "eq table");
    x.ck(zkh_fr_mul(x.c, dW.p, dW.p, dAL.p, D), "eq .* AL");
    {
        Fr c1;
        x.ck(zkh_fr_dot(x.c, dW.p, dz.p, D, c1.v), "c1");
        tr.absorb_fr("c1", c1);
        const Had h = hadamard(x, tr, c1, dW, dz, dOnes, y.logD, obdir + "/hp_c1.bin");
        const std::vector<Fr> pt(h.ws.rbegin(), h.ws.rend());
        if (cf.on()) claim("z_c1", cz, NCOL, B, pt, h.S_f2);
        else open_prove(x, dz, B, NCOL, gd, Q, pt, obdir + "/ipa_z_c1.bin", tr);
    }
    {
        Fr c2;
        x.ck(zkh_fr_dot(x.c, dW.p, dmxb.p, D, c2.v), "c2");
        tr.absorb_fr("c2", c2);
        const Had h = hadamard(x, tr, c2, dW, dmxb, dOnes, y.logD, obdir + "/hp_c2.bin");
        const std::vector<Fr> pt(h.ws.rbegin(), h.ws.rend()), pt_rows(pt.begin() + y.logC, pt.end());
        if (cf.on()) claim("mx_c2", cmx, B, 1, pt_rows, h.S_f2);
        else open_prove(x, dmx, 1, B, gmx, Q, pt_rows, obdir + "/ipa_mx_c2.bin", tr);
    }
    {   // the limb planes at (u_r [, plane bit])
        Fr lv[2] = {zero, zero};
        for (uint32_t p = 0; p < NPL; p++) {
            const std::vector<Fr> pt = NPL == 1 ? u_r : plane_point(u_r, p);
            x.ck(zkh_fr_mle_eval(x.c, dL.p, pt.data(), y.logDL, lv[p].v), "plane evaluation");
            tr.absorb_fr(p ? "v1" : "v0", lv[p]);
        }
        { std::vector<uint8_t> f; put(f, lv, (size_t)NPL * FRB); write_file(obdir + "/lvals.bin", f); }
        for (uint32_t p = 0; p < NPL; p++) {
            const std::vector<Fr> pt = NPL == 1 ? u_r : plane_point(u_r, p);
            if (cf.on()) claim(p ? "L_p1" : "L_p0", cL, NCOL, NPL * B, pt, lv[p]);
            else open_prove(x, dL, NPL * B, NCOL, gd, Q, pt, obdir + (p ? "/ipa_L_p1.bin" : "/ipa_L_p0.bin"), tr);
        }
    }
    if (y.MODE == 1 && tstar) {                                     // T-BIND
        const std::vector<Fr> u_t = tr.challenge_vec(y.logB);
        tbind_weights(x, u_t, y, *tstar, dW);
        const Had h = hadamard(x, tr, one, dW, dS, dOnes, y.logD, obdir + "/hp_tbind.bin");
        const std::vector<Fr> pt(h.ws.rbegin(), h.ws.rend());
        if (cf.on()) claim("S_tbind", cS, NCOL, B, pt, h.S_f2);
        else open_prove(x, dS, B, NCOL, gd, Q, pt, obdir + "/ipa_S_tbind.bin", tr);
    }
    if (cf.on()) {
        drvstate_emit(cf.accdir, cf.obid, tr.st);
        std::cout << "PROVED rowmax obligation (claim mode) -> " << obdir << std::endl;
        return 0;
    }
    std::cout << "PROVED rowmax obligation -> " << obdir << std::endl;
    return 0;
}

// the round checks of one Hadamard sumcheck from the claim `cur`; ws the challenges; eq_acc the product of eq(u[nu - 1 - k], w_k) over
// the first nu rounds when u is given
bool hadamard_rounds(Transcript& tr, const Hp& hp, uint32_t logn, const char* tag, const Fr& inv2, const Fr& inv6, std::vector<Fr>& ws, Fr& cur,
                     const std::vector<Fr>* u = nullptr, Fr* eq_acc = nullptr) {
    for (uint32_t k = 0; k < logn; k++) {
        const std::array<Fr, 4> e = {hp.ev[4 * k], hp.ev[4 * k + 1], hp.ev[4 * k + 2], hp.ev[4 * k + 3]};
        if (!fr_eq(cur, fr_add(e[0], e[1]))) return rj(std::string(tag) + " round " + std::to_string(k) + " p(0)+p(1) != claim");
        tr.absorb_fr("hp0", e[0]); tr.absorb_fr("hp1", e[1]); tr.absorb_fr("hp2", e[2]); tr.absorb_fr("hp3", e[3]);
        const Fr w = tr.challenge_fr();
        ws.push_back(w);
        cur = lagrange4(e, w, inv6, inv2);
        if (u && k < u->size()) *eq_acc = fr_mul(*eq_acc, eq1((*u)[u->size() - 1 - k], w));
    }
    return true;
}

bool verify(Ctx& x, const std::string& obdir, const std::string& seed, const Lay& y, const std::vector<uint8_t>& gen, const std::vector<uint8_t>& genmx,
            const std::vector<uint8_t>& q, const std::vector<int32_t>* tstar, const ClaimFlags& cf) {
    if (!layout_error(y, gen.size(), genmx.size()).empty()) return rj("bad layout params");
    { const std::string te = tstar_error(y, tstar); if (!te.empty()) return rj(te); }
    const uint32_t B = y.B, NCOL = y.NCOL, D = y.D, LEN_R = y.LEN_R, NPL = y.NPL, logD = y.logD, logB = y.logB;
    {
        const std::vector<uint8_t> f = read_file(obdir + "/dims.bin");
        if (f.size() < 24) return rj("dims.bin short read");
        uint32_t dm[6];
        memcpy(dm, f.data(), 24);
        if (dm[0] != B || dm[1] != NCOL || dm[2] != y.MODE || dm[3] != y.V || dm[4] != LEN_R || dm[5] != NPL) return rj("dims.bin mismatch");
    }
    const std::vector<uint8_t> comz = read_file(obdir + "/com_z.bin"), comS = read_file(obdir + "/com_S.bin"), commx = read_file(obdir + "/com_mx.bin"),
                               comL = read_file(obdir + "/com_L.bin"), commL = read_file(obdir + "/com_m_L.bin"), comAL = read_file(obdir + "/com_A_L.bin");
    const size_t rB = (size_t)B * G1B;
    if (comz.size() != rB || comS.size() != rB || commx.size() != G1B || comL.size() != NPL * rB || comAL.size() != NPL * rB ||
        commL.size() != (size_t)(LEN_R / NCOL) * G1B)
        return rj("commitment row counts");
    std::vector<Fr> lev;
    Fr A_f, S_f, m_f;
    {
        const std::vector<uint8_t> f = read_file(obdir + "/lookup_L.bin");
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
    const bool tb = y.MODE == 1 && tstar;
    Hp hp_bin, hp_sum, hp_mask, hp_att, hp_c1, hp_c2, hp_tb;
    if (!read_hp(obdir + "/hp_bin.bin", 4 * logD, hp_bin) || !read_hp(obdir + "/hp_sum.bin", 4 * logD, hp_sum) || !read_hp(obdir + "/hp_mask.bin", 4 * logD, hp_mask) ||
        !read_hp(obdir + "/hp_att.bin", 4 * logD, hp_att) || !read_hp(obdir + "/hp_c1.bin", 4 * logD, hp_c1) || !read_hp(obdir + "/hp_c2.bin", 4 * logD, hp_c2) ||
        (tb && !read_hp(obdir + "/hp_tbind.bin", 4 * logD, hp_tb)))
        return rj("hadamard round count");
    Fr lv[2] = {fr_u32(0), fr_u32(0)};
    {
        const std::vector<uint8_t> f = read_file(obdir + "/lvals.bin");
        if (f.size() < (size_t)NPL * FRB) return rj("lvals.bin short read");
        memcpy(lv, f.data(), (size_t)NPL * FRB);
        for (uint32_t p = 0; p < NPL; p++) if (!fr_lt(lv[p], FR_MOD)) return rj("non-canonical lvals");
    }
    const Fr zero = fr_u32(0), one = fr_u32(1);
    if (!fr_eq(hp_bin.claim, zero)) return rj("BIN claim_H != protocol constant 0");
    if (!fr_eq(hp_sum.claim, one)) return rj("SUM claim_H != protocol constant 1");
    if (!fr_eq(hp_mask.claim, zero)) return rj("MASK claim_H != protocol constant 0");
    if (tb && !fr_eq(hp_tb.claim, one)) return rj("T-BIND claim_H != protocol constant 1");
    Laps laps("rowmax_verify");
    const std::vector<Fr> ALf = mask_grid(y), none;
    Dev dAL(x, ALf.data(), ALf.size() * FRB), gd(x, gen.data(), gen.size()), gmx(x, genmx.data(), genmx.size()), dW(x, (size_t)D * FRB);
    const uint8_t* Q = q.data();
    const Fr inv2 = fr_inv(fr_u32(2)), inv6 = fr_inv(fr_u32(6));

    Transcript tr(seed);
    absorb_head(tr, y, tstar);
    tr.absorb("com_z", comz.data(), comz.size()); tr.absorb("com_S", comS.data(), comS.size()); tr.absorb("com_mx", commx.data(), commx.size());
    tr.absorb("com_L", comL.data(), comL.size()); tr.absorb("com_m_L", commL.data(), commL.size());
    const Fr beta = tr.challenge_fr();
    tr.absorb("com_A_L", comAL.data(), comAL.size());
    const Fr alpha = tr.challenge_fr();
    const std::vector<Fr> u_L = tr.challenge_vec(y.logDL);
    std::vector<Fr> wsl;
    {
        std::vector<int64_t> tab(LEN_R);
        for (uint32_t i = 0; i < LEN_R; i++) tab[i] = i;
        const std::vector<Fr> Tp = lift(tab);
        Dev td(x, Tp.data(), Tp.size() * FRB);
        if (!lookup_verify(x, tr, lev, A_f, S_f, m_f, alpha, beta, u_L, td, y.logDL, y.logN, wsl, laps, "limb lookup")) return false;
    }
    tr.absorb_fr("A_f", A_f); tr.absorb_fr("S_f", S_f); tr.absorb_fr("m_f", m_f);
    const std::vector<Fr> u_ptL(wsl.rbegin(), wsl.rend()), u_mL(wsl.rbegin(), wsl.rend() - y.n1);
    if (!cf.on()) {
        if (!open_check(x, comAL, NCOL, gd, Q, u_ptL, A_f, obdir + "/ipa_A_L.bin", tr)) return rj("IPA opening of A_f vs com_A_L");
        if (!open_check(x, comL, NCOL, gd, Q, u_ptL, S_f, obdir + "/ipa_L_lk.bin", tr)) return rj("IPA opening of S_f vs com_L");
        if (!open_check(x, commL, NCOL, gd, Q, u_mL, m_f, obdir + "/ipa_m_L.bin", tr)) return rj("IPA opening of m_f vs com_m_L");
    }
    std::vector<Fr> ws_bin, ws_sum, ws_mask, ws_att, ws_c1, ws_c2, ws_tb;
    Fr cur;
    // BIN: the eq product over every round; U is bound to com_S only through U_f2 == S_f2 - 1
    const std::vector<Fr> u_bin = tr.challenge_vec(logD);
    {
        Fr eq_acc = one;
        cur = zero;
        if (!hadamard_rounds(tr, hp_bin, logD, "BIN", inv2, inv6, ws_bin, cur, &u_bin, &eq_acc)) return false;
        if (!fr_eq(hp_bin.U_f2, fr_sub(hp_bin.S_f2, one))) return rj("BIN U_f2 != S_f2 - 1");
        if (!fr_eq(cur, fr_mul(eq_acc, fr_mul(hp_bin.S_f2, hp_bin.U_f2)))) return rj("BIN terminal identity");
    }
    tr.absorb_fr("S_f2", hp_bin.S_f2); tr.absorb_fr("U_f2", hp_bin.U_f2);
    const std::vector<Fr> pt_bin(ws_bin.rbegin(), ws_bin.rend());
    if (!cf.on() && !open_check(x, comS, NCOL, gd, Q, pt_bin, hp_bin.S_f2, obdir + "/ipa_S_bin.bin", tr)) return rj("IPA opening of S (BIN) vs com_S");
    // SUM, MASK (and T-BIND below): a constant claim, U_f2 == 1, the verifier's own weights folded
    auto weighted_leg = [&](const Hp& hp, const Fr& start, const char* tag, std::vector<Fr>& ws) {
        cur = start;
        if (!hadamard_rounds(tr, hp, logD, tag, inv2, inv6, ws, cur)) return false;
        if (!fr_eq(hp.U_f2, one)) return rj(std::string(tag) + " U_f2 != 1");
        const Fr W_f = fold_public(x, dW, D, ws);
        if (!fr_eq(cur, fr_mul(W_f, fr_mul(hp.S_f2, hp.U_f2)))) return rj(std::string(tag) + " terminal identity");
        tr.absorb_fr("S_f2", hp.S_f2); tr.absorb_fr("U_f2", hp.U_f2);
        return true;
    };
    const std::vector<Fr> u_s = tr.challenge_vec(logB);
    row_weights(x, u_s, y, 1, dW);
    if (!weighted_leg(hp_sum, one, "SUM", ws_sum)) return false;
    const std::vector<Fr> pt_s(ws_sum.rbegin(), ws_sum.rend());
    if (!cf.on() && !open_check(x, comS, NCOL, gd, Q, pt_s, hp_sum.S_f2, obdir + "/ipa_S_sum.bin", tr)) return rj("IPA opening of S (SUM) vs com_S");
    const std::vector<Fr> u_m = tr.challenge_vec(logB);
    row_weights(x, u_m, y, 0, dW);
    if (!weighted_leg(hp_mask, zero, "MASK", ws_mask)) return false;
    const std::vector<Fr> pt_m(ws_mask.rbegin(), ws_mask.rend());
    if (!cf.on() && !open_check(x, comS, NCOL, gd, Q, pt_m, hp_mask.S_f2, obdir + "/ipa_S_mask.bin", tr)) return rj("IPA opening of S (MASK) vs com_S");
    // ATT: a pure row-broadcast weight, the eq product over the row rounds (the row bits are the high bits)
    const std::vector<Fr> u_a = tr.challenge_vec(logB);
    tr.absorb_fr("ev_mx", hp_att.claim);
    {
        Fr eq_acc = one;
        cur = hp_att.claim;
        if (!hadamard_rounds(tr, hp_att, logD, "ATT", inv2, inv6, ws_att, cur, &u_a, &eq_acc)) return false;
        if (!fr_eq(cur, fr_mul(eq_acc, fr_mul(hp_att.S_f2, hp_att.U_f2)))) return rj("ATT terminal identity");
    }
    tr.absorb_fr("S_f2", hp_att.S_f2); tr.absorb_fr("U_f2", hp_att.U_f2);
    const std::vector<Fr> pt_a(ws_att.rbegin(), ws_att.rend());
    if (!cf.on()) {
        if (!open_check(x, comS, NCOL, gd, Q, pt_a, hp_att.S_f2, obdir + "/ipa_S_att.bin", tr)) return rj("IPA opening of S (ATT) vs com_S");
        if (!open_check(x, comz, NCOL, gd, Q, pt_a, hp_att.U_f2, obdir + "/ipa_z_att.bin", tr)) return rj("IPA opening of z (ATT) vs com_z");
        if (!open_check(x, commx, B, gmx, Q, u_a, hp_att.claim, obdir + "/ipa_mx_att.bin", tr)) return rj("IPA opening of ev_mx vs com_mx");
    }
    // DOM: c1 and c2 with the weight eq(u_r) . AL
    const std::vector<Fr> u_r = tr.challenge_vec(logD);
    auto masked_weight = [&]() {
        x.ck(zkh_fr_eq_build(x.c, u_r.data(), logD, dW.p), "eq table");
        x.ck(zkh_fr_mul(x.c, dW.p, dW.p, dAL.p, D), "eq .* AL");
    };
    tr.absorb_fr("c1", hp_c1.claim);
    masked_weight();
    if (!weighted_leg(hp_c1, hp_c1.claim, "c1", ws_c1)) return false;
    const std::vector<Fr> pt_c1(ws_c1.rbegin(), ws_c1.rend());
    if (!cf.on() && !open_check(x, comz, NCOL, gd, Q, pt_c1, hp_c1.S_f2, obdir + "/ipa_z_c1.bin", tr)) return rj("IPA opening of z (c1) vs com_z");
    tr.absorb_fr("c2", hp_c2.claim);
    masked_weight();
    if (!weighted_leg(hp_c2, hp_c2.claim, "c2", ws_c2)) return false;
    const std::vector<Fr> pt_c2(ws_c2.rbegin(), ws_c2.rend()), pt_c2_rows(pt_c2.begin() + y.logC, pt_c2.end());
    if (!cf.on() && !open_check(x, commx, B, gmx, Q, pt_c2_rows, hp_c2.S_f2, obdir + "/ipa_mx_c2.bin", tr)) return rj("IPA opening of c2 terminal vs com_mx");
    // the limb planes
    for (uint32_t p = 0; p < NPL; p++) tr.absorb_fr(p ? "v1" : "v0", lv[p]);
    if (!cf.on())
        for (uint32_t p = 0; p < NPL; p++)
            if (!open_check(x, comL, NCOL, gd, Q, NPL == 1 ? u_r : plane_point(u_r, p), lv[p], obdir + (p ? "/ipa_L_p1.bin" : "/ipa_L_p0.bin"), tr))
                return rj("IPA opening of L plane " + std::to_string(p) + " vs com_L");
    std::vector<Fr> pt_t;
    if (tb) {
        const std::vector<Fr> u_t = tr.challenge_vec(logB);
        tbind_weights(x, u_t, y, *tstar, dW);
        if (!weighted_leg(hp_tb, one, "T-BIND", ws_tb)) return false;
        pt_t.assign(ws_tb.rbegin(), ws_tb.rend());
        if (!cf.on() && !open_check(x, comS, NCOL, gd, Q, pt_t, hp_tb.S_f2, obdir + "/ipa_S_tbind.bin", tr)) return rj("IPA opening of S (T-BIND) vs com_S");
    }
    {   // c2 - c1 == v0 [+ LEN_R v1]
        const Fr rec = NPL == 2 ? fr_add(lv[0], fr_mul(fr_u32(LEN_R), lv[1])) : lv[0];
        if (!fr_eq(fr_sub(hp_c2.claim, hp_c1.claim), rec)) return rj("DOM bracket identity");
    }
    if (cf.on()) {
        auto claim = [&](const char* tensor, const std::string& comref, uint32_t domain, uint32_t rows, const std::vector<Fr>& pt, const Fr& eval) {
            claim_emit(cf.accdir, make_claim(cf.obid, tensor, comref, domain, rows, pt, none, eval));
        };
        const std::string cS = obdir + "/com_S.bin", cz = obdir + "/com_z.bin", cmx = obdir + "/com_mx.bin", cL = obdir + "/com_L.bin";
        claim("A_L", obdir + "/com_A_L.bin", NCOL, NPL * B, u_ptL, A_f);
        claim("L_lk", cL, NCOL, NPL * B, u_ptL, S_f);
        claim("m_L", obdir + "/com_m_L.bin", NCOL, LEN_R / NCOL, u_mL, m_f);
        claim("S_bin", cS, NCOL, B, pt_bin, hp_bin.S_f2);
        claim("S_sum", cS, NCOL, B, pt_s, hp_sum.S_f2);
        claim("S_mask", cS, NCOL, B, pt_m, hp_mask.S_f2);
        claim("S_att", cS, NCOL, B, pt_a, hp_att.S_f2);
        claim("z_att", cz, NCOL, B, pt_a, hp_att.U_f2);
        claim("mx_att", cmx, B, 1, u_a, hp_att.claim);
        claim("z_c1", cz, NCOL, B, pt_c1, hp_c1.S_f2);
        claim("mx_c2", cmx, B, 1, pt_c2_rows, hp_c2.S_f2);
        for (uint32_t p = 0; p < NPL; p++) claim(p ? "L_p1" : "L_p0", cL, NCOL, NPL * B, NPL == 1 ? u_r : plane_point(u_r, p), lv[p]);
        if (tb) claim("S_tbind", cS, NCOL, B, pt_t, hp_tb.S_f2);
        drvstate_emit(cf.accdir, cf.obid, tr.st);
        std::cout << "ACCEPT-conditional (claims emitted; final verdict gated on opening_batch)" << std::endl;
        return true;
    }
    std::cout << "ACCEPT" << std::endl;
    return true;
}

int do_verify(int argc, char** argv) {
    const ClaimFlags cf = claim_flags(argc, argv);
    argc = cf.base_argc;
    if (argc != 13 && argc != 14) throw std::invalid_argument("verify <obdir> <seed> <B> <NCOL> <MODE> <V> <LEN_R> <NPL> <gen_grid> <gen_mx> <q.bin> [tstar-int32]");
    const Lay y = lay_of(argv[4], argv[5], argv[6], argv[7], argv[8], argv[9]);
    const std::vector<uint8_t> gen = read_file(argv[10]), genmx = read_file(argv[11]), q = read_file(argv[12]);
    if (q.size() < G1B) throw std::runtime_error("q.bin holds no point");
    std::vector<int32_t> tst;
    if (argc == 14) tst = load_ints(argv[13], y.B);
    const std::vector<int32_t>* tstar = argc == 14 ? &tst : nullptr;
    if (!layout_error(y, gen.size(), genmx.size()).empty()) return rj("bad layout params") ? 0 : 1;
    { const std::string te = tstar_error(y, tstar); if (!te.empty()) return rj(te) ? 0 : 1; }
    Ctx x;
    return verify(x, argv[2], argv[3], y, gen, genmx, q, tstar, cf) ? 0 : 1;
}

int run1(int argc, char** argv) {
    const std::string mode = argc > 1 ? argv[1] : "";
    try {
        if (mode == "prove") return do_prove(argc, argv);
        if (mode == "verify") return do_verify(argc, argv);
    } catch (const std::invalid_argument& e) {
        std::cerr << "zkob_rowmax: " << e.what() << std::endl;
        return 2;
    }
    std::cerr << "usage: zkob_rowmax prove ... [--claims <accdir> <obid>] | verify ... [--claims <vaccdir> <obid>] | serve" << std::endl;
    return 2;
}

}  // namespace

int main(int argc, char** argv) {
    try {
        if (argc > 1 && std::string(argv[1]) == "serve") return serve_loop(argv[0], run1);
        return run1(argc, argv);
    } catch (const std::exception& e) {
        std::cerr << "zkob_rowmax: " << e.what() << std::endl;
        return 3;
    }
}
