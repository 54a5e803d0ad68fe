// Driver for the rotary-embedding obligation (layer.attn.rope.{q,k}) of the reference's first proof stack, with the command line,
// the files and the exit codes of the reference's zkob_rope (zkllm-src/zkob_rope.cu:1-60, :146-316 prove, :323-452 verify).  For
// the chained B x C int32 tensor T on the padded B x C_pad grid it binds the exact integer relation
//   Y64[t, e] = T[t, e] W1[t, e] + T[t, e xor HD/2] W2[t, e],   W1 = cos table, W2 = +-sin table (sign from bit HD/2 of e),
// with one challenge u: ev = Y64~(u) = c1 + c2, c1 and c2 each a Hadamard sumcheck with the PUBLIC weights eq(u) .* W1 / W2, the
// tensor (or its column-flipped copy, never committed) and a column of ones.  The second terminal opens the SAME com_T at the
// point with coordinate log2(HD) - 1 replaced by its complement.  The rounding is a separate zkob_rescale run on the Y64 file.
//
//   zkob_rope prove  <obdir> <seed> <T-int32.bin> <B> <C> <HD> <cos-int32.bin> <sin-int32.bin> <gen.bin> <q.bin> [Y64-i64-out.bin]
//                    [--claims <accdir> <obid>]
//   zkob_rope verify <obdir> <seed> <B> <C> <HD> <cos-int32.bin> <sin-int32.bin> <gen.bin> <q.bin> [--claims <vaccdir> <obid>]
//   zkob_rope serve
//
// Files in <obdir> (byte for byte the reference's): dims.bin, com_T.bin, com_Y64.bin, ev.bin, hp1.bin, hp2.bin, ipa_T1.bin,
// ipa_T2.bin, ipa_Y.bin.  Exit 0 = success / ACCEPT, 1 = REJECT, anything else = failure.
#include "zkob_common.hpp"

using namespace zkob;

namespace {

constexpr uint32_t SCALE_R = 16;                                    // the tables' scale 2^16

struct Lay { uint32_t B, C, HD, Cp, logB, logCp, logD, D, fb; };
Lay lay_of(const char* b, const char* c, const char* hd) {
    Lay y;
    y.B = (uint32_t)atoi(b); y.C = (uint32_t)atoi(c); y.HD = (uint32_t)atoi(hd);
    if (!y.B || !y.C || !y.HD) throw std::runtime_error("bad dimensions");
    y.Cp = 1u << clog2(y.C);
    y.logB = clog2(y.B); y.logCp = clog2(y.Cp); y.logD = y.logB + y.logCp;
    y.D = y.B * y.Cp;
    y.fb = clog2(y.HD) ? clog2(y.HD) - 1 : 0;
    return y;
}
std::string layout_error(const Lay& y, size_t gen) {
    if (y.B != (1u << y.logB)) return "B not a power of two";
    if (y.HD < 2 || y.HD != (1u << clog2(y.HD))) return "HD must be a power of two >= 2";
    if (y.C % y.HD) return "HD must divide C";
    if (y.Cp % y.HD) return "HD must divide C_pad";
    if (y.C / y.HD < 2) return "NH = C/HD must be >= 2";
    if (gen != (size_t)y.Cp * G1B) return "generator size != C_pad";
    return "";
}
std::vector<int32_t> load_table(const std::string& path, const Lay& y) {
    const std::vector<uint8_t> raw = read_file(path);
    if (raw.size() != (size_t)y.B * y.HD * 4) throw std::runtime_error("table file size != B*HD int32: " + path);
    std::vector<int32_t> v((size_t)y.B * y.HD);
    memcpy(v.data(), raw.data(), raw.size());
    return v;
}
// the public weights on the padded grid (build_weights)
void build_weights(std::vector<int64_t>& W1, std::vector<int64_t>& W2, const std::vector<int32_t>& cosT, const std::vector<int32_t>& sinT, const Lay& y) {
    const uint32_t flipv = y.HD / 2;
    W1.assign(y.D, 0); W2.assign(y.D, 0);
    for (uint32_t t = 0; t < y.B; t++)
        for (uint32_t e = 0; e < y.C; e++) {
            const size_t g = (size_t)t * y.Cp + e;
            W1[g] = cosT[(size_t)t * y.HD + (e % y.HD)];
            W2[g] = ((e & flipv) ? 1 : -1) * (int64_t)sinT[(size_t)t * y.HD + (e % y.HD)];
        }
}
void absorb_head(Transcript& tr, const Lay& y) {
    tr.absorb_u32("B", y.B); tr.absorb_u32("C", y.C); tr.absorb_u32("HD", y.HD); tr.absorb_u32("SCALE_R", SCALE_R);
}

struct Had { Fr claim, S_f2, U_f2; std::vector<Fr> ws; };
// one Hadamard leg of the prover: E = eq(u) .* W, c = sum E S, the sumcheck over (E, S, ones), the terminals absorbed and the file written
Had hadamard(Ctx& x, Transcript& tr, const Dev& dE_u, const std::vector<int64_t>& W, const Dev& dS, const Dev& dOnes, const Lay& y, const char* clabel,
             const std::string& path) {
    const std::vector<Fr> Wf = lift(W);
    Dev dE(x, Wf.data(), Wf.size() * FRB);
    x.ck(zkh_fr_mul(x.c, dE.p, dE_u.p, dE.p, y.D), "weights");
    Had h;
    x.ck(zkh_fr_dot(x.c, dE.p, dS.p, y.D, h.claim.v), "claim");
    tr.absorb_fr(clabel, h.claim);
    std::vector<Fr> hev((size_t)4 * y.logD);
    h.ws.resize(y.logD);
    Fr fin[3];
    const void* cols[3] = {dE.p, dS.p, dOnes.p};
    const char* labels[4] = {"hp0", "hp1", "hp2", "hp3"};
    x.ck(zkh_fr_sumcheck(x.c, cols, 3, y.logD, labels, tr.st, hev.data(), h.ws.data(), fin), "hadamard sumcheck");
    h.S_f2 = fin[1]; h.U_f2 = fin[2];
    tr.absorb_fr("S_f2", h.S_f2); tr.absorb_fr("U_f2", h.U_f2);
    write_hp(path, h.claim, hev, h.S_f2, h.U_f2);
    return h;
}

int do_prove(int argc, char** argv) {
    const ClaimFlags cf = claim_flags(argc, argv);
    argc = cf.base_argc;
    if (argc != 12 && argc != 13) throw std::invalid_argument("prove <obdir> <seed> <T-int32> <B> <C> <HD> <cos-int32> <sin-int32> <gen> <q.bin> [Y64-out]");
    const std::string obdir = argv[2], seed = argv[3];
    const Lay y = lay_of(argv[5], argv[6], argv[7]);
    const uint32_t B = y.B, C = y.C, Cp = y.Cp, D = y.D;
    std::vector<int32_t> Th((size_t)B * C);
    {
        const std::vector<uint8_t> raw = read_file(argv[4]);
        if (raw.size() < Th.size() * 4) throw std::runtime_error(std::string("short read / wrong dims: ") + argv[4]);
        memcpy(Th.data(), raw.data(), Th.size() * 4);
    }
    const std::vector<int32_t> cosT = load_table(argv[8], y), sinT = load_table(argv[9], y);
    const std::vector<uint8_t> gen = read_file(argv[10]), q = read_file(argv[11]);
    if (q.size() < G1B) throw std::runtime_error("q.bin holds no point");
    const std::string le = layout_error(y, gen.size());
    if (!le.empty()) throw std::runtime_error(le);
    std::vector<int64_t> W1, W2;
    build_weights(W1, W2, cosT, sinT, y);
    const uint32_t flipv = y.HD / 2;
    std::vector<int64_t> Tg(D, 0), Txg(D), Yg(D);
    for (uint32_t t = 0; t < B; t++)
        for (uint32_t e = 0; e < C; e++) Tg[(size_t)t * Cp + e] = Th[(size_t)t * C + e];
    for (uint32_t t = 0; t < B; t++)
        for (uint32_t e = 0; e < Cp; e++) Txg[(size_t)t * Cp + e] = Tg[(size_t)t * Cp + (e ^ flipv)];
    for (size_t g = 0; g < D; g++) {
        Yg[g] = Tg[g] * W1[g] + Txg[g] * W2[g];
        if (std::llabs(Yg[g]) >= (1LL << 47)) throw std::runtime_error("|Y64| >= 2^47 (int32 chain format after rescale at risk)");
    }
    if (argc == 13) {                                               // the chain file: the unpadded B x C tensor as int64, scale 2^32
        std::vector<int64_t> yo((size_t)B * C);
        for (uint32_t t = 0; t < B; t++)
            for (uint32_t e = 0; e < C; e++) yo[(size_t)t * C + e] = Yg[(size_t)t * Cp + e];
        std::vector<uint8_t> b(yo.size() * 8);
        memcpy(b.data(), yo.data(), b.size());
        write_file(argv[12], b);
    }
    Ctx x;
    Dev gd(x, gen.data(), gen.size());
    const std::vector<Fr> Tf = lift(Tg), Txf = lift(Txg), Yf = lift(Yg), ones((size_t)D, fr_u32(1)), none;
    Dev dT(x, Tf.data(), Tf.size() * FRB), dTx(x, Txf.data(), Txf.size() * FRB), dY(x, Yf.data(), Yf.size() * FRB), dOnes(x, ones.data(), ones.size() * FRB);
    const std::vector<uint8_t> comT = commit_rows(x, gd, dT, B, Cp), comY = commit_rows(x, gd, dY, B, Cp);
    write_file(obdir + "/com_T.bin", comT);
    write_file(obdir + "/com_Y64.bin", comY);
    { std::vector<uint8_t> f; const uint32_t dm[4] = {B, C, y.HD, SCALE_R}; put(f, dm, 16); write_file(obdir + "/dims.bin", f); }

    Transcript tr(seed);
    absorb_head(tr, y);
    tr.absorb("com_T", comT.data(), comT.size());
    tr.absorb("com_Y64", comY.data(), comY.size());
    const std::vector<Fr> u = tr.challenge_vec(y.logD);
    Fr ev;
    x.ck(zkh_fr_mle_eval(x.c, dY.p, u.data(), y.logD, ev.v), "ev");
    tr.absorb_fr("ev", ev);
    { std::vector<uint8_t> f; put(f, ev.v, FRB); write_file(obdir + "/ev.bin", f); }
    Dev dE_u(x, (size_t)D * FRB);
    x.ck(zkh_fr_eq_build(x.c, u.data(), y.logD, dE_u.p), "eq table");

    const std::string comTref = obdir + "/com_T.bin", comYref = obdir + "/com_Y64.bin";
    const Had h1 = hadamard(x, tr, dE_u, W1, dT, dOnes, y, "c1", obdir + "/hp1.bin");
    const std::vector<Fr> pt1(h1.ws.rbegin(), h1.ws.rend());
    if (!fr_eq(h1.U_f2, fr_u32(1))) throw std::runtime_error("h1 terminal != multi_dim_me / 1 (convention bug)");
    if (cf.on()) {
        const std::string witT = cf.accdir + "/wit_" + cf.obid + "_T.fr";
        save_scalars(witT, Tf);
        claim_emit(cf.accdir, make_claim(cf.obid, "T1", comTref, Cp, B, pt1, none, h1.S_f2));
        witref_emit(cf.accdir, comTref, witT);
    } else {
        open_prove(x, dT, B, Cp, gd, q.data(), pt1, obdir + "/ipa_T1.bin", tr);
    }
    const Had h2 = hadamard(x, tr, dE_u, W2, dTx, dOnes, y, "c2", obdir + "/hp2.bin");
    std::vector<Fr> pt2p(h2.ws.rbegin(), h2.ws.rend());
    pt2p[y.fb] = fr_sub(fr_u32(1), pt2p[y.fb]);
    {   // completeness guard: T~ at the flipped point is the flipped copy's terminal
        Fr chk;
        x.ck(zkh_fr_mle_eval(x.c, dT.p, pt2p.data(), y.logD, chk.v), "flip check");
        if (!fr_eq(chk, h2.S_f2)) throw std::runtime_error("T~(pt2') != h2 S_f2 (flip convention bug)");
        if (!fr_eq(h2.U_f2, fr_u32(1))) throw std::runtime_error("h2 U_f2 != 1 (convention bug)");
    }
    if (cf.on()) {
        claim_emit(cf.accdir, make_claim(cf.obid, "T2", comTref, Cp, B, pt2p, none, h2.S_f2));
        const std::string witY = cf.accdir + "/wit_" + cf.obid + "_Y.fr";
        save_scalars(witY, Yf);
        claim_emit(cf.accdir, make_claim(cf.obid, "Y", comYref, Cp, B, u, none, ev));
        witref_emit(cf.accdir, comYref, witY);
        drvstate_emit(cf.accdir, cf.obid, tr.st);
        std::cout << "PROVED rope obligation (claim mode, 3 claims emitted) -> " << obdir << std::endl;
        return 0;
    }
    open_prove(x, dT, B, Cp, gd, q.data(), pt2p, obdir + "/ipa_T2.bin", tr);
    open_prove(x, dY, B, Cp, gd, q.data(), u, obdir + "/ipa_Y.bin", tr);
    std::cout << "PROVED rope obligation -> " << obdir << std::endl;
    return 0;
}

// one Hadamard leg of the verifier: round checks, U_f2 == 1, the verifier's own folded weights; the round challenges in ws
bool hadamard_check(Ctx& x, Transcript& tr, const Hp& hp, const Dev& dE_u, const std::vector<int64_t>& W, const Lay& y, const char* clabel, const char* tag,
                    const Fr& inv2, const Fr& inv6, std::vector<Fr>& ws) {
    tr.absorb_fr(clabel, hp.claim);
    Fr cur = hp.claim;
    for (uint32_t k = 0; k < y.logD; k++) {
        const std::array<Fr, 4> e = {hp.ev[4 * k], hp.ev[4 * k + 1], hp.ev[4 * k + 2], hp.ev[4 * k + 3]};
        if (!fr_eq(cur, fr_add(e[0], e[1]))) return rj(std::string(tag) + " round " + std::to_string(k) + " p(0)+p(1) != claim");
        tr.absorb_fr("hp0", e[0]); tr.absorb_fr("hp1", e[1]); tr.absorb_fr("hp2", e[2]); tr.absorb_fr("hp3", e[3]);
        const Fr w = tr.challenge_fr();
        ws.push_back(w);
        cur = lagrange4(e, w, inv6, inv2);
    }
    if (!fr_eq(hp.U_f2, fr_u32(1))) return rj(std::string(tag) + " U_f2 != 1");
    const std::vector<Fr> Wf = lift(W);
    Dev dE(x, Wf.data(), Wf.size() * FRB);
    x.ck(zkh_fr_mul(x.c, dE.p, dE_u.p, dE.p, y.D), "weights");
    uint64_t sz = y.D;
    for (const Fr& w : ws) { x.ck(zkh_fr_fold(x.c, dE.p, sz / 2, w.v, dE.p), "fold weights"); sz /= 2; }
    Fr W_f;
    x.ck(zkh_download(x.c, W_f.v, dE.p, FRB), "download");
    if (!fr_eq(cur, fr_mul(W_f, fr_mul(hp.S_f2, hp.U_f2)))) return rj(std::string(tag) + " weight terminal");
    tr.absorb_fr("S_f2", hp.S_f2); tr.absorb_fr("U_f2", hp.U_f2);
    return true;
}

bool verify(Ctx& x, const std::string& obdir, const std::string& seed, const Lay& y, const std::vector<int32_t>& cosT, const std::vector<int32_t>& sinT,
            const std::vector<uint8_t>& gen, const std::vector<uint8_t>& q, const ClaimFlags& cf) {
    if (!layout_error(y, gen.size()).empty()) return rj("bad layout params");
    const uint32_t B = y.B, Cp = y.Cp;
    {
        const std::vector<uint8_t> f = read_file(obdir + "/dims.bin");
        uint32_t dm[4];
        if (f.size() < 16) return rj("dims.bin short read");
        memcpy(dm, f.data(), 16);
        if (dm[0] != B || dm[1] != y.C || dm[2] != y.HD || dm[3] != SCALE_R) return rj("dims.bin mismatch");
    }
    const std::vector<uint8_t> comT = read_file(obdir + "/com_T.bin"), comY = read_file(obdir + "/com_Y64.bin");
    if (comT.size() != (size_t)B * G1B || comY.size() != (size_t)B * G1B) return rj("commitment row counts");
    Hp hp1, hp2;
    if (!read_hp(obdir + "/hp1.bin", 4 * y.logD, hp1) || !read_hp(obdir + "/hp2.bin", 4 * y.logD, hp2)) return rj("hadamard round count");
    Fr ev;
    {
        const std::vector<uint8_t> f = read_file(obdir + "/ev.bin");
        if (f.size() < FRB) return rj("ev.bin short read");
        memcpy(ev.v, f.data(), FRB);
        if (!fr_lt(ev, FR_MOD)) return rj("non-canonical ev");
    }
    std::vector<int64_t> W1, W2;                                    // from the verifier's own table copies
    build_weights(W1, W2, cosT, sinT, y);
    Transcript tr(seed);
    absorb_head(tr, y);
    tr.absorb("com_T", comT.data(), comT.size());
    tr.absorb("com_Y64", comY.data(), comY.size());
    const std::vector<Fr> u = tr.challenge_vec(y.logD), none;
    tr.absorb_fr("ev", ev);
    const Fr inv2 = fr_inv(fr_u32(2)), inv6 = fr_inv(fr_u32(6));
    Dev dE_u(x, (size_t)y.D * FRB), gd(x, gen.data(), gen.size());
    x.ck(zkh_fr_eq_build(x.c, u.data(), y.logD, dE_u.p), "eq table");

    std::vector<Fr> ws1, ws2;
    if (!hadamard_check(x, tr, hp1, dE_u, W1, y, "c1", "h1", inv2, inv6, ws1)) return false;
    const std::vector<Fr> pt1(ws1.rbegin(), ws1.rend());
    if (!cf.on() && !open_check(x, comT, Cp, gd, q.data(), pt1, hp1.S_f2, obdir + "/ipa_T1.bin", tr)) return rj("IPA opening of h1 terminal vs com_T");
    if (!hadamard_check(x, tr, hp2, dE_u, W2, y, "c2", "h2", inv2, inv6, ws2)) return false;
    std::vector<Fr> pt2p(ws2.rbegin(), ws2.rend());
    pt2p[y.fb] = fr_sub(fr_u32(1), pt2p[y.fb]);                     // the verifier flips the coordinate itself
    if (!cf.on()) {
        if (!open_check(x, comT, Cp, gd, q.data(), pt2p, hp2.S_f2, obdir + "/ipa_T2.bin", tr)) return rj("IPA opening of h2 terminal vs com_T at the flipped point");
        if (!open_check(x, comY, Cp, gd, q.data(), u, ev, obdir + "/ipa_Y.bin", tr)) return rj("IPA opening of ev vs com_Y64");
    }
    if (!fr_eq(fr_add(hp1.claim, hp2.claim), ev)) return rj("c1 + c2 != ev");
    if (cf.on()) {
        claim_emit(cf.accdir, make_claim(cf.obid, "T1", obdir + "/com_T.bin", Cp, B, pt1, none, hp1.S_f2));
        claim_emit(cf.accdir, make_claim(cf.obid, "T2", obdir + "/com_T.bin", Cp, B, pt2p, none, hp2.S_f2));
        claim_emit(cf.accdir, make_claim(cf.obid, "Y", obdir + "/com_Y64.bin", Cp, B, u, none, ev));
        drvstate_emit(cf.accdir, cf.obid, tr.st);
        std::cout << "ACCEPT-conditional (3 claims emitted; final verdict gated on opening_batch)" << std::endl;
        return true;
    }
    std::cout << "ACCEPT" << std::endl;
    return true;
}

int do_verify(int argc, char** argv) {
    const ClaimFlags cf = claim_flags(argc, argv);
    argc = cf.base_argc;
    if (argc != 11) throw std::invalid_argument("verify <obdir> <seed> <B> <C> <HD> <cos-int32> <sin-int32> <gen> <q.bin>");
    const Lay y = lay_of(argv[4], argv[5], argv[6]);
    const std::vector<int32_t> cosT = load_table(argv[7], y), sinT = load_table(argv[8], y);
    const std::vector<uint8_t> gen = read_file(argv[9]), q = read_file(argv[10]);
    if (q.size() < G1B) throw std::runtime_error("q.bin holds no point");
    if (!layout_error(y, gen.size()).empty()) return rj("bad layout params") ? 0 : 1;
    Ctx x;
    return verify(x, argv[2], argv[3], y, cosT, sinT, gen, q, cf) ? 0 : 1;
}

int run1(int argc, char** argv) {
    const std::string mode = argc > 1 ? argv[1] : "";
    try {
        if (mode == "prove") return do_prove(argc, argv);
        if (mode == "verify") return do_verify(argc, argv);
    } catch (const std::invalid_argument& e) {
        std::cerr << "zkob_rope: " << e.what() << std::endl;
        return 2;
    }
    std::cerr << "usage: zkob_rope prove ... [--claims <accdir> <obid>] | verify ... [--claims <vaccdir> <obid>] | serve" << std::endl;
    return 2;
}

}  // namespace

int main(int argc, char** argv) {
    try {
        if (argc > 1 && std::string(argv[1]) == "serve") return serve_loop(argv[0], run1);
        return run1(argc, argv);
    } catch (const std::exception& e) {
        std::cerr << "zkob_rope: " << e.what() << std::endl;
        return 3;
    }
}
