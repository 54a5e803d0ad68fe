// Driver for the head-merge obligation (layer.attn.merge) of the reference's first proof stack, with the command line, the files
// and the exit codes of the reference's zkob_headmerge (zkllm-src/zkob_headmerge.cu:1-66, :161-309 prove, :316-431 verify).  It
// binds the NH per-head outputs out_h (B x HD) to the merged tensor O2 (B x C), either through the pipeline's transpose-and-
// reshape permutation ("pi157": O2[i, j] = M[t, e] with m = i C + j, t = m mod B, e = m div B, M the head concatenation) or as
// the plain concatenation ("concat"): one challenge u over the padded O2 grid, the claim ev = O2~(u), then per head a Hadamard
// sumcheck with the PUBLIC weights Wm_h (the equality table of u gathered through the permutation), the head's outputs and a
// column of ones, the terminal opened against com_O{hh}; finally O2 opened at u and the check sum_h c_h == ev.
//
//   zkob_headmerge prove  <obdir> <seed> <Oh-prefix> <B> <C> <HD> <perm> <gen_big.bin> <gen_small.bin> <q.bin> [O2-int32-out.bin]
//                         [--claims <accdir> <obid>]
//   zkob_headmerge verify <obdir> <seed> <B> <C> <HD> <perm> <gen_big.bin> <gen_small.bin> <q.bin> [--claims <vaccdir> <obid>]
//   zkob_headmerge serve
//
// <Oh-prefix>{hh}.i32.bin is read for hh = 00 .. NH-1.  Files in <obdir> (byte for byte the reference's): dims.bin, com_O2.bin,
// com_O{hh}.bin, ev.bin, hp{hh}.bin, ipa_O{hh}.bin, ipa_O2.bin.  Exit 0 = success / ACCEPT, 1 = REJECT, anything else = failure.
#include "zkob_common.hpp"

using namespace zkob;

namespace {

struct Lay { uint32_t B, C, HD, perm, Cp, logB, logCp, logHD, NH, D, DH, logDH; };
std::string hh2(uint32_t h) { char b[16]; snprintf(b, sizeof b, "%02u", h); return b; }
Lay lay_of(const char* b, const char* c, const char* hd, const char* perm) {
    Lay y;
    y.B = (uint32_t)atoi(b); y.C = (uint32_t)atoi(c); y.HD = (uint32_t)atoi(hd);
    if (!y.B || !y.C || !y.HD) throw std::runtime_error("bad dimensions");
    const std::string p = perm;
    if (p == "pi157") y.perm = 0;
    else if (p == "concat") y.perm = 1;
    else throw std::runtime_error("perm must be 'pi157' or 'concat'");
    y.Cp = 1u << clog2(y.C);
    y.logB = clog2(y.B); y.logCp = clog2(y.Cp); y.logHD = clog2(y.HD);
    y.NH = y.C / y.HD; y.D = y.B * y.Cp; y.DH = y.B * y.HD; y.logDH = y.logB + y.logHD;
    return y;
}
std::string layout_error(const Lay& y, size_t big, size_t small) {
    if (y.B != (1u << y.logB)) return "B not a power of two";
    if (y.HD < 2 || y.HD != (1u << y.logHD)) return "HD must be a power of two >= 2";
    if (y.C % y.HD) return "HD must divide C";
    if (y.Cp % y.HD) return "HD must divide C_pad";
    if (y.C / y.HD < 2) return "NH = C/HD must be >= 2";
    if (big != (size_t)y.Cp * G1B) return "gen_big size != C_pad";
    if (small != (size_t)y.HD * G1B) return "gen_small size != HD";
    return "";
}
// the weights of head h: the equality table of u gathered through the inverse permutation (gather_Wm)
std::vector<Fr> gather_Wm(const std::vector<Fr>& Eh, const Lay& y, uint32_t h) {
    std::vector<Fr> Wm((size_t)y.DH);
    for (uint32_t t = 0; t < y.B; t++)
        for (uint32_t d = 0; d < y.HD; d++) {
            const size_t e = (size_t)y.HD * h + d;
            size_t i, j;
            if (y.perm == 0) { const size_t m = e * y.B + t; i = m / y.C; j = m % y.C; }
            else { i = t; j = e; }
            Wm[(size_t)t * y.HD + d] = Eh[i * y.Cp + j];
        }
    return Wm;
}
void absorb_head(Transcript& tr, const Lay& y) {
    tr.absorb_u32("B", y.B); tr.absorb_u32("C", y.C); tr.absorb_u32("HD", y.HD); tr.absorb_u32("PERM", y.perm);
}
std::vector<Fr> eq_table_host(Ctx& x, const std::vector<Fr>& u, uint32_t D) {
    Dev e(x, (size_t)D * FRB);
    x.ck(zkh_fr_eq_build(x.c, u.data(), (uint32_t)u.size(), e.p), "eq table");
    const std::vector<uint8_t> raw = e.host();
    std::vector<Fr> Eh(D);
    memcpy(Eh.data(), raw.data(), raw.size());
    return Eh;
}

int do_prove(int argc, char** argv) {
    const ClaimFlags cf = claim_flags(argc, argv);
    argc = cf.base_argc;
    if (argc != 12 && argc != 13) throw std::invalid_argument("prove <obdir> <seed> <Oh-prefix> <B> <C> <HD> <perm> <gen_big> <gen_small> <q.bin> [O2-out]");
    const std::string obdir = argv[2], seed = argv[3], prefix = argv[4];
    const Lay y = lay_of(argv[5], argv[6], argv[7], argv[8]);
    const std::vector<uint8_t> gb = read_file(argv[9]), gs = read_file(argv[10]), q = read_file(argv[11]);
    if (q.size() < G1B) throw std::runtime_error("q.bin holds no point");
    const std::string le = layout_error(y, gb.size(), gs.size());
    if (!le.empty()) throw std::runtime_error(le);
    const uint32_t B = y.B, C = y.C, HD = y.HD, NH = y.NH;
    std::vector<std::vector<int32_t>> outs(NH);
    for (uint32_t h = 0; h < NH; h++) {
        const std::string path = prefix + hh2(h) + ".i32.bin";
        const std::vector<uint8_t> raw = read_file(path);
        if (raw.size() != (size_t)y.DH * 4) throw std::runtime_error("file size != expected int32 count: " + path);
        outs[h].resize(y.DH);
        memcpy(outs[h].data(), raw.data(), raw.size());
    }
    // O2 on the padded grid
    std::vector<int64_t> O2g((size_t)y.D, 0);
    for (uint32_t i = 0; i < B; i++)
        for (uint32_t j = 0; j < C; j++) {
            if (y.perm == 0) {
                const size_t m = (size_t)i * C + j;
                const uint32_t t = (uint32_t)(m % B), e = (uint32_t)(m / B);
                O2g[(size_t)i * y.Cp + j] = outs[e / HD][(size_t)t * HD + (e % HD)];
            } else {
                O2g[(size_t)i * y.Cp + j] = outs[j / HD][(size_t)i * HD + (j % HD)];
            }
        }
    if (argc == 13) {                                              // the chain file: the unpadded B x C tensor as int32
        std::vector<int32_t> oo((size_t)B * C);
        for (uint32_t i = 0; i < B; i++)
            for (uint32_t j = 0; j < C; j++) oo[(size_t)i * C + j] = (int32_t)O2g[(size_t)i * y.Cp + j];
        std::vector<uint8_t> b(oo.size() * 4);
        memcpy(b.data(), oo.data(), b.size());
        write_file(argv[12], b);
    }
    Ctx x;
    Dev gbd(x, gb.data(), gb.size()), gsd(x, gs.data(), gs.size());
    std::vector<Fr> O2f(O2g.size());
    for (size_t i = 0; i < O2g.size(); i++) O2f[i] = fr_from_i64(O2g[i]);
    Dev dO2(x, O2f.data(), O2f.size() * FRB);
    const std::vector<uint8_t> comO2 = commit_rows(x, gbd, dO2, B, y.Cp);
    write_file(obdir + "/com_O2.bin", comO2);
    std::vector<std::vector<Fr>> outf(NH);
    std::vector<std::unique_ptr<Dev>> dO(NH);
    std::vector<std::vector<uint8_t>> comO(NH);
    for (uint32_t h = 0; h < NH; h++) {
        outf[h].resize(y.DH);
        for (uint32_t i = 0; i < y.DH; i++) outf[h][i] = fr_from_i64(outs[h][i]);
        dO[h].reset(new Dev(x, outf[h].data(), outf[h].size() * FRB));
        comO[h] = commit_rows(x, gsd, *dO[h], B, HD);
        write_file(obdir + "/com_O" + hh2(h) + ".bin", comO[h]);
    }
    { std::vector<uint8_t> f; const uint32_t dm[4] = {B, C, HD, y.perm}; put(f, dm, 16); write_file(obdir + "/dims.bin", f); }

    Transcript tr(seed);
    absorb_head(tr, y);
    tr.absorb("com_O2", comO2.data(), comO2.size());
    for (uint32_t h = 0; h < NH; h++) tr.absorb(("com_O" + hh2(h)).c_str(), comO[h].data(), comO[h].size());
    const std::vector<Fr> u = tr.challenge_vec(y.logB + y.logCp);
    Fr ev;
    x.ck(zkh_fr_mle_eval(x.c, dO2.p, u.data(), (uint32_t)u.size(), ev.v), "ev");
    tr.absorb_fr("ev", ev);
    { std::vector<uint8_t> f; put(f, ev.v, FRB); write_file(obdir + "/ev.bin", f); }
    const std::vector<Fr> Eh = eq_table_host(x, u, y.D);
    const std::vector<Fr> ones((size_t)y.DH, fr_u32(1)), none;
    Dev dOnes(x, ones.data(), ones.size() * FRB);
    Fr csum{};
    for (uint32_t h = 0; h < NH; h++) {
        const std::vector<Fr> Wm = gather_Wm(Eh, y, h);
        Dev dW(x, Wm.data(), Wm.size() * FRB);
        Fr c;
        x.ck(zkh_fr_dot(x.c, dW.p, dO[h]->p, y.DH, c.v), "head claim");
        tr.absorb_fr(("c" + hh2(h)).c_str(), c);
        csum = fr_add(csum, c);
        std::vector<Fr> hev((size_t)4 * y.logDH), ws(y.logDH);
        Fr fin[3];
        const void* cols[3] = {dW.p, dO[h]->p, dOnes.p};
        const char* labels[4] = {"hp0", "hp1", "hp2", "hp3"};
        x.ck(zkh_fr_sumcheck(x.c, cols, 3, y.logDH, labels, tr.st, hev.data(), ws.data(), fin), "hadamard sumcheck");
        tr.absorb_fr("S_f2", fin[1]); tr.absorb_fr("U_f2", fin[2]);
        {
            std::vector<uint8_t> f;
            const uint32_t n = 4 * y.logDH;
            put(f, c.v, FRB); put(f, &n, 4); put(f, hev.data(), hev.size() * FRB); put(f, fin[1].v, FRB); put(f, fin[2].v, FRB);
            write_file(obdir + "/hp" + hh2(h) + ".bin", f);
        }
        const std::vector<Fr> pt(ws.rbegin(), ws.rend());
        if (cf.on()) {
            const std::string comref = obdir + "/com_O" + hh2(h) + ".bin", wit = cf.accdir + "/wit_" + cf.obid + "_O" + hh2(h) + ".fr";
            claim_emit(cf.accdir, make_claim(cf.obid, ("O" + hh2(h)).c_str(), comref, HD, B, pt, none, fin[1]));
            save_scalars(wit, outf[h]);
            witref_emit(cf.accdir, comref, wit);
        } else {
            open_prove(x, *dO[h], B, HD, gsd, q.data(), pt, obdir + "/ipa_O" + hh2(h) + ".bin", tr);
        }
    }
    if (!fr_eq(csum, ev)) throw std::runtime_error("sum of head claims != ev (pi formula bug)");
    if (cf.on()) {
        const std::string comref = obdir + "/com_O2.bin", wit = cf.accdir + "/wit_" + cf.obid + "_O2.fr";
        claim_emit(cf.accdir, make_claim(cf.obid, "O2", comref, y.Cp, B, u, none, ev));
        save_scalars(wit, O2f);
        witref_emit(cf.accdir, comref, wit);
        drvstate_emit(cf.accdir, cf.obid, tr.st);
        std::cout << "PROVED headmerge obligation (claim mode, " << NH + 1 << " claims emitted) -> " << obdir << std::endl;
        return 0;
    }
    open_prove(x, dO2, B, y.Cp, gbd, q.data(), u, obdir + "/ipa_O2.bin", tr);
    std::cout << "PROVED headmerge obligation -> " << obdir << std::endl;
    return 0;
}

bool verify(Ctx& x, const std::string& obdir, const std::string& seed, const Lay& y, const std::vector<uint8_t>& gb, const std::vector<uint8_t>& gs,
            const std::vector<uint8_t>& q, const ClaimFlags& cf) {
    if (!layout_error(y, gb.size(), gs.size()).empty()) return rj("bad layout params");
    const uint32_t B = y.B, HD = y.HD, NH = y.NH;
    {
        const std::vector<uint8_t> f = read_file(obdir + "/dims.bin");
        uint32_t dm[4];
        if (f.size() < 16) return rj("dims.bin short read");
        memcpy(dm, f.data(), 16);
        if (dm[0] != B || dm[1] != y.C || dm[2] != HD || dm[3] != y.perm) return rj("dims.bin mismatch");
    }
    const std::vector<uint8_t> comO2 = read_file(obdir + "/com_O2.bin");
    if (comO2.size() != (size_t)B * G1B) return rj("com_O2 row count");
    std::vector<std::vector<uint8_t>> comO(NH);
    std::vector<Hp> hps(NH);
    for (uint32_t h = 0; h < NH; h++) {
        comO[h] = read_file(obdir + "/com_O" + hh2(h) + ".bin");
        if (comO[h].size() != (size_t)B * G1B) return rj("com_O" + hh2(h) + " row count");
        if (!read_hp(obdir + "/hp" + hh2(h) + ".bin", 4 * y.logDH, hps[h])) return rj("hadamard " + hh2(h) + " round count");
    }
    Fr ev;
    {
        const std::vector<uint8_t> f = read_file(obdir + "/ev.bin");
        if (f.size() < FRB) return rj("ev.bin short read");
        memcpy(ev.v, f.data(), FRB);
        if (!fr_lt(ev, FR_MOD)) return rj("non-canonical ev");
    }
    Transcript tr(seed);
    absorb_head(tr, y);
    tr.absorb("com_O2", comO2.data(), comO2.size());
    for (uint32_t h = 0; h < NH; h++) tr.absorb(("com_O" + hh2(h)).c_str(), comO[h].data(), comO[h].size());
    const std::vector<Fr> u = tr.challenge_vec(y.logB + y.logCp), none;
    tr.absorb_fr("ev", ev);
    const Fr inv2 = fr_inv(fr_u32(2)), inv6 = fr_inv(fr_u32(6)), one = fr_u32(1);
    const std::vector<Fr> Eh = eq_table_host(x, u, y.D);
    Dev gbd(x, gb.data(), gb.size()), gsd(x, gs.data(), gs.size());
    Fr csum{};
    std::vector<std::vector<Fr>> pts;
    for (uint32_t h = 0; h < NH; h++) {
        const Hp& hp = hps[h];
        tr.absorb_fr(("c" + hh2(h)).c_str(), hp.claim);
        csum = fr_add(csum, hp.claim);
        Fr cur = hp.claim;
        std::vector<Fr> ws;
        for (uint32_t k = 0; k < y.logDH; k++) {
            const std::array<Fr, 4> e = {hp.ev[4 * k], hp.ev[4 * k + 1], hp.ev[4 * k + 2], hp.ev[4 * k + 3]};
            if (!fr_eq(cur, fr_add(e[0], e[1]))) return rj("merge hadamard " + hh2(h) + " round " + std::to_string(k) + " p(0)+p(1) != claim");
            tr.absorb_fr("hp0", e[0]); tr.absorb_fr("hp1", e[1]); tr.absorb_fr("hp2", e[2]); tr.absorb_fr("hp3", e[3]);
            const Fr w = tr.challenge_fr();
            ws.push_back(w);
            cur = lagrange4(e, w, inv6, inv2);
        }
        if (!fr_eq(hp.U_f2, one)) return rj("merge hadamard " + hh2(h) + " U_f2 != 1");
        {   // the verifier's own weights, folded over the round challenges
            const std::vector<Fr> Wm = gather_Wm(Eh, y, h);
            Dev dW(x, Wm.data(), Wm.size() * FRB);
            uint64_t sz = y.DH;
            for (const Fr& w : ws) { x.ck(zkh_fr_fold(x.c, dW.p, sz / 2, w.v, dW.p), "fold weights"); sz /= 2; }
            Fr W_f;
            x.ck(zkh_download(x.c, W_f.v, dW.p, FRB), "download");
            if (!fr_eq(cur, fr_mul(W_f, fr_mul(hp.S_f2, hp.U_f2)))) return rj("merge hadamard " + hh2(h) + " terminal");
        }
        tr.absorb_fr("S_f2", hp.S_f2); tr.absorb_fr("U_f2", hp.U_f2);
        const std::vector<Fr> pt(ws.rbegin(), ws.rend());
        if (cf.on()) pts.push_back(pt);
        else if (!open_check(x, comO[h], HD, gsd, q.data(), pt, hp.S_f2, obdir + "/ipa_O" + hh2(h) + ".bin", tr))
            return rj("IPA opening of head " + hh2(h) + " terminal vs com_O" + hh2(h));
    }
    if (!cf.on() && !open_check(x, comO2, y.Cp, gbd, q.data(), u, ev, obdir + "/ipa_O2.bin", tr)) return rj("IPA opening of ev vs com_O2");
    if (!fr_eq(csum, ev)) return rj("sum of head claims != ev");
    if (cf.on()) {
        for (uint32_t h = 0; h < NH; h++)
            claim_emit(cf.accdir, make_claim(cf.obid, ("O" + hh2(h)).c_str(), obdir + "/com_O" + hh2(h) + ".bin", HD, B, pts[h], none, hps[h].S_f2));
        claim_emit(cf.accdir, make_claim(cf.obid, "O2", obdir + "/com_O2.bin", y.Cp, B, u, none, ev));
        drvstate_emit(cf.accdir, cf.obid, tr.st);
        std::cout << "ACCEPT-conditional (" << NH + 1 << " claims emitted; final verdict gated on opening_batch)" << std::endl;
        return true;
    }
    std::cout << "ACCEPT" << std::endl;
    return true;
}

int do_verify(int argc, char** argv) {
    const ClaimFlags cf = claim_flags(argc, argv);
    argc = cf.base_argc;
    if (argc != 11) throw std::invalid_argument("verify <obdir> <seed> <B> <C> <HD> <perm> <gen_big> <gen_small> <q.bin>");
    const Lay y = lay_of(argv[4], argv[5], argv[6], argv[7]);
    const std::vector<uint8_t> gb = read_file(argv[8]), gs = read_file(argv[9]), q = read_file(argv[10]);
    if (q.size() < G1B) throw std::runtime_error("q.bin holds no point");
    if (!layout_error(y, gb.size(), gs.size()).empty()) return rj("bad layout params") ? 0 : 1;
    Ctx x;
    return verify(x, argv[2], argv[3], y, gb, gs, q, cf) ? 0 : 1;
}

int run1(int argc, char** argv) {
    const std::string mode = argc > 1 ? argv[1] : "";
    try {
        if (mode == "prove") return do_prove(argc, argv);
        if (mode == "verify") return do_verify(argc, argv);
    } catch (const std::invalid_argument& e) {
        std::cerr << "zkob_headmerge: " << e.what() << std::endl;
        return 2;
    }
    std::cerr << "usage: zkob_headmerge prove ... [--claims <accdir> <obid>] | verify ... [--claims <vaccdir> <obid>] | serve" << std::endl;
    return 2;
}

}  // namespace

int main(int argc, char** argv) {
    try {
        if (argc > 1 && std::string(argv[1]) == "serve") return serve_loop(argv[0], run1);
        return run1(argc, argv);
    } catch (const std::exception& e) {
        std::cerr << "zkob_headmerge: " << e.what() << std::endl;
        return 3;
    }
}
