// Driver for the per-head slicing obligation (layer.attn.slice) of the reference's first proof stack, with the command line,
// the files and the exit codes of the reference's zkob_headslice (zkllm-src/zkob_headslice.cu:1-55, :136-317 prove, :323-446
// verify).  It binds the 3 NH per-head operand commitments (Qh, KhT, Vh per head) to the full-tensor commitments com_Q, com_K,
// com_V: one challenge v = (v_d || v_t); per head and tensor ONE claimed evaluation opened twice, against the slice commitment
// and against the full commitment at the head-selector point (v_d || bits(h) || v_t); the transposed KhT opens at (v_t || v_d).
//
//   zkob_headslice prove  <obdir> <seed> <Q-int32.bin> <K-int32.bin> <V-int32.bin> <B> <C> <HD> <gen_big.bin> <gen_small.bin>
//                         <q.bin> [slice-out-dir] [--claims <accdir> <obid>]
//   zkob_headslice verify <obdir> <seed> <B> <C> <HD> <gen_big.bin> <gen_small.bin> <q.bin> [--claims <vaccdir> <obid>]
//   zkob_headslice serve
//
// Files in <obdir> (byte for byte the reference's): dims.bin, com_Q / com_K / com_V.bin, com_Qh{hh} / com_KhT{hh} / com_Vh{hh}.bin,
// evals.bin (eQ00, eK00, eV00, eQ01, ...), ipa_Qh / Qf / Kh / Kf / Vh / Vf{hh}.bin; in [slice-out-dir] the per-head operand files
// for the downstream matmul runs.  Exit 0 = success / ACCEPT, 1 = REJECT, anything else = failure.
#include "zkob_common.hpp"

using namespace zkob;

namespace {

struct Lay { uint32_t B, C, HD, Cp, logB, logCp, logHD, nhb, NH; };
std::string hh2(uint32_t h) { char b[16]; snprintf(b, sizeof b, "%02u", h); return b; }
Lay lay_of(const char* b, const char* c, const char* hd) {
    Lay y;
    y.B = (uint32_t)atoi(b); y.C = (uint32_t)atoi(c); y.HD = (uint32_t)atoi(hd);
    if (!y.B || !y.C || !y.HD) throw std::runtime_error("bad dimensions");
    y.Cp = 1u << clog2(y.C);
    y.logB = clog2(y.B); y.logCp = clog2(y.Cp); y.logHD = clog2(y.HD);
    y.nhb = y.logCp >= y.logHD ? y.logCp - y.logHD : 0;
    y.NH = y.C / y.HD;
    return y;
}
// the layout rules of the reference (layout_guards); the empty string when they hold
std::string layout_error(const Lay& y, size_t big, size_t small) {
    if (y.B != (1u << y.logB)) return "B not a power of two";
    if (y.HD < 2 || y.HD != (1u << y.logHD)) return "HD must be a power of two >= 2";
    if (y.C % y.HD) return "HD must divide C";
    if (y.Cp % y.HD) return "HD must divide C_pad";
    if (y.C / y.HD < 2) return "NH = C/HD must be >= 2";
    if (big != (size_t)y.Cp * G1B) return "gen_big size != C_pad";
    if (small != (size_t)y.HD * G1B) return "gen_small size != HD";
    if (big != (size_t)y.B * G1B && small != (size_t)y.B * G1B) return "no generator set of size B for the KhT commitments";
    return "";
}
std::vector<int32_t> load_exact(const std::string& path, size_t expect) {
    const std::vector<uint8_t> raw = read_file(path);
    if (raw.size() != expect * 4) throw std::runtime_error("file size != expected int32 count: " + path);
    std::vector<int32_t> v(expect);
    memcpy(v.data(), raw.data(), raw.size());
    return v;
}
// (v_d || bits(h) || v_t), the bits of h lowest first
std::vector<Fr> full_point(const std::vector<Fr>& v_d, const std::vector<Fr>& v_t, uint32_t h, uint32_t nhb) {
    std::vector<Fr> pt(v_d);
    for (uint32_t k = 0; k < nhb; k++) pt.push_back(fr_u32((h >> k) & 1u));
    pt.insert(pt.end(), v_t.begin(), v_t.end());
    return pt;
}
std::vector<Fr> lift32(const std::vector<int32_t>& v) {
    std::vector<Fr> o(v.size());
    for (size_t i = 0; i < v.size(); i++) o[i] = fr_from_i64(v[i]);
    return o;
}
void absorb_head(Transcript& tr, const Lay& y) { tr.absorb_u32("B", y.B); tr.absorb_u32("C", y.C); tr.absorb_u32("HD", y.HD); }

int do_prove(int argc, char** argv) {
    const ClaimFlags cf = claim_flags(argc, argv);
    argc = cf.base_argc;
    if (argc != 13 && argc != 14) throw std::invalid_argument("prove <obdir> <seed> <Q> <K> <V> <B> <C> <HD> <gen_big> <gen_small> <q.bin> [slice-out-dir]");
    const std::string obdir = argv[2], seed = argv[3], slice_dir = argc == 14 ? argv[13] : "";
    const Lay y = lay_of(argv[7], argv[8], argv[9]);
    const std::vector<int32_t> Qi = load_exact(argv[4], (size_t)y.B * y.C), Ki = load_exact(argv[5], (size_t)y.B * y.C), Vi = load_exact(argv[6], (size_t)y.B * y.C);
    const std::vector<uint8_t> gb = read_file(argv[10]), gs = read_file(argv[11]), q = read_file(argv[12]);
    if (q.size() < G1B) throw std::runtime_error("q.bin holds no point");
    const std::string le = layout_error(y, gb.size(), gs.size());
    if (!le.empty()) throw std::runtime_error(le);
    const bool big_is_B = gb.size() == (size_t)y.B * G1B;          // the KhT rows have width B
    // the slice gathers: Qh, Vh as B x HD, KhT as HD x B
    const uint32_t B = y.B, C = y.C, HD = y.HD, NH = y.NH;
    std::vector<std::vector<int32_t>> Qs(NH), Ks(NH), Vs(NH);
    for (uint32_t h = 0; h < NH; h++) {
        Qs[h].resize((size_t)B * HD); Ks[h].resize((size_t)B * HD); Vs[h].resize((size_t)B * HD);
        for (uint32_t t = 0; t < B; t++)
            for (uint32_t d = 0; d < HD; d++) {
                Qs[h][(size_t)t * HD + d] = Qi[(size_t)t * C + HD * h + d];
                Ks[h][(size_t)d * B + t] = Ki[(size_t)t * C + HD * h + d];
                Vs[h][(size_t)t * HD + d] = Vi[(size_t)t * C + HD * h + d];
            }
    }
    if (!slice_dir.empty())
        for (uint32_t h = 0; h < NH; h++) {
            auto wr = [&](const std::string& name, const std::vector<int32_t>& v) {
                std::vector<uint8_t> b(v.size() * 4);
                memcpy(b.data(), v.data(), b.size());
                write_file(slice_dir + "/" + name, b);
            };
            wr("Qh" + hh2(h) + ".i32.bin", Qs[h]); wr("KhT" + hh2(h) + ".i32.bin", Ks[h]); wr("Vh" + hh2(h) + ".i32.bin", Vs[h]);
        }
    Ctx x;
    Dev gbd(x, gb.data(), gb.size()), gsd(x, gs.data(), gs.size());
    const Dev& gBd = big_is_B ? gbd : gsd;
    auto padded = [&](const std::vector<int32_t>& v) { const std::vector<int64_t> w(v.begin(), v.end()); return pad_matrix(w.data(), B, C, B, y.Cp); };
    const std::vector<Fr> Qp = padded(Qi), Kp = padded(Ki), Vp = padded(Vi);
    Dev dQ(x, Qp.data(), Qp.size() * FRB), dK(x, Kp.data(), Kp.size() * FRB), dV(x, Vp.data(), Vp.size() * FRB);
    const std::vector<uint8_t> comQ = commit_rows(x, gbd, dQ, B, y.Cp), comK = commit_rows(x, gbd, dK, B, y.Cp), comV = commit_rows(x, gbd, dV, B, y.Cp);
    write_file(obdir + "/com_Q.bin", comQ); write_file(obdir + "/com_K.bin", comK); write_file(obdir + "/com_V.bin", comV);
    std::vector<std::vector<Fr>> Qf(NH), Kf(NH), Vf(NH);
    std::vector<std::unique_ptr<Dev>> dQh(NH), dKh(NH), dVh(NH);
    std::vector<std::vector<uint8_t>> comQh(NH), comKh(NH), comVh(NH);
    for (uint32_t h = 0; h < NH; h++) {
        Qf[h] = lift32(Qs[h]); Kf[h] = lift32(Ks[h]); Vf[h] = lift32(Vs[h]);
        dQh[h].reset(new Dev(x, Qf[h].data(), Qf[h].size() * FRB));
        dKh[h].reset(new Dev(x, Kf[h].data(), Kf[h].size() * FRB));
        dVh[h].reset(new Dev(x, Vf[h].data(), Vf[h].size() * FRB));
        comQh[h] = commit_rows(x, gsd, *dQh[h], B, HD);
        comKh[h] = commit_rows(x, gBd, *dKh[h], HD, B);
        comVh[h] = commit_rows(x, gsd, *dVh[h], B, HD);
        write_file(obdir + "/com_Qh" + hh2(h) + ".bin", comQh[h]);
        write_file(obdir + "/com_KhT" + hh2(h) + ".bin", comKh[h]);
        write_file(obdir + "/com_Vh" + hh2(h) + ".bin", comVh[h]);
    }
    { std::vector<uint8_t> f; const uint32_t dm[3] = {B, C, HD}; put(f, dm, 12); write_file(obdir + "/dims.bin", f); }

    Transcript tr(seed);
    absorb_head(tr, y);
    tr.absorb("com_Q", comQ.data(), comQ.size()); tr.absorb("com_K", comK.data(), comK.size()); tr.absorb("com_V", comV.data(), comV.size());
    for (uint32_t h = 0; h < NH; h++) {
        tr.absorb(("com_Qh" + hh2(h)).c_str(), comQh[h].data(), comQh[h].size());
        tr.absorb(("com_KhT" + hh2(h)).c_str(), comKh[h].data(), comKh[h].size());
        tr.absorb(("com_Vh" + hh2(h)).c_str(), comVh[h].data(), comVh[h].size());
    }
    const std::vector<Fr> v = tr.challenge_vec(y.logHD + y.logB);
    const std::vector<Fr> v_d(v.begin(), v.begin() + y.logHD), v_t(v.begin() + y.logHD, v.end()), vdt(v);
    std::vector<Fr> vtd(v_t);
    vtd.insert(vtd.end(), v_d.begin(), v_d.end());
    const std::vector<Fr> none;
    std::vector<Fr> evals;
    for (uint32_t h = 0; h < NH; h++) {
        const std::vector<Fr> fpt = full_point(v_d, v_t, h, y.nhb);
        const std::string t = hh2(h);
        Fr eQ, eK, eV;
        x.ck(zkh_fr_mle_eval(x.c, dQh[h]->p, vdt.data(), (uint32_t)vdt.size(), eQ.v), "eQ");
        x.ck(zkh_fr_mle_eval(x.c, dKh[h]->p, vtd.data(), (uint32_t)vtd.size(), eK.v), "eK");
        x.ck(zkh_fr_mle_eval(x.c, dVh[h]->p, vdt.data(), (uint32_t)vdt.size(), eV.v), "eV");
        struct Pair { const char* name; const Fr* e; Dev* slice; const Dev* sgen; uint32_t srows, sG; const std::vector<Fr>* spt; const char* scom; Dev* full; const char* fcom; };
        const Pair pairs[3] = {{"Q", &eQ, dQh[h].get(), &gsd, B, HD, &vdt, "/com_Qh", &dQ, "/com_Q.bin"},
                               {"K", &eK, dKh[h].get(), &gBd, HD, B, &vtd, "/com_KhT", &dK, "/com_K.bin"},
                               {"V", &eV, dVh[h].get(), &gsd, B, HD, &vdt, "/com_Vh", &dV, "/com_V.bin"}};
        for (const Pair& p : pairs) {
            tr.absorb_fr((std::string("e") + p.name + t).c_str(), *p.e);
            if (cf.on()) {                                          // both members of the pair carry the SAME absorbed evaluation
                claim_emit(cf.accdir, make_claim(cf.obid, (std::string(p.name) + "h" + t).c_str(), obdir + p.scom + t + ".bin", p.sG, p.srows, *p.spt, none, *p.e));
                claim_emit(cf.accdir, make_claim(cf.obid, (std::string(p.name) + "f" + t).c_str(), obdir + p.fcom, y.Cp, B, fpt, none, *p.e));
            } else {
                open_prove(x, *p.slice, p.srows, p.sG, *p.sgen, q.data(), *p.spt, obdir + "/ipa_" + p.name + "h" + t + ".bin", tr);
                open_prove(x, *p.full, B, y.Cp, gbd, q.data(), fpt, obdir + "/ipa_" + p.name + "f" + t + ".bin", tr);
            }
        }
        evals.push_back(eQ); evals.push_back(eK); evals.push_back(eV);
    }
    save_scalars(obdir + "/evals.bin", evals);
    if (cf.on()) {
        auto wref = [&](const std::string& tag, const std::string& comref, const std::vector<Fr>& t) {
            const std::string wit = cf.accdir + "/wit_" + cf.obid + "_" + tag + ".fr";
            save_scalars(wit, t);
            witref_emit(cf.accdir, comref, wit);
        };
        wref("Q", obdir + "/com_Q.bin", Qp); wref("K", obdir + "/com_K.bin", Kp); wref("V", obdir + "/com_V.bin", Vp);
        for (uint32_t h = 0; h < NH; h++) {
            wref("Qh" + hh2(h), obdir + "/com_Qh" + hh2(h) + ".bin", Qf[h]);
            wref("Kh" + hh2(h), obdir + "/com_KhT" + hh2(h) + ".bin", Kf[h]);
            wref("Vh" + hh2(h), obdir + "/com_Vh" + hh2(h) + ".bin", Vf[h]);
        }
        drvstate_emit(cf.accdir, cf.obid, tr.st);
        std::cout << "PROVED headslice obligation (claim mode, " << 6 * NH << " claims emitted) -> " << obdir << std::endl;
        return 0;
    }
    std::cout << "PROVED headslice obligation -> " << obdir << std::endl;
    return 0;
}

bool verify(const std::string& obdir, const std::string& seed, const Lay& y, const std::vector<uint8_t>& gb, const std::vector<uint8_t>& gs,
            const std::vector<uint8_t>& q, const ClaimFlags& cf) {
    if (!layout_error(y, gb.size(), gs.size()).empty()) return rj("bad layout params");
    const uint32_t B = y.B, HD = y.HD, NH = y.NH;
    {
        const std::vector<uint8_t> f = read_file(obdir + "/dims.bin");
        uint32_t dm[3];
        if (f.size() < 12) return rj("dims.bin short read");
        memcpy(dm, f.data(), 12);
        if (dm[0] != B || dm[1] != y.C || dm[2] != HD) return rj("dims.bin mismatch");
    }
    const std::vector<uint8_t> comQ = read_file(obdir + "/com_Q.bin"), comK = read_file(obdir + "/com_K.bin"), comV = read_file(obdir + "/com_V.bin");
    if (comQ.size() != (size_t)B * G1B || comK.size() != (size_t)B * G1B || comV.size() != (size_t)B * G1B) return rj("full-tensor commitment row counts");
    std::vector<std::vector<uint8_t>> comQh(NH), comKh(NH), comVh(NH);
    for (uint32_t h = 0; h < NH; h++) {
        comQh[h] = read_file(obdir + "/com_Qh" + hh2(h) + ".bin");
        comKh[h] = read_file(obdir + "/com_KhT" + hh2(h) + ".bin");
        comVh[h] = read_file(obdir + "/com_Vh" + hh2(h) + ".bin");
        if (comQh[h].size() != (size_t)B * G1B || comKh[h].size() != (size_t)HD * G1B || comVh[h].size() != (size_t)B * G1B)
            return rj("slice commitment row counts (head " + hh2(h) + ")");
    }
    std::vector<Fr> evals((size_t)3 * NH);
    {
        const std::vector<uint8_t> f = read_file(obdir + "/evals.bin");
        if (f.size() != evals.size() * FRB) return rj("evals.bin size");
        memcpy(evals.data(), f.data(), f.size());
        for (const Fr& e : evals) if (!fr_lt(e, FR_MOD)) return rj("non-canonical evaluation");
    }
    Transcript tr(seed);
    absorb_head(tr, y);
    tr.absorb("com_Q", comQ.data(), comQ.size()); tr.absorb("com_K", comK.data(), comK.size()); tr.absorb("com_V", comV.data(), comV.size());
    for (uint32_t h = 0; h < NH; h++) {
        tr.absorb(("com_Qh" + hh2(h)).c_str(), comQh[h].data(), comQh[h].size());
        tr.absorb(("com_KhT" + hh2(h)).c_str(), comKh[h].data(), comKh[h].size());
        tr.absorb(("com_Vh" + hh2(h)).c_str(), comVh[h].data(), comVh[h].size());
    }
    const std::vector<Fr> v = tr.challenge_vec(y.logHD + y.logB);
    const std::vector<Fr> v_d(v.begin(), v.begin() + y.logHD), v_t(v.begin() + y.logHD, v.end()), vdt(v), none;
    std::vector<Fr> vtd(v_t);
    vtd.insert(vtd.end(), v_d.begin(), v_d.end());
    std::unique_ptr<Ctx> x;
    std::unique_ptr<Dev> gbd, gsd;
    if (!cf.on()) {
        x.reset(new Ctx());
        gbd.reset(new Dev(*x, gb.data(), gb.size()));
        gsd.reset(new Dev(*x, gs.data(), gs.size()));
    }
    const bool big_is_B = gb.size() == (size_t)B * G1B;
    for (uint32_t h = 0; h < NH; h++) {
        const std::vector<Fr> fpt = full_point(v_d, v_t, h, y.nhb);
        const std::string t = hh2(h);
        struct Pair { const char* name; const Fr* e; const std::vector<uint8_t>* scom; bool sgen_big; uint32_t srows, sG; const std::vector<Fr>* spt; const char* sfile;
                      const char* slabel; const std::vector<uint8_t>* fcom; const char* ffile; };
        const Pair pairs[3] = {{"Q", &evals[3 * h], &comQh[h], false, B, HD, &vdt, "/com_Qh", "com_Qh", &comQ, "/com_Q.bin"},
                               {"K", &evals[3 * h + 1], &comKh[h], big_is_B, HD, B, &vtd, "/com_KhT", "com_KhT", &comK, "/com_K.bin"},
                               {"V", &evals[3 * h + 2], &comVh[h], false, B, HD, &vdt, "/com_Vh", "com_Vh", &comV, "/com_V.bin"}};
        for (const Pair& p : pairs) {
            tr.absorb_fr((std::string("e") + p.name + t).c_str(), *p.e);
            if (cf.on()) {
                claim_emit(cf.accdir, make_claim(cf.obid, (std::string(p.name) + "h" + t).c_str(), obdir + p.sfile + t + ".bin", p.sG, p.srows, *p.spt, none, *p.e));
                claim_emit(cf.accdir, make_claim(cf.obid, (std::string(p.name) + "f" + t).c_str(), obdir + p.ffile, y.Cp, B, fpt, none, *p.e));
            } else {
                if (!open_check(*x, *p.scom, p.sG, p.sgen_big ? *gbd : *gsd, q.data(), *p.spt, *p.e, obdir + "/ipa_" + p.name + "h" + t + ".bin", tr))
                    return rj(std::string("IPA opening of e") + p.name + t + " vs " + p.slabel + t);
                if (!open_check(*x, *p.fcom, y.Cp, *gbd, q.data(), fpt, *p.e, obdir + "/ipa_" + p.name + "f" + t + ".bin", tr))
                    return rj(std::string("IPA opening of e") + p.name + t + " vs com_" + p.name + " (head-selector point)");
            }
        }
    }
    if (cf.on()) {
        drvstate_emit(cf.accdir, cf.obid, tr.st);
        std::cout << "ACCEPT-conditional (" << 6 * NH << " claims emitted; final verdict gated on opening_batch)" << std::endl;
        return true;
    }
    std::cout << "ACCEPT" << std::endl;
    return true;
}

int do_verify(int argc, char** argv) {
    const ClaimFlags cf = claim_flags(argc, argv);
    argc = cf.base_argc;
    if (argc != 10) throw std::invalid_argument("verify <obdir> <seed> <B> <C> <HD> <gen_big> <gen_small> <q.bin>");
    const Lay y = lay_of(argv[4], argv[5], argv[6]);
    const std::vector<uint8_t> gb = read_file(argv[7]), gs = read_file(argv[8]), q = read_file(argv[9]);
    if (q.size() < G1B) throw std::runtime_error("q.bin holds no point");
    return verify(argv[2], argv[3], y, gb, gs, q, cf) ? 0 : 1;
}

int run1(int argc, char** argv) {
    const std::string mode = argc > 1 ? argv[1] : "";
    try {
        if (mode == "prove") return do_prove(argc, argv);
        if (mode == "verify") return do_verify(argc, argv);
    } catch (const std::invalid_argument& e) {
        std::cerr << "zkob_headslice: " << e.what() << std::endl;
        return 2;
    }
    std::cerr << "usage: zkob_headslice prove ... [--claims <accdir> <obid>] | verify ... [--claims <vaccdir> <obid>] | serve" << std::endl;
    return 2;
}

}  // namespace

int main(int argc, char** argv) {
    try {
        if (argc > 1 && std::string(argv[1]) == "serve") return serve_loop(argv[0], run1);
        return run1(argc, argv);
    } catch (const std::exception& e) {
        std::cerr << "zkob_headslice: " << e.what() << std::endl;
        return 3;
    }
}
