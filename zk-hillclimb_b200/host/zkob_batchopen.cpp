// The opening_batch program of the reference's first proof stack: ONE batch-evaluation sumcheck over every claim the
// claim-mode drivers put into an accumulator directory, then ONE inner-product argument per generator domain over the
// homomorphic combination of the row-folded tensors (zkllm-src/zkob_batchopen.cu:17-30, protocol in zkob_claims.cuh:832-1061
// prove, :1063-1274 verify), with the reference's command line, files and exit codes.
//
//   zkob_batchopen prove  <accdir> <run_seed> <q.bin> <G>=<gen.bin> ...
//   zkob_batchopen verify <prover-accdir> <verifier-accdir> <run_seed> <q.bin> <G>=<gen.bin> ...
//   zkob_batchopen genq   <out.bin>
//   zkob_batchopen serve
//
// prove reads claims.bin, drvstates.bin, witrefs.txt and the witness tensors and writes batch_sumcheck.bin, batch_vfin.bin and
// ipa_batch_<G>.bin (byte for byte the reference's).  verify takes the claim list the VERIFIER recomputed, compares the
// prover's claims.bin with it byte for byte, and answers "opening_batch ACCEPT" (exit 0) or "REJECT[opening_batch.<locus>]"
// (exit 1) with the reference's locus names.  The transcript is seeded "<run_seed>:opening_batch".  The weight sub-batch over
// committed evaluations (wprove / wverify) is not built: those modes answer exit code 2.
//
// Schedule: absorb the claim count, every claim, the SHA-256 of every distinct commitment file, every driver state -> rho;
// M_j = sum_i rho^i eq(point_i) per tensor; m_max rounds over sum_j M_j P_j (a tensor with fewer variables contributes the
// constant c2_j S_j (1 - T)^2 until its own variables come up); terminal values v'_j; rho'; per domain the vector
// a_G = sum_j rho'^j kappa_j rowfold(P_j) and its argument against the generators.
#include "zkob_common.hpp"

#include <map>
#include <memory>
#include <set>

using namespace zkob;

namespace {

struct Tensor {
    std::string comref;
    uint32_t domain = 0, n_rows = 0, vars = 0, logG = 0;
    std::vector<uint32_t> claim_idx;
};
// distinct tensors in order of first appearance; claims on one tensor must agree on its shape (derive_tensors)
bool derive_tensors(const std::vector<Claim>& cs, std::vector<Tensor>& out, std::string& err) {
    out.clear();
    std::map<std::string, uint32_t> key;
    for (uint32_t i = 0; i < cs.size(); i++) {
        const Claim& c = cs[i];
        if (c.domain < 2 || (c.domain & (c.domain - 1))) { err = "claim " + c.id + ": domain not a power of two >= 2"; return false; }
        const uint32_t logG = clog2(c.domain), vars = (uint32_t)c.point.size();
        if (vars < logG) { err = "claim " + c.id + ": point shorter than logG"; return false; }
        if (vars - logG >= 32 || c.n_rows != (1u << (vars - logG))) { err = "claim " + c.id + ": n_rows != 2^{vars-logG}"; return false; }
        auto it = key.find(c.comref);
        if (it == key.end()) {
            Tensor t;
            t.comref = c.comref; t.domain = c.domain; t.n_rows = c.n_rows; t.vars = vars; t.logG = logG;
            t.claim_idx.push_back(i);
            key[c.comref] = (uint32_t)out.size();
            out.push_back(t);
        } else {
            Tensor& t = out[it->second];
            if (t.domain != c.domain || t.n_rows != c.n_rows || t.vars != vars) {
                err = "claim " + c.id + ": shape disagrees with earlier claim on same tensor"; return false;
            }
            t.claim_idx.push_back(i);
        }
    }
    return true;
}
std::map<uint32_t, std::string> gen_specs(int argc, char** argv, int from) {
    std::map<uint32_t, std::string> m;
    for (int i = from; i < argc; i++) {
        const std::string s = argv[i];
        const size_t eq = s.find('=');
        if (eq == std::string::npos) throw std::invalid_argument("bad gen spec (want <G>=<file>): " + s);
        m[(uint32_t)std::stoul(s.substr(0, eq))] = s.substr(eq + 1);
    }
    return m;
}
std::map<std::string, std::string> witrefs_load(const std::string& accdir) {
    std::map<std::string, std::string> m;
    const std::vector<uint8_t> b = read_file(accdir + "/witrefs.txt");
    const std::string all((const char*)b.data(), b.size());
    size_t pos = 0;
    while (pos < all.size()) {
        size_t nl = all.find('\n', pos);
        if (nl == std::string::npos) nl = all.size();
        const std::string line = all.substr(pos, nl - pos);
        pos = nl + 1;
        const size_t tab = line.find('\t');
        if (tab != std::string::npos) m[line.substr(0, tab)] = line.substr(tab + 1);
    }
    return m;
}
// the first absorbs of the batch transcript (batch_absorb_g0)
void absorb_g0(Transcript& tr, const std::vector<Claim>& cs, const std::vector<Tensor>& ts, const std::vector<DrvState>& dss) {
    tr.absorb_u32("n_claims", (uint32_t)cs.size());
    for (const Claim& c : cs) { const std::vector<uint8_t> b = claim_blob(c); tr.absorb("claim", b.data(), b.size()); }
    for (const Tensor& t : ts) {
        std::vector<uint8_t> b;
        put_u32(b, (uint32_t)t.comref.size()); put(b, t.comref.data(), t.comref.size());
        const std::vector<uint8_t> file = read_file(t.comref);
        uint8_t h[32];
        zkh_tr_init(h, file.data(), file.size());                   // SHA-256 of the commitment file
        put(b, h, 32);
        tr.absorb("comref", b.data(), b.size());
    }
    for (const DrvState& d : dss) {
        std::vector<uint8_t> b;
        put_u32(b, (uint32_t)d.id.size()); put(b, d.id.data(), d.id.size());
        put(b, d.state, 32);
        tr.absorb("drvstate", b.data(), b.size());
    }
}
std::vector<Fr> powers(const Fr& x, size_t n) {
    std::vector<Fr> p(n);
    if (n) p[0] = fr_u32(1);
    for (size_t i = 1; i < n; i++) p[i] = fr_mul(p[i - 1], x);
    return p;
}
// kappa_j = prod_{v >= vars_j} (1 - r[v]); M_j(r) with the high-variable factors included (bo_kappa, bo_Mj_at_r)
Fr kappa(uint32_t vars, const std::vector<Fr>& r) {
    Fr k = fr_u32(1);
    for (size_t v = vars; v < r.size(); v++) k = fr_mul(k, fr_sub(fr_u32(1), r[v]));
    return k;
}
Fr Mj_at_r(const Tensor& t, const std::vector<Claim>& cs, const std::vector<Fr>& rho_pows, const std::vector<Fr>& r) {
    const Fr kap = kappa(t.vars, r);
    Fr acc{};
    for (uint32_t idx : t.claim_idx) {
        Fr term = rho_pows[idx];
        for (uint32_t v = 0; v < t.vars; v++) term = fr_mul(term, eq1(cs[idx].point[v], r[v]));
        acc = fr_add(acc, fr_mul(term, kap));
    }
    return acc;
}
std::string batch_ipa_path(const std::string& dir, uint32_t G) { return dir + "/ipa_batch_" + std::to_string(G) + ".bin"; }

int do_prove(int argc, char** argv) {
    if (argc < 5) throw std::invalid_argument("prove <accdir> <run_seed> <q.bin> <G>=<gen.bin> ...");
    const std::string accdir = argv[2], run_seed = argv[3];
    const std::map<uint32_t, std::string> genpaths = gen_specs(argc, argv, 5);
    const std::vector<Claim> cs = claims_load(accdir + "/claims.bin");
    if (cs.empty()) throw std::runtime_error("batch_prove: zero claims");
    std::vector<Tensor> ts;
    std::string err;
    if (!derive_tensors(cs, ts, err)) throw std::runtime_error("batch_prove: " + err);
    std::vector<DrvState> dss;
    if (file_exists(accdir + "/drvstates.bin")) dss = drvstates_load(accdir + "/drvstates.bin");
    const std::map<std::string, std::string> wits = witrefs_load(accdir);
    const std::vector<uint8_t> q = read_file(argv[4]);
    if (q.size() < G1B) throw std::runtime_error("q.bin holds no point");
    uint32_t m_max = 0;
    for (const Tensor& t : ts) m_max = std::max(m_max, t.vars);
    const uint32_t nT = (uint32_t)ts.size();
    std::vector<std::string> witpath(nT);
    for (uint32_t j = 0; j < nT; j++) {
        auto it = wits.find(ts[j].comref);
        if (it == wits.end()) throw std::runtime_error("batch_prove: no witref for " + ts[j].comref);
        witpath[j] = it->second;
    }
    Laps laps("batch_prove");
    Transcript tr(run_seed + ":opening_batch");
    absorb_g0(tr, cs, ts, dss);
    const Fr rho = tr.challenge_fr();
    const std::vector<Fr> rho_pows = powers(rho, cs.size());

    Ctx x;
    // per tensor: M_j = sum_i rho^i eq(point_i), P_j = the witness; S_j = <M_j, P_j> for the tensors with fewer variables
    std::vector<std::unique_ptr<Dev>> M(nT), P(nT);
    std::vector<uint64_t> cur_size(nT);
    std::vector<Fr> c2(nT, fr_u32(1)), S(nT, Fr{});
    {
        Dev eq(x, ((size_t)1 << m_max) * FRB);
        for (uint32_t j = 0; j < nT; j++) {
            const uint64_t n = (uint64_t)1 << ts[j].vars;
            const std::vector<uint8_t> w = read_file(witpath[j]);
            if (w.size() != (size_t)ts[j].n_rows * ts[j].domain * FRB) throw std::runtime_error("batch_prove: witness size mismatch for " + ts[j].comref);
            P[j].reset(new Dev(x, w.data(), w.size()));
            const std::vector<uint8_t> zero(w.size(), 0);
            M[j].reset(new Dev(x, zero.data(), zero.size()));
            cur_size[j] = n;
            for (uint32_t idx : ts[j].claim_idx) {
                x.ck(zkh_fr_eq_build(x.c, cs[idx].point.data(), ts[j].vars, eq.p), "eq table");
                x.ck(zkh_fr_axpy(x.c, M[j]->p, eq.p, rho_pows[idx].v, n), "M_j");
            }
            if (ts[j].vars < m_max) x.ck(zkh_fr_dot(x.c, M[j]->p, P[j]->p, n, S[j].v), "S_j");
        }
    }
    laps.lap("setup");
    Fr cur{};
    for (size_t i = 0; i < cs.size(); i++) cur = fr_add(cur, fr_mul(rho_pows[i], cs[i].eval));

    // rounds: round t binds variable v = m_max - 1 - t
    std::vector<Fr> ev, r(m_max, Fr{});
    for (uint32_t t = 0; t < m_max; t++) {
        const uint32_t v = m_max - 1 - t;
        Fr p0{}, p1{}, p2{};
        for (uint32_t j = 0; j < nT; j++) {
            if (ts[j].vars <= v) {                                  // both factors carry (1 - x_v): + S at T = 0 and 2, nothing at 1
                const Fr term = fr_mul(c2[j], S[j]);
                p0 = fr_add(p0, term);
                p2 = fr_add(p2, term);
            } else {
                Fr qv[3];
                x.ck(zkh_fr_round_sums(x.c, M[j]->p, P[j]->p, cur_size[j] / 2, qv), "round sums");
                p0 = fr_add(p0, fr_mul(c2[j], qv[0]));
                p1 = fr_add(p1, fr_mul(c2[j], qv[1]));
                p2 = fr_add(p2, fr_mul(c2[j], qv[2]));
            }
        }
        if (!fr_eq(cur, fr_add(p0, p1))) throw std::runtime_error("batch_prove: round " + std::to_string(t) + " inconsistency (witness/claims bug)");
        tr.absorb_fr("bp0", p0); tr.absorb_fr("bp1", p1); tr.absorb_fr("bp2", p2);
        const Fr xr = tr.challenge_fr();
        r[v] = xr;
        ev.push_back(p0); ev.push_back(p1); ev.push_back(p2);
        cur = lagrange3(p0, p1, p2, xr);
        const Fr omx = fr_sub(fr_u32(1), xr), omx2 = fr_mul(omx, omx);
        for (uint32_t j = 0; j < nT; j++) {
            if (ts[j].vars <= v) {
                c2[j] = fr_mul(c2[j], omx2);
            } else {
                const uint64_t half = cur_size[j] / 2;
                for (Dev* d : {M[j].get(), P[j].get()}) x.ck(zkh_fr_fold(x.c, d->p, half, xr.v, d->p), "fold");     // in place
                cur_size[j] = half;
            }
        }
    }
    {
        std::vector<uint8_t> f;
        const uint32_t nc = (uint32_t)cs.size(), ne = (uint32_t)ev.size();
        put(f, "ZKBS", 4); put(f, &nc, 4); put(f, &m_max, 4); put(f, &ne, 4); put(f, ev.data(), ev.size() * FRB);
        write_file(accdir + "/batch_sumcheck.bin", f);
    }
    laps.lap("rounds");
    // terminal values v'_j = P_j(r[0..vars_j)), in tensor order
    std::vector<Fr> vfin(nT);
    for (uint32_t j = 0; j < nT; j++) x.ck(zkh_download(x.c, vfin[j].v, P[j]->p, FRB), "download");
    for (uint32_t j = 0; j < nT; j++) tr.absorb_fr("vfin", vfin[j]);
    {
        std::vector<uint8_t> f;
        put(f, "ZKBV", 4); put(f, &nT, 4); put(f, vfin.data(), vfin.size() * FRB);
        write_file(accdir + "/batch_vfin.bin", f);
        Fr chk{};
        for (uint32_t j = 0; j < nT; j++) chk = fr_add(chk, fr_mul(fr_mul(Mj_at_r(ts[j], cs, rho_pows, r), kappa(ts[j].vars, r)), vfin[j]));
        if (!fr_eq(chk, cur)) throw std::runtime_error("batch_prove: G3 terminal self-check failed");
    }
    for (uint32_t j = 0; j < nT; j++) { M[j].reset(); P[j].reset(); }
    laps.lap("terminal");
    // per generator domain, ascending: a_G = sum_j rho'^j kappa_j rowfold(P_j), one argument against the domain's generators
    const Fr rhop = tr.challenge_fr();
    const std::vector<Fr> rhop_pows = powers(rhop, nT);
    std::set<uint32_t> domains;
    for (const Tensor& t : ts) domains.insert(t.domain);
    for (uint32_t G : domains) {
        const uint32_t logG = clog2(G);
        const std::vector<uint8_t> zero((size_t)G * FRB, 0);
        Dev a(x, zero.data(), zero.size());
        for (uint32_t j = 0; j < nT; j++) {
            if (ts[j].domain != G) continue;
            const Fr coef = fr_mul(rhop_pows[j], kappa(ts[j].vars, r));
            const std::vector<Fr> u_row(r.begin() + logG, r.begin() + ts[j].vars);
            const std::vector<uint8_t> w = read_file(witpath[j]);
            Dev wd(x, w.data(), w.size());
            if (u_row.empty()) {
                x.ck(zkh_fr_axpy(x.c, a.p, wd.p, coef.v, G), "a_G");
            } else {
                Dev rf(x, (size_t)G * FRB);
                partial_me(x, wd, 1, (uint32_t)u_row.size(), G, u_row, rf);
                x.ck(zkh_fr_axpy(x.c, a.p, rf.p, coef.v, G), "a_G");
                x.ck(zkh_ctx_sync(x.c), "sync");
            }
            x.ck(zkh_ctx_sync(x.c), "sync");
        }
        auto git = genpaths.find(G);
        if (git == genpaths.end()) throw std::runtime_error("batch_prove: no generator file for domain " + std::to_string(G));
        const std::vector<uint8_t> g = read_file(git->second);
        if (g.size() != (size_t)G * G1B) throw std::runtime_error("batch_prove: generator size mismatch for domain " + std::to_string(G));
        Dev gd(x, g.data(), g.size());
        ipa_to_file(x, batch_ipa_path(accdir, G), a, std::vector<Fr>(r.begin(), r.begin() + logG), gd, q.data(), G, tr);
    }
    laps.lap("ipa");
    std::cout << "PROVED opening_batch -> " << accdir << std::endl;
    return 0;
}

bool reject(const std::string& locus, const std::string& detail) {
    printf("REJECT[opening_batch.%s]: %s\n", locus.c_str(), detail.c_str());
    fflush(stdout);
    return false;
}

bool verify(const std::string& paccdir, const std::string& vaccdir, const std::string& run_seed, const std::map<uint32_t, std::string>& genpaths,
            const std::string& qpath) {
    std::vector<Claim> cs;
    try {
        cs = claims_load(vaccdir + "/claims.bin");
    } catch (const std::invalid_argument& e) {
        return reject("evalvar", e.what());
    }
    std::vector<DrvState> dss;
    if (file_exists(vaccdir + "/drvstates.bin")) dss = drvstates_load(vaccdir + "/drvstates.bin");
    if (cs.empty()) return reject("empty", "zero claims (a batch over no claims is not a valid obligation)");
    {
        const std::vector<uint8_t> mine = claims_serialize(cs);
        if (!file_exists(paccdir + "/claims.bin")) return reject("claims_match", "prover claims.bin missing");
        if (mine != read_file(paccdir + "/claims.bin")) return reject("claims_match", "prover claim list != verifier-recomputed list");
    }
    std::vector<Tensor> ts;
    std::string err;
    if (!derive_tensors(cs, ts, err)) return reject("shape", err);
    const uint32_t nT = (uint32_t)ts.size();
    uint32_t m_max = 0;
    for (const Tensor& t : ts) m_max = std::max(m_max, t.vars);
    if (m_max < 1) return reject("shape", "m_max < 1");
    const bool require_rel = getenv("ZKOB_REQUIRE_RELATIVE_COMREF") != nullptr;
    std::vector<std::vector<uint8_t>> coms;
    for (const Tensor& t : ts) {
        if (require_rel && !t.comref.empty() && t.comref[0] == '/') return reject("shape", "absolute comref under relative-comref policy: " + t.comref);
        if (!file_exists(t.comref)) return reject("shape", "commitment file missing: " + t.comref);
        coms.push_back(read_file(t.comref));
        if (coms.back().size() / G1B != t.n_rows || coms.back().size() % G1B)
            return reject("shape", "commitment row count " + std::to_string(coms.back().size() / G1B) + " != n_rows " + std::to_string(t.n_rows) + " (" + t.comref + ")");
    }
    std::map<uint32_t, std::vector<uint8_t>> gens;
    for (const Tensor& t : ts) {
        if (gens.count(t.domain)) continue;
        auto git = genpaths.find(t.domain);
        if (git == genpaths.end()) return reject("shape", "no generator file mapped for domain " + std::to_string(t.domain));
        gens[t.domain] = read_file(git->second);
        if (gens[t.domain].size() != (size_t)t.domain * G1B) return reject("shape", "generator file size != domain " + std::to_string(t.domain));
    }
    const std::vector<uint8_t> q = read_file(qpath);
    if (q.size() < G1B) throw std::runtime_error("q.bin holds no point");

    Transcript tr(run_seed + ":opening_batch");
    absorb_g0(tr, cs, ts, dss);
    const Fr rho = tr.challenge_fr();
    const std::vector<Fr> rho_pows = powers(rho, cs.size());

    std::vector<Fr> ev;
    {
        std::vector<uint8_t> f;
        try { f = read_file(paccdir + "/batch_sumcheck.bin"); } catch (const std::exception& e) { return reject("xcheck", e.what()); }
        if (f.size() < 16 || memcmp(f.data(), "ZKBS", 4)) return reject("xcheck", "read_batch_sumcheck: header");
        uint32_t nc, mm, ne;
        memcpy(&nc, &f[4], 4); memcpy(&mm, &f[8], 4); memcpy(&ne, &f[12], 4);
        if (f.size() != 16 + (size_t)ne * FRB) return reject("xcheck", "read_pod_vec: body");
        if (nc != cs.size()) return reject("xcheck", "batch_sumcheck.bin n_claims field != derived claim count");
        if (mm != m_max) return reject("xcheck", "batch_sumcheck.bin m_max field != derived m_max");
        if (ne != 3u * m_max) return reject("xcheck", "batch_sumcheck.bin round-eval count != 3*m_max");
        ev.resize(ne);
        memcpy(ev.data(), &f[16], (size_t)ne * FRB);
        for (const Fr& e : ev) if (!fr_lt(e, FR_MOD)) return reject("xcheck", "non-canonical round evaluation");
    }
    Fr cur{};
    for (size_t i = 0; i < cs.size(); i++) cur = fr_add(cur, fr_mul(rho_pows[i], cs[i].eval));
    std::vector<Fr> r(m_max, Fr{});
    for (uint32_t t = 0; t < m_max; t++) {
        const Fr &p0 = ev[3 * t], &p1 = ev[3 * t + 1], &p2 = ev[3 * t + 2];
        if (!fr_eq(cur, fr_add(p0, p1))) return reject("round" + std::to_string(t), "p(0)+p(1) != running claim");
        tr.absorb_fr("bp0", p0); tr.absorb_fr("bp1", p1); tr.absorb_fr("bp2", p2);
        const Fr xr = tr.challenge_fr();
        r[m_max - 1 - t] = xr;
        cur = lagrange3(p0, p1, p2, xr);
    }
    std::vector<Fr> vfin;
    {
        std::vector<uint8_t> f;
        try { f = read_file(paccdir + "/batch_vfin.bin"); } catch (const std::exception& e) { return reject("vfin_count", e.what()); }
        if (f.size() < 8 || memcmp(f.data(), "ZKBV", 4)) return reject("vfin_count", "read_batch_vfin: header");
        uint32_t n;
        memcpy(&n, &f[4], 4);
        if (f.size() != 8 + (size_t)n * FRB) return reject("vfin_count", "read_pod_vec: body");
        if (n != nT) return reject("vfin_count", "batch_vfin.bin entry count != distinct tensor count");
        vfin.resize(n);
        memcpy(vfin.data(), &f[8], (size_t)n * FRB);
        for (const Fr& e : vfin) if (!fr_lt(e, FR_MOD)) return reject("vfin_count", "non-canonical terminal value");
    }
    for (uint32_t j = 0; j < nT; j++) tr.absorb_fr("vfin", vfin[j]);
    {
        Fr chk{};
        for (uint32_t j = 0; j < nT; j++) chk = fr_add(chk, fr_mul(fr_mul(Mj_at_r(ts[j], cs, rho_pows, r), kappa(ts[j].vars, r)), vfin[j]));
        if (!fr_eq(chk, cur)) return reject("terminal", "sum_j M_j(r)*kappa_j*v'_j != running claim");
    }
    const Fr rhop = tr.challenge_fr();
    const std::vector<Fr> rhop_pows = powers(rhop, nT);
    std::set<uint32_t> domains;
    for (const Tensor& t : ts) domains.insert(t.domain);
    Ctx x;
    for (uint32_t G : domains) {
        const uint32_t logG = clog2(G);
        const std::string ipath = batch_ipa_path(paccdir, G);
        if (!file_exists(ipath)) return reject("group_missing", "ipa_batch_" + std::to_string(G) + ".bin missing");
        // P0 = sum_j coef_j fold(com_j) + v* Q as a group element: each tensor's rows folded by one multi-scalar product with the
        // equality weights of its row point, then one product over the folded points and Q (padded to a power of two with
        // zero scalars)
        std::vector<uint8_t> pts;
        std::vector<Fr> scal;
        Fr vstar{};
        for (uint32_t j = 0; j < nT; j++) {
            if (ts[j].domain != G) continue;
            const Fr coef = fr_mul(rhop_pows[j], kappa(ts[j].vars, r));
            const std::vector<Fr> u_row(r.begin() + logG, r.begin() + ts[j].vars);
            uint8_t cj[G1B];
            if (u_row.empty()) {
                memcpy(cj, coms[j].data(), G1B);
            } else {
                Dev cd(x, coms[j].data(), coms[j].size()), wd(x, (size_t)ts[j].n_rows * FRB);
                x.ck(zkh_fr_eq_build(x.c, u_row.data(), (uint32_t)u_row.size(), wd.p), "row weights");
                x.ck(zkh_g1_msm(x.c, cd.p, wd.p, ts[j].n_rows, cj), "folded commitment");
            }
            put(pts, cj, G1B);
            scal.push_back(coef);
            vstar = fr_add(vstar, fr_mul(coef, vfin[j]));
        }
        put(pts, q.data(), G1B);
        scal.push_back(vstar);
        uint32_t np = 1;
        while (np < scal.size()) np <<= 1;
        while (scal.size() < np) { put(pts, q.data(), G1B); scal.push_back(Fr{}); }
        uint8_t P0[G1B];
        {
            Dev pd(x, pts.data(), pts.size()), sd(x, scal.data(), scal.size() * FRB);
            x.ck(zkh_g1_msm(x.c, pd.p, sd.p, np, P0), "statement point");
        }
        Ipa pf;
        try { pf = read_ipa(ipath); } catch (const std::exception& e) { return reject("ipa" + std::to_string(G), e.what()); }
        bool ok = pf.rounds == logG && fr_lt(pf.af, FR_MOD);
        if (ok) {
            Dev gd(x, gens[G].data(), gens[G].size());
            const std::vector<Fr> u_b(r.begin(), r.begin() + logG);
            int acc = 0;
            x.ck(zkh_g1_ipa_verify(x.c, gd.p, G, q.data(), P0, u_b.data(), pf.L.data(), pf.R.data(), pf.af.v, tr.st, &acc), "ipa_verify");
            ok = acc == 1;
        }
        if (!ok) return reject("ipa" + std::to_string(G), "batched IPA for domain " + std::to_string(G) + " failed");
    }
    printf("opening_batch ACCEPT (%u claims, %u tensors, %zu domains)\n", (unsigned)cs.size(), nT, domains.size());
    fflush(stdout);
    return true;
}

// q.bin with two slots (Q and the H slot of the hiding modes): two multiples of the group's generator by fresh random scalars
int do_genq(const char* out) {
    static const uint32_t GEN[36] = {
        0xfd530c16u, 0x5cb38790u, 0x9976fff5u, 0x7817fc67u, 0x143ba1c1u, 0x154f95c7u, 0xf3d0e747u, 0xf0ae6acdu, 0x21dbf440u,
        0xedce6eccu, 0x9e0bfb75u, 0x12017741u, 0x0ce72271u, 0xbaac93d5u, 0x7918fd8eu, 0x8c22631au, 0x570725ceu, 0xdd595f13u,
        0x50405194u, 0x51ac5829u, 0xad0059c0u, 0x0e1c8c3fu, 0x5008a26au, 0x0bbc3efcu, 0x0002fffdu, 0x76090000u, 0xc40c0002u,
        0xebf4000bu, 0x53c758bau, 0x5f489857u, 0x70525745u, 0x77ce5853u, 0xa256ec6du, 0x5c071a97u, 0xfa80e493u, 0x15f65ec3u};
    FILE* u = fopen("/dev/urandom", "rb");
    if (!u) throw std::runtime_error("no /dev/urandom");
    Ctx x;
    Dev gd(x, GEN, sizeof GEN);
    std::vector<uint8_t> pts(2 * G1B);
    for (int i = 0; i < 2; i++) {
        Fr k;
        if (fread(k.v, 1, FRB, u) != FRB) { fclose(u); throw std::runtime_error("short read from /dev/urandom"); }
        k.v[7] %= 1944954707u;
        Dev kd(x, k.v, FRB);
        x.ck(zkh_g1_msm(x.c, gd.p, kd.p, 1, &pts[(size_t)i * G1B]), "random point");
    }
    fclose(u);
    write_file(out, pts);
    std::cout << "wrote 2-slot q file (Q + H slot) -> " << out << std::endl;
    return 0;
}

int run1(int argc, char** argv) {
    const std::string mode = argc > 1 ? argv[1] : "";
    try {
        if (mode == "prove") return do_prove(argc, argv);
        if (mode == "verify" && argc >= 6) return verify(argv[2], argv[3], argv[4], gen_specs(argc, argv, 6), argv[5]) ? 0 : 1;
        if (mode == "genq" && argc == 3) return do_genq(argv[2]);
        if (mode == "wprove" || mode == "wverify" || mode == "wselftest") {
            std::cerr << "zkob_batchopen: the weight sub-batch over committed evaluations is not built in this program" << std::endl;
            return 2;
        }
    } catch (const std::exception& e) {
        std::cerr << "ERROR: " << e.what() << std::endl;
        return 2;
    }
    std::cerr << "usage: zkob_batchopen prove <accdir> <run_seed> <q.bin> <G>=<gen.bin> ... | verify <prover-accdir> <verifier-accdir> <run_seed> <q.bin> "
                 "<G>=<gen.bin> ... | genq <out> | serve" << std::endl;
    return 2;
}

}  // namespace

int main(int argc, char** argv) {
    try {
        if (argc > 1 && std::string(argv[1]) == "serve") return serve_loop(argv[0], run1);
        return run1(argc, argv);
    } catch (const std::exception& e) {
        std::cerr << "zkob_batchopen: " << e.what() << std::endl;
        return 3;
    }
}
