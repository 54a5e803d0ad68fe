// C-ABI window onto the UNMODIFIED reference headers (TEST INFRASTRUCTURE ONLY).
//
// Built by oracle/Makefile into oracle/_ref/libp3ref.so with the reference's
// header directory on the include path; no reference source is copied here.
// The host entry points run anywhere (they are the pins for oracle/zkh_oracle.c
// and the source of tests/golden/); the *_gpu entry points call the
// reference's own CUDA code paths and only work on a machine with a GPU,
// where they serve as the "reference CUDA prover" for parity at large sizes
// and as a timing baseline.  Nothing in the product library links to this.
//
// Serialised layouts are the ones documented in oracle/zkh_oracle.h.
#include <cstdint>
#include <cstring>
#include <string>
#include <map>
#include <vector>
#include "p3_goldilocks.cuh"
#include "fs_transcript.hpp"
#include "p3_fri.cuh"
#include "p3_basefold.cuh"
#include "p3_scgpu.cuh"
#include "p3_gkr.cuh"
#include "p3_logup.cuh"
#include "p3_hawkeye.cuh"
#include "p3_int_gadgets.cuh"
#include "p3_int_layer.cuh"
#include "p3_swiglu.cuh"
#include "p3_bfadd.cuh"
#include "p3_quant.cuh"
#include "p3_rope.cuh"
#include "p3_softmax.cuh"
#include "p3_transformer.cuh"
#include "p3_model.cuh"

namespace {
fs::Transcript tr_from(const uint8_t st[32]) {
    fs::Transcript tr(std::string(""));
    memcpy(tr.state, st, 32);
    return tr;
}
void put(uint8_t*& p, const void* src, size_t n) { memcpy(p, src, n); p += n; }

size_t bf_size(uint32_t v, uint32_t R, uint32_t Q) {
    size_t s = 12 + (size_t)v * 32 + (size_t)v * 24 + ((size_t)8 << R);
    for (uint32_t r = 0; r < v; r++) s += (size_t)Q * (16 + 2 * (size_t)(v + R - r) * 32);
    return s + (size_t)v * 8 + 8;
}
size_t bf_serialize(const p3bf::EvalProof& pf, uint8_t* out, size_t cap) {
    size_t need = bf_size(pf.logN, pf.R, pf.Q);
    if (!out) return need;
    if (cap < need) return 0;
    uint8_t* p = out;
    put(p, &pf.logN, 4); put(p, &pf.R, 4); put(p, &pf.Q, 4);
    for (auto& h : pf.roots) put(p, h.data(), 32);
    for (auto& m : pf.msgs) put(p, &m, 24);
    put(p, pf.final_word.data(), pf.final_word.size() * 8);
    for (auto& q : pf.queries)
        for (auto& ro : q.rounds) {
            put(p, &ro.a, 8); put(p, &ro.b, 8);
            for (auto& h : ro.pa) put(p, h.data(), 32);
            for (auto& h : ro.pb) put(p, h.data(), 32);
        }
    put(p, pf.z.data(), pf.z.size() * 8);
    put(p, &pf.y, 8);
    return (size_t)(p - out);
}
bool bf_deserialize(const uint8_t* in, size_t len, p3bf::EvalProof& pf) {
    if (len < 12) return false;
    const uint8_t* p = in;
    memcpy(&pf.logN, p, 4); memcpy(&pf.R, p + 4, 4); memcpy(&pf.Q, p + 8, 4); p += 12;
    uint32_t v = pf.logN, R = pf.R, Q = pf.Q;
    if (v > 40 || R > 8 || len != bf_size(v, R, Q)) return false;
    pf.roots.resize(v);
    for (auto& h : pf.roots) { memcpy(h.data(), p, 32); p += 32; }
    pf.msgs.resize(v);
    for (auto& m : pf.msgs) { memcpy(&m, p, 24); p += 24; }
    pf.final_word.resize((size_t)1 << R);
    memcpy(pf.final_word.data(), p, pf.final_word.size() * 8); p += pf.final_word.size() * 8;
    pf.queries.resize(Q);
    for (auto& q : pf.queries) {
        q.rounds.resize(v);
        for (uint32_t r = 0; r < v; r++) {
            auto& ro = q.rounds[r];
            memcpy(&ro.a, p, 8); memcpy(&ro.b, p + 8, 8); p += 16;
            uint32_t plen = v + R - r;
            ro.pa.resize(plen); ro.pb.resize(plen);
            for (auto& h : ro.pa) { memcpy(h.data(), p, 32); p += 32; }
            for (auto& h : ro.pb) { memcpy(h.data(), p, 32); p += 32; }
        }
    }
    pf.z.resize(v);
    memcpy(pf.z.data(), p, (size_t)v * 8); p += (size_t)v * 8;
    memcpy(&pf.y, p, 8);
    return true;
}
size_t gkr_size(uint32_t L) {
    size_t s = 16;
    for (uint32_t h = L; h >= 1; h--) s += 4 + (size_t)(L - h) * 32 + 32;
    return s;
}
size_t gkr_serialize(const p3gkr::Proof& pf, uint8_t* out, size_t cap) {
    uint32_t L = (uint32_t)pf.lay.size();
    if (cap < gkr_size(L)) return 0;
    uint8_t* p = out;
    put(p, &pf.P, 8); put(p, &pf.Q, 8);
    for (auto& ly : pf.lay) {
        uint32_t nm = (uint32_t)ly.msgs.size();
        put(p, &nm, 4);
        for (auto& m : ly.msgs) put(p, &m, 32);
        gl_t t[4] = {ly.p0, ly.p1, ly.q0, ly.q1};
        put(p, t, 32);
    }
    return (size_t)(p - out);
}
bool gkr_deserialize(const uint8_t* in, size_t len, uint32_t L, p3gkr::Proof& pf) {
    if (len != gkr_size(L)) return false;
    const uint8_t* p = in;
    memcpy(&pf.P, p, 8); memcpy(&pf.Q, p + 8, 8); p += 16;
    pf.lay.resize(L);
    for (auto& ly : pf.lay) {
        uint32_t nm; memcpy(&nm, p, 4); p += 4;
        if (nm > L) return false;
        ly.msgs.resize(nm);
        for (auto& m : ly.msgs) { memcpy(&m, p, 32); p += 32; }
        gl_t t[4]; memcpy(t, p, 32); p += 32;
        ly.p0 = t[0]; ly.p1 = t[1]; ly.q0 = t[2]; ly.q1 = t[3];
    }
    return true;
}
// BatchProof <-> the byte layout documented in oracle/zkh_oracle.c (non-zk fields)
size_t bo_serialize(const p3bo::BatchProof& pf, uint8_t* out, size_t cap) {
    std::vector<uint8_t> b;
    auto app = [&](const void* s, size_t n) { const uint8_t* q = (const uint8_t*)s; b.insert(b.end(), q, q + n); };
    app(&pf.v, 4); app(&pf.R, 4); app(&pf.Q, 4); app(&pf.nc, 4);
    app(pf.ystar.data(), pf.ystar.size() * 8);
    for (auto& m : pf.rmsgs) app(&m, 24);
    for (auto& h : pf.roots) app(h.data(), 32);
    for (auto& m : pf.omsgs) app(&m, 24);
    app(pf.final_word.data(), pf.final_word.size() * 8);
    for (auto& q : pf.queries)
        for (auto& ro : q.rounds) {
            app(&ro.a, 8); app(&ro.b, 8);
            for (auto& h : ro.pa) app(h.data(), 32);
            for (auto& h : ro.pb) app(h.data(), 32);
        }
    for (auto& oc : pf.q0c) {
        uint32_t nv = (uint32_t)oc.vals.size(), nn = (uint32_t)oc.nodes.size();
        app(&nv, 4); app(oc.vals.data(), (size_t)nv * 8);
        if (p3zkc::G.on) for (auto& sl : oc.salts) app(sl.data(), 32);
        app(&nn, 4);
        for (auto& h : oc.nodes) app(h.data(), 32);
    }
    if (p3zkc::G.on) { app(pf.bl_root.data(), 32); app(&pf.bl_y, 8); }
    if (b.size() > cap) return 0;
    memcpy(out, b.data(), b.size());
    return b.size();
}
bool bo_deserialize(const uint8_t* in, size_t len, p3bo::BatchProof& pf) {
    const uint8_t* p = in; const uint8_t* end = in + len;
    auto need = [&](size_t n) { return (size_t)(end - p) >= n; };
    if (!need(16)) return false;
    memcpy(&pf.v, p, 4); memcpy(&pf.R, p + 4, 4); memcpy(&pf.Q, p + 8, 4); memcpy(&pf.nc, p + 12, 4); p += 16;
    uint32_t v = pf.v, R = pf.R, Q = pf.Q, nc = pf.nc;
    if (v > 40 || R > 8 || Q > 4096 || nc > (1u << 20)) return false;
    if (!need((size_t)nc * 8)) return false;
    pf.ystar.resize(nc); memcpy(pf.ystar.data(), p, (size_t)nc * 8); p += (size_t)nc * 8;
    if (!need((size_t)v * 24)) return false;
    pf.rmsgs.resize(v); for (auto& m : pf.rmsgs) { memcpy(&m, p, 24); p += 24; }
    uint32_t nr = v ? v - 1 : 0;
    if (!need((size_t)nr * 32)) return false;
    pf.roots.resize(nr); for (auto& h : pf.roots) { memcpy(h.data(), p, 32); p += 32; }
    if (!need((size_t)v * 24)) return false;
    pf.omsgs.resize(v); for (auto& m : pf.omsgs) { memcpy(&m, p, 24); p += 24; }
    if (!need((size_t)8 << R)) return false;
    pf.final_word.resize((size_t)1 << R); memcpy(pf.final_word.data(), p, (size_t)8 << R); p += (size_t)8 << R;
    pf.queries.resize(Q);
    for (auto& q : pf.queries) {
        q.rounds.resize(nr);
        for (uint32_t r = 1; r < v; r++) {
            auto& ro = q.rounds[r - 1];
            uint32_t plen = v + R - r;
            if (!need(16 + (size_t)2 * plen * 32)) return false;
            memcpy(&ro.a, p, 8); memcpy(&ro.b, p + 8, 8); p += 16;
            ro.pa.resize(plen); ro.pb.resize(plen);
            for (auto& h : ro.pa) { memcpy(h.data(), p, 32); p += 32; }
            for (auto& h : ro.pb) { memcpy(h.data(), p, 32); p += 32; }
        }
    }
    pf.q0c.resize(nc);
    for (auto& oc : pf.q0c) {
        uint32_t nv, nn;
        if (!need(4)) return false;
        memcpy(&nv, p, 4); p += 4;
        if (!need((size_t)nv * 8 + 4)) return false;
        oc.vals.resize(nv); memcpy(oc.vals.data(), p, (size_t)nv * 8); p += (size_t)nv * 8;
        if (p3zkc::G.on) {
            if (!need((size_t)nv * 32 + 4)) return false;
            oc.salts.resize(nv);
            for (auto& sl : oc.salts) { memcpy(sl.data(), p, 32); p += 32; }
        }
        memcpy(&nn, p, 4); p += 4;
        if (!need((size_t)nn * 32)) return false;
        oc.nodes.resize(nn); for (auto& h : oc.nodes) { memcpy(h.data(), p, 32); p += 32; }
    }
    if (p3zkc::G.on) {
        if (!need(40)) return false;
        memcpy(pf.bl_root.data(), p, 32); memcpy(&pf.bl_y, p + 32, 8); p += 40;
    }
    return p == end;
}
// p3zkc::Blind <-> bytes: u32 nb | nb == 5: four roots, else one | H | nb == 6: ystar, else yB[4] |
//                         nb == 6: u32 rounds, rounds x 24 bytes, yw
void blind_serialize(const p3zkc::Blind& bl, std::vector<uint8_t>& b) {
    auto app = [&](const void* s, size_t n) { const uint8_t* q = (const uint8_t*)s; b.insert(b.end(), q, q + n); };
    app(&bl.nb, 4);
    for (uint32_t j = 0; j < (bl.nb == 5 ? 4u : 1u); j++) app(bl.rt[j].data(), 32);
    app(&bl.H, 8);
    app(bl.yB, bl.nb == 6 ? 8 : 32);
    if (bl.nb == 6) {
        uint32_t n = (uint32_t)bl.ip.size();
        app(&n, 4);
        for (auto& m : bl.ip) app(m.data(), 24);
        app(&bl.yw, 8);
    }
}
bool blind_deserialize(const uint8_t*& p, const uint8_t* end, p3zkc::Blind& bl) {
    auto need = [&](size_t n) { return (size_t)(end - p) >= n; };
    if (!need(4)) return false;
    memcpy(&bl.nb, p, 4); p += 4;
    if (bl.nb < 4 || bl.nb > 6) return false;
    const uint32_t nr = bl.nb == 5 ? 4 : 1, ny = bl.nb == 6 ? 1 : 4;
    if (!need((size_t)nr * 32 + 8 + (size_t)ny * 8)) return false;
    for (uint32_t j = 0; j < nr; j++) { memcpy(bl.rt[j].data(), p, 32); p += 32; }
    memcpy(&bl.H, p, 8); p += 8;
    memcpy(bl.yB, p, (size_t)ny * 8); p += (size_t)ny * 8;
    if (bl.nb == 6) {
        uint32_t n;
        if (!need(4)) return false;
        memcpy(&n, p, 4); p += 4;
        if (n > 64 || !need((size_t)n * 24 + 8)) return false;
        bl.ip.resize(n);
        for (auto& m : bl.ip) { memcpy(m.data(), p, 24); p += 24; }
        memcpy(&bl.yw, p, 8); p += 8;
    }
    return true;
}
// GroupProof (merged lookup, non-zk) <-> bytes:
//   u32 m, c, ns | root_cnt 32 | gkT | per subgroup: u32 n, k | gk | per member: u32 nW, yW.., u32 nV, yv.., u32 nX, extra..
size_t lu_serialize(const p3lu::GroupProof& pf, uint8_t* out, size_t cap) {
    std::vector<uint8_t> b;
    auto app = [&](const void* s, size_t n) { const uint8_t* q = (const uint8_t*)s; b.insert(b.end(), q, q + n); };
    auto appg = [&](const p3gkr::Proof& g) {
        std::vector<uint8_t> t(gkr_size((uint32_t)g.lay.size()));
        gkr_serialize(g, t.data(), t.size());
        app(t.data(), t.size());
    };
    uint32_t ns = (uint32_t)pf.sub.size();
    app(&pf.m, 4); app(&pf.c, 4); app(&ns, 4); app(pf.root_cnt.data(), 32);
    if (p3zkc::G.on) { app(pf.rt_pmT.data(), 32); app(pf.rt_qmT.data(), 32); }
    appg(pf.gkT);
    for (auto& sb : pf.sub) {
        app(&sb.n, 4); app(&sb.k, 4);
        if (p3zkc::G.on) { app(sb.rt_pm.data(), 32); app(sb.rt_qm.data(), 32); }
        appg(sb.gk);
        for (auto& mm : sb.mem) {
            uint32_t a = (uint32_t)mm.yW.size(), v = (uint32_t)mm.y_virt.size(), x = (uint32_t)mm.extra.size();
            app(&a, 4); app(mm.yW.data(), (size_t)a * 8);
            app(&v, 4); app(mm.y_virt.data(), (size_t)v * 8);
            app(&x, 4); app(mm.extra.data(), (size_t)x * 8);
        }
    }
    if (b.size() > cap) return 0;
    memcpy(out, b.data(), b.size());
    return b.size();
}
bool lu_deserialize(const uint8_t* in, size_t len, p3lu::GroupProof& pf) {
    const uint8_t* p = in; const uint8_t* end = in + len;
    auto need = [&](size_t n) { return (size_t)(end - p) >= n; };
    uint32_t ns;
    if (!need(44)) return false;
    memcpy(&pf.m, p, 4); memcpy(&pf.c, p + 4, 4); memcpy(&ns, p + 8, 4); memcpy(pf.root_cnt.data(), p + 12, 32); p += 44;
    if (pf.m > 40 || ns > 4096) return false;
    const bool zk = p3zkc::G.on;        // zk: mask-leaf roots ride along and the trees run over the interleaved augmented domains
    if (zk) {
        if (!need(64)) return false;
        memcpy(pf.rt_pmT.data(), p, 32); memcpy(pf.rt_qmT.data(), p + 32, 32); p += 64;
    }
    const uint32_t LT = zk ? p3zkc::vfull(pf.m) + 1 : pf.m;
    if (!need(gkr_size(LT)) || !gkr_deserialize(p, gkr_size(LT), LT, pf.gkT)) return false;
    p += gkr_size(LT);
    pf.sub.resize(ns);
    for (auto& sb : pf.sub) {
        if (!need(8)) return false;
        memcpy(&sb.n, p, 4); memcpy(&sb.k, p + 4, 4); p += 8;
        if (sb.n > 40 || sb.k == 0 || sb.k > 4096) return false;
        if (zk) {
            if (!need(64)) return false;
            memcpy(sb.rt_pm.data(), p, 32); memcpy(sb.rt_qm.data(), p + 32, 32); p += 64;
        }
        uint32_t g = 0; while ((1u << g) < sb.k) g++;
        uint32_t L = zk ? p3zkc::vfull(sb.n) + g + 1 : sb.n + g;
        if (!need(gkr_size(L)) || !gkr_deserialize(p, gkr_size(L), L, sb.gk)) return false;
        p += gkr_size(L);
        sb.mem.resize(sb.k);
        for (auto& mm : sb.mem) {
            std::vector<gl_t>* vs[3] = {&mm.yW, &mm.y_virt, &mm.extra};
            for (auto* v : vs) {
                uint32_t a;
                if (!need(4)) return false;
                memcpy(&a, p, 4); p += 4;
                if (a > 4096 || !need((size_t)a * 8)) return false;
                v->resize(a); memcpy(v->data(), p, (size_t)a * 8); p += (size_t)a * 8;
            }
        }
    }
    return p == end;
}
// p3imm::Proof (non-zk) <-> bytes: u32 lj, lk, li | messages (lj+lk+li)*40 | yY yX yW | u32 nb | nb x (u32 len, BatchProof)
size_t imm_serialize(const p3imm::Proof& pf, uint8_t* out, size_t cap) {
    std::vector<uint8_t> b;
    auto app = [&](const void* s, size_t n) { const uint8_t* q = (const uint8_t*)s; b.insert(b.end(), q, q + n); };
    app(&pf.lj, 4); app(&pf.lk, 4); app(&pf.li, 4);
    for (auto& m : pf.m) app(&m, 40);
    app(&pf.yY, 8); app(&pf.yX, 8); app(&pf.yW, 8);
    if (p3zkc::G.on) blind_serialize(pf.bl, b);
    uint32_t nb = (uint32_t)pf.tail.batches.size();
    app(&nb, 4);
    for (auto& bp : pf.tail.batches) {
        std::vector<uint8_t> t((size_t)64 << 20);
        uint32_t n = (uint32_t)bo_serialize(bp, t.data(), t.size());
        app(&n, 4); app(t.data(), n);
    }
    if (b.size() > cap) return 0;
    memcpy(out, b.data(), b.size());
    return b.size();
}
bool imm_deserialize(const uint8_t* in, size_t len, p3imm::Proof& pf) {
    const uint8_t* p = in; const uint8_t* end = in + len;
    auto need = [&](size_t n) { return (size_t)(end - p) >= n; };
    if (!need(12)) return false;
    memcpy(&pf.lj, p, 4); memcpy(&pf.lk, p + 4, 4); memcpy(&pf.li, p + 8, 4); p += 12;
    if (pf.lj + pf.lk + pf.li > 60) return false;
    uint32_t lt = p3zkc::vfull(pf.lj + pf.lk + pf.li);      // the chain runs over the augmented domain when zk is on
    if (lt > 64 || !need((size_t)lt * 40 + 28)) return false;
    pf.m.resize(lt);
    for (auto& m : pf.m) { memcpy(&m, p, 40); p += 40; }
    memcpy(&pf.yY, p, 8); memcpy(&pf.yX, p + 8, 8); memcpy(&pf.yW, p + 16, 8); p += 24;
    if (p3zkc::G.on && !blind_deserialize(p, end, pf.bl)) return false;
    if (!need(4)) return false;
    uint32_t nb; memcpy(&nb, p, 4); p += 4;
    if (nb > 64) return false;
    pf.tail.batches.resize(nb);
    for (auto& bp : pf.tail.batches) {
        uint32_t n;
        if (!need(4)) return false;
        memcpy(&n, p, 4); p += 4;
        if (!need(n) || !bo_deserialize(p, n, bp)) return false;
        p += n;
    }
    return p == end;
}
// LookupProof (standalone logUp, non-zk, per-instance openings) <-> bytes:
//   u32 n, m, c | root_cnt root_hA root_hT | S | msgsA n*32 | msgsT m*32 | u32 len, open_hA |
//   u32 count, (u32 len, open_W)* | u32 count, y_virt* | u32 len, open_hT | u32 len, open_cnt
size_t lup_serialize(const p3lu::LookupProof& pf, uint8_t* out, size_t cap) {
    std::vector<uint8_t> b;
    auto app = [&](const void* s, size_t n) { const uint8_t* q = (const uint8_t*)s; b.insert(b.end(), q, q + n); };
    auto appe = [&](const p3bf::EvalProof& e) {
        std::vector<uint8_t> t(bf_size(e.logN, e.R, e.Q));
        uint32_t n = (uint32_t)bf_serialize(e, t.data(), t.size());
        app(&n, 4); app(t.data(), n);
    };
    app(&pf.n, 4); app(&pf.m, 4); app(&pf.c, 4);
    app(pf.root_cnt.data(), 32); app(pf.root_hA.data(), 32); app(pf.root_hT.data(), 32);
    app(&pf.S, 8);
    for (auto& m : pf.msgsA) app(&m, 32);
    for (auto& m : pf.msgsT) app(&m, 32);
    appe(pf.open_hA);
    uint32_t nw = (uint32_t)pf.open_W.size(); app(&nw, 4);
    for (auto& e : pf.open_W) appe(e);
    uint32_t nv = (uint32_t)pf.y_virt.size(); app(&nv, 4);
    app(pf.y_virt.data(), (size_t)nv * 8);
    appe(pf.open_hT); appe(pf.open_cnt);
    if (b.size() > cap) return 0;
    memcpy(out, b.data(), b.size());
    return b.size();
}
bool lup_deserialize(const uint8_t* in, size_t len, p3lu::LookupProof& pf) {
    const uint8_t* p = in; const uint8_t* end = in + len;
    auto need = [&](size_t n) { return (size_t)(end - p) >= n; };
    auto gete = [&](p3bf::EvalProof& e) {
        uint32_t n;
        if (!need(4)) return false;
        memcpy(&n, p, 4); p += 4;
        if (!need(n) || !bf_deserialize(p, n, e)) return false;
        p += n;
        return true;
    };
    if (!need(12 + 96 + 8)) return false;
    memcpy(&pf.n, p, 4); memcpy(&pf.m, p + 4, 4); memcpy(&pf.c, p + 8, 4); p += 12;
    memcpy(pf.root_cnt.data(), p, 32); memcpy(pf.root_hA.data(), p + 32, 32); memcpy(pf.root_hT.data(), p + 64, 32); p += 96;
    memcpy(&pf.S, p, 8); p += 8;
    if (pf.n > 40 || pf.m > 40 || pf.c > 64 || !need(((size_t)pf.n + pf.m) * 32)) return false;
    pf.msgsA.resize(pf.n); pf.msgsT.resize(pf.m);
    for (auto& m : pf.msgsA) { memcpy(&m, p, 32); p += 32; }
    for (auto& m : pf.msgsT) { memcpy(&m, p, 32); p += 32; }
    if (!gete(pf.open_hA)) return false;
    uint32_t nw;
    if (!need(4)) return false;
    memcpy(&nw, p, 4); p += 4;
    if (nw > 64) return false;
    pf.open_W.resize(nw);
    for (auto& e : pf.open_W) if (!gete(e)) return false;
    uint32_t nv;
    if (!need(4)) return false;
    memcpy(&nv, p, 4); p += 4;
    if (nv > 64 || !need((size_t)nv * 8)) return false;
    pf.y_virt.resize(nv); memcpy(pf.y_virt.data(), p, (size_t)nv * 8); p += (size_t)nv * 8;
    if (!gete(pf.open_hT) || !gete(pf.open_cnt)) return false;
    return p == end;
}
// gadget tail (p3ig::Tail) <-> bytes: u32 groups, each u32 len + GroupProof | u32 batches, each u32 len + BatchProof
void tail_append(const p3ig::Tail& t, std::vector<uint8_t>& b) {
    auto app = [&](const void* s, size_t n) { const uint8_t* q = (const uint8_t*)s; b.insert(b.end(), q, q + n); };
    std::vector<uint8_t> tmp((size_t)64 << 20);
    uint32_t ng = (uint32_t)t.lug.size();
    app(&ng, 4);
    for (auto& g : t.lug) { uint32_t n = (uint32_t)lu_serialize(g, tmp.data(), tmp.size()); app(&n, 4); app(tmp.data(), n); }
    uint32_t nb = (uint32_t)t.batches.size();
    app(&nb, 4);
    for (auto& bp : t.batches) { uint32_t n = (uint32_t)bo_serialize(bp, tmp.data(), tmp.size()); app(&n, 4); app(tmp.data(), n); }
}
bool tail_parse(const uint8_t*& p, const uint8_t* end, p3ig::Tail& t) {
    auto need = [&](size_t n) { return (size_t)(end - p) >= n; };
    uint32_t ng;
    if (!need(4)) return false;
    memcpy(&ng, p, 4); p += 4;
    if (ng > 64) return false;
    t.lug.resize(ng);
    for (auto& g : t.lug) {
        uint32_t n;
        if (!need(4)) return false;
        memcpy(&n, p, 4); p += 4;
        if (!need(n) || !lu_deserialize(p, n, g)) return false;
        p += n;
    }
    uint32_t nb;
    if (!need(4)) return false;
    memcpy(&nb, p, 4); p += 4;
    if (nb > 64) return false;
    t.batches.resize(nb);
    for (auto& bp : t.batches) {
        uint32_t n;
        if (!need(4)) return false;
        memcpy(&n, p, 4); p += 4;
        if (!need(n) || !bo_deserialize(p, n, bp)) return false;
        p += n;
    }
    return true;
}
size_t emit(const std::vector<uint8_t>& b, uint8_t* out, size_t cap) {
    if (b.size() > cap) return 0;
    memcpy(out, b.data(), b.size());
    return b.size();
}
// p3iadd::Proof <-> bytes: u32 le | messages le*40 | yA yB yO | tail
size_t iadd_serialize(const p3iadd::Proof& pf, uint8_t* out, size_t cap) {
    std::vector<uint8_t> b;
    auto app = [&](const void* s, size_t n) { const uint8_t* q = (const uint8_t*)s; b.insert(b.end(), q, q + n); };
    app(&pf.le, 4);
    for (auto& m : pf.m) app(&m, 40);
    app(&pf.yA, 8); app(&pf.yB, 8); app(&pf.yO, 8);
    if (p3zkc::G.on) blind_serialize(pf.bl, b);
    tail_append(pf.tail, b);
    return emit(b, out, cap);
}
bool iadd_deserialize(const uint8_t* in, size_t len, p3iadd::Proof& pf) {
    const uint8_t* p = in; const uint8_t* end = in + len;
    if (len < 4) return false;
    memcpy(&pf.le, p, 4); p += 4;
    if (pf.le > 40 || (size_t)(end - p) < (size_t)p3zkc::vfull(pf.le) * 40 + 24) return false;
    pf.m.resize(p3zkc::vfull(pf.le));
    for (auto& m : pf.m) { memcpy(&m, p, 40); p += 40; }
    memcpy(&pf.yA, p, 8); memcpy(&pf.yB, p + 8, 8); memcpy(&pf.yO, p + 16, 8); p += 24;
    if (p3zkc::G.on && !blind_deserialize(p, end, pf.bl)) return false;
    return tail_parse(p, end, pf.tail) && p == end;
}
// p3iswg::Proof <-> bytes: u32 le | rSIL rREM | messages le*40 | ySIL yU yM yR | tail
size_t iswg_serialize(const p3iswg::Proof& pf, uint8_t* out, size_t cap) {
    std::vector<uint8_t> b;
    auto app = [&](const void* s, size_t n) { const uint8_t* q = (const uint8_t*)s; b.insert(b.end(), q, q + n); };
    app(&pf.le, 4); app(pf.rSIL.data(), 32); app(pf.rREM.data(), 32);
    for (auto& m : pf.m) app(&m, 40);
    app(&pf.ySIL, 8); app(&pf.yU, 8); app(&pf.yM, 8); app(&pf.yR, 8);
    if (p3zkc::G.on) blind_serialize(pf.bl, b);
    tail_append(pf.tail, b);
    return emit(b, out, cap);
}
bool iswg_deserialize(const uint8_t* in, size_t len, p3iswg::Proof& pf) {
    const uint8_t* p = in; const uint8_t* end = in + len;
    if (len < 68) return false;
    memcpy(&pf.le, p, 4); memcpy(pf.rSIL.data(), p + 4, 32); memcpy(pf.rREM.data(), p + 36, 32); p += 68;
    if (pf.le > 40 || (size_t)(end - p) < (size_t)p3zkc::vfull(pf.le) * 40 + 32) return false;
    pf.m.resize(p3zkc::vfull(pf.le));
    for (auto& m : pf.m) { memcpy(&m, p, 40); p += 40; }
    memcpy(&pf.ySIL, p, 8); memcpy(&pf.yU, p + 8, 8); memcpy(&pf.yM, p + 16, 8); memcpy(&pf.yR, p + 24, 8); p += 32;
    if (p3zkc::G.on && !blind_deserialize(p, end, pf.bl)) return false;
    return tail_parse(p, end, pf.tail) && p == end;
}
// p3irope::Proof <-> bytes: u32 lT, ld, fb | rREM | messages (lT+ld)*40 | yQ yQx yY yR | tail
size_t irope_serialize(const p3irope::Proof& pf, uint8_t* out, size_t cap) {
    std::vector<uint8_t> b;
    auto app = [&](const void* s, size_t n) { const uint8_t* q = (const uint8_t*)s; b.insert(b.end(), q, q + n); };
    app(&pf.lT, 4); app(&pf.ld, 4); app(&pf.fb, 4); app(pf.rREM.data(), 32);
    for (auto& m : pf.m) app(&m, 40);
    app(&pf.yQ, 8); app(&pf.yQx, 8); app(&pf.yY, 8); app(&pf.yR, 8);
    if (p3zkc::G.on) blind_serialize(pf.bl, b);
    tail_append(pf.tail, b);
    return emit(b, out, cap);
}
bool irope_deserialize(const uint8_t* in, size_t len, p3irope::Proof& pf) {
    const uint8_t* p = in; const uint8_t* end = in + len;
    if (len < 44) return false;
    memcpy(&pf.lT, p, 4); memcpy(&pf.ld, p + 4, 4); memcpy(&pf.fb, p + 8, 4); memcpy(pf.rREM.data(), p + 12, 32); p += 44;
    if ((size_t)pf.lT + pf.ld > 40) return false;
    const size_t le = p3zkc::vfull(pf.lT + pf.ld);
    if ((size_t)(end - p) < le * 40 + 32) return false;
    pf.m.resize(le);
    for (auto& m : pf.m) { memcpy(&m, p, 40); p += 40; }
    memcpy(&pf.yQ, p, 8); memcpy(&pf.yQx, p + 8, 8); memcpy(&pf.yY, p + 16, 8); memcpy(&pf.yR, p + 24, 8); p += 32;
    if (p3zkc::G.on && !blind_deserialize(p, end, pf.bl)) return false;
    return tail_parse(p, end, pf.tail) && p == end;
}
p3irope::Pub rope_pub(const int32_t* ct, const int32_t* st, uint32_t lseq, uint32_t ldh) {
    p3irope::Pub P;
    P.lseq = lseq; P.ldh = ldh;
    const size_t n = ((size_t)1 << lseq) << (ldh - 1);
    P.ct.assign(ct, ct + n); P.st.assign(st, st + n);
    return P;
}
// p3irms::Proof <-> bytes: u32 lT, ld | 18 row roots | 3 element roots | yM yMX | mS (lT+ld)*40 | mB lT*40 | yB[18] |
//   mE (lT+ld)*40 | yE[3] | yEX yEY yER yEG | tail
size_t irms_serialize(const p3irms::Proof& pf, uint8_t* out, size_t cap) {
    std::vector<uint8_t> b;
    auto app = [&](const void* s, size_t n) { const uint8_t* q = (const uint8_t*)s; b.insert(b.end(), q, q + n); };
    app(&pf.lT, 4); app(&pf.ld, 4);
    for (int c = 0; c < p3irms::NDB; c++) app(pf.rdb[c].data(), 32);
    for (int c = 0; c < p3irms::NDE; c++) app(pf.rde[c].data(), 32);
    app(&pf.yM, 8); app(&pf.yMX, 8);
    for (auto& m : pf.mS) app(&m, 40);
    for (auto& m : pf.mB) app(&m, 40);
    app(pf.yB, 8 * p3irms::NDB);
    for (auto& m : pf.mE) app(&m, 40);
    app(pf.yE, 8 * p3irms::NDE);
    app(&pf.yEX, 8); app(&pf.yEY, 8); app(&pf.yER, 8); app(&pf.yEG, 8);
    if (p3zkc::G.on) for (int j = 0; j < 3; j++) blind_serialize(pf.bl[j], b);
    tail_append(pf.tail, b);
    return emit(b, out, cap);
}
bool irms_deserialize(const uint8_t* in, size_t len, p3irms::Proof& pf) {
    const uint8_t* p = in; const uint8_t* end = in + len;
    if (len < 8) return false;
    memcpy(&pf.lT, p, 4); memcpy(&pf.ld, p + 4, 4); p += 8;
    if ((size_t)pf.lT + pf.ld > 40) return false;
    const size_t le = p3zkc::vfull(pf.lT + pf.ld), lTf = p3zkc::vfull(pf.lT);   // chains run over the augmented domains when zk is on
    const size_t fixed = 32 * (p3irms::NDB + p3irms::NDE) + 16 + 40 * (2 * le + lTf) + 8 * (p3irms::NDB + p3irms::NDE) + 32;
    if ((size_t)(end - p) < fixed) return false;
    for (int c = 0; c < p3irms::NDB; c++) { memcpy(pf.rdb[c].data(), p, 32); p += 32; }
    for (int c = 0; c < p3irms::NDE; c++) { memcpy(pf.rde[c].data(), p, 32); p += 32; }
    memcpy(&pf.yM, p, 8); memcpy(&pf.yMX, p + 8, 8); p += 16;
    pf.mS.resize(le); pf.mB.resize(lTf); pf.mE.resize(le);
    for (auto& m : pf.mS) { memcpy(&m, p, 40); p += 40; }
    for (auto& m : pf.mB) { memcpy(&m, p, 40); p += 40; }
    memcpy(pf.yB, p, 8 * p3irms::NDB); p += 8 * p3irms::NDB;
    for (auto& m : pf.mE) { memcpy(&m, p, 40); p += 40; }
    memcpy(pf.yE, p, 8 * p3irms::NDE); p += 8 * p3irms::NDE;
    memcpy(&pf.yEX, p, 8); memcpy(&pf.yEY, p + 8, 8); memcpy(&pf.yER, p + 16, 8); memcpy(&pf.yEG, p + 24, 8); p += 32;
    if (p3zkc::G.on) for (int j = 0; j < 3; j++) if (!blind_deserialize(p, end, pf.bl[j])) return false;
    return tail_parse(p, end, pf.tail) && p == end;
}
// p3ismx::Proof <-> bytes: u32 la, lseq | 7 element roots | 2 row roots | mSel le*40 | ySel | ySrow | mS le*40 | ySE |
//   mE le*40 | yEZ | yE[7] | yEP yEMX yES | tail        (le = la + 2*lseq)
size_t ismx_serialize(const p3ismx::Proof& pf, uint8_t* out, size_t cap) {
    std::vector<uint8_t> b;
    auto app = [&](const void* s, size_t n) { const uint8_t* q = (const uint8_t*)s; b.insert(b.end(), q, q + n); };
    app(&pf.la, 4); app(&pf.lseq, 4);
    for (int c = 0; c < p3ismx::NXE; c++) app(pf.rxe[c].data(), 32);
    for (int c = 0; c < p3ismx::NXB; c++) app(pf.rxb[c].data(), 32);
    for (auto& m : pf.mSel) app(&m, 40);
    app(&pf.ySel, 8); app(&pf.ySrow, 8);
    for (auto& m : pf.mS) app(&m, 40);
    app(&pf.ySE, 8);
    for (auto& m : pf.mE) app(&m, 40);
    app(&pf.yEZ, 8); app(pf.yE, 8 * p3ismx::NXE); app(&pf.yEP, 8); app(&pf.yEMX, 8); app(&pf.yES, 8);
    if (p3zkc::G.on) for (int j = 0; j < 3; j++) blind_serialize(pf.bl[j], b);
    tail_append(pf.tail, b);
    return emit(b, out, cap);
}
bool ismx_deserialize(const uint8_t* in, size_t len, p3ismx::Proof& pf) {
    const uint8_t* p = in; const uint8_t* end = in + len;
    if (len < 8) return false;
    memcpy(&pf.la, p, 4); memcpy(&pf.lseq, p + 4, 4); p += 8;
    if ((size_t)pf.la + 2 * (size_t)pf.lseq > 40) return false;
    const size_t le = p3zkc::vfull(pf.la + 2 * pf.lseq);      // the chains run over the augmented domain when zk is on
    const size_t fixed = 32 * (p3ismx::NXE + p3ismx::NXB) + 120 * le + 8 * (3 + 1 + p3ismx::NXE + 3);
    if ((size_t)(end - p) < fixed) return false;
    for (int c = 0; c < p3ismx::NXE; c++) { memcpy(pf.rxe[c].data(), p, 32); p += 32; }
    for (int c = 0; c < p3ismx::NXB; c++) { memcpy(pf.rxb[c].data(), p, 32); p += 32; }
    pf.mSel.resize(le); pf.mS.resize(le); pf.mE.resize(le);
    for (auto& m : pf.mSel) { memcpy(&m, p, 40); p += 40; }
    memcpy(&pf.ySel, p, 8); memcpy(&pf.ySrow, p + 8, 8); p += 16;
    for (auto& m : pf.mS) { memcpy(&m, p, 40); p += 40; }
    memcpy(&pf.ySE, p, 8); p += 8;
    for (auto& m : pf.mE) { memcpy(&m, p, 40); p += 40; }
    memcpy(&pf.yEZ, p, 8); p += 8;
    memcpy(pf.yE, p, 8 * p3ismx::NXE); p += 8 * p3ismx::NXE;
    memcpy(&pf.yEP, p, 8); memcpy(&pf.yEMX, p + 8, 8); memcpy(&pf.yES, p + 16, 8); p += 24;
    if (p3zkc::G.on) for (int j = 0; j < 3; j++) if (!blind_deserialize(p, end, pf.bl[j])) return false;
    return tail_parse(p, end, pf.tail) && p == end;
}
size_t irs_serialize(const p3irs::Proof& pf, uint8_t* out, size_t cap);
bool irs_deserialize(const uint8_t* in, size_t len, p3irs::Proof& pf);
// p3itf::TfProof <-> bytes: 6 x u32 dims | length-prefixed sub-proofs in proving order (rms1, mm Q K V, rsq rsk rsv,
// rpq rpk, mmqk[A], rsz, smx, mmpv[A], rsat, mm O, rso, add1, rms2, mm G U, rsg rsu, swg, mm D, rsd, add2) | 28 roots |
// u32 groups (len, GroupProof)* | ioin ioout | u32 batches (len, BatchProof)*
struct SubIO {
    std::vector<uint8_t>* b = nullptr;          // writing
    const uint8_t* p = nullptr; const uint8_t* end = nullptr; bool ok = true;   // reading
    std::vector<uint8_t> tmp = std::vector<uint8_t>((size_t)64 << 20);
    template <typename PF, typename SER> void put(const PF& pf, SER ser) {
        uint32_t n = (uint32_t)ser(pf, tmp.data(), tmp.size());
        const uint8_t* q = (const uint8_t*)&n;
        b->insert(b->end(), q, q + 4);
        b->insert(b->end(), tmp.data(), tmp.data() + n);
    }
    template <typename PF, typename DES> void get(PF& pf, DES des) {
        if (!ok || (size_t)(end - p) < 4) { ok = false; return; }
        uint32_t n; memcpy(&n, p, 4); p += 4;
        if ((size_t)(end - p) < n || !des(p, n, pf)) { ok = false; return; }
        p += n;
    }
};
template <typename IO, typename PFT>
void itf_walk(IO& io, PFT& pf, bool writing) {
    using namespace p3itf;
    auto RMS = [&](auto& x) { if (writing) io.put(x, irms_serialize); else io.get(const_cast<p3irms::Proof&>(x), irms_deserialize); };
    auto MM = [&](auto& x) { if (writing) io.put(x, imm_serialize); else io.get(const_cast<p3imm::Proof&>(x), imm_deserialize); };
    auto RS = [&](auto& x) { if (writing) io.put(x, irs_serialize); else io.get(const_cast<p3irs::Proof&>(x), irs_deserialize); };
    auto RP = [&](auto& x) { if (writing) io.put(x, irope_serialize); else io.get(const_cast<p3irope::Proof&>(x), irope_deserialize); };
    auto SMX = [&](auto& x) { if (writing) io.put(x, ismx_serialize); else io.get(const_cast<p3ismx::Proof&>(x), ismx_deserialize); };
    auto SWG = [&](auto& x) { if (writing) io.put(x, iswg_serialize); else io.get(const_cast<p3iswg::Proof&>(x), iswg_deserialize); };
    auto ADD = [&](auto& x) { if (writing) io.put(x, iadd_serialize); else io.get(const_cast<p3iadd::Proof&>(x), iadd_deserialize); };
    const uint32_t A = pf.batch * pf.nh;
    auto& P = const_cast<TfProof&>(pf);
    if (!writing) { P.mmqk.resize(A); P.mmpv.resize(A); }
    RMS(pf.rms1);
    MM(pf.mm[W_Q]); MM(pf.mm[W_K]); MM(pf.mm[W_V]);
    RS(pf.rsq); RS(pf.rsk); RS(pf.rsv);
    RP(pf.rpq); RP(pf.rpk);
    for (uint32_t a = 0; a < A; a++) MM(pf.mmqk[a]);
    RS(pf.rsz);
    SMX(pf.smx);
    for (uint32_t a = 0; a < A; a++) MM(pf.mmpv[a]);
    RS(pf.rsat);
    MM(pf.mm[W_O]);
    RS(pf.rso);
    ADD(pf.add1);
    RMS(pf.rms2);
    MM(pf.mm[W_G]); MM(pf.mm[W_U]);
    RS(pf.rsg); RS(pf.rsu);
    SWG(pf.swg);
    MM(pf.mm[W_D]);
    RS(pf.rsd);
    ADD(pf.add2);
}
std::vector<p3fri::Hash*> itf_roots(p3itf::TfProof& pf) {
    std::vector<p3fri::Hash*> r = {&pf.rX0, &pf.rH1};
    for (int i = 0; i < p3itf::NW; i++) r.push_back(&pf.rACC[i]);
    for (auto* h : {&pf.rYQ, &pf.rYK, &pf.rYV, &pf.rRQ, &pf.rRK, &pf.rSC, &pf.rZ, &pf.rP, &pf.rPVA, &pf.rAT, &pf.rYO, &pf.rRES1,
                    &pf.rH2, &pf.rGG, &pf.rUU, &pf.rMO, &pf.rYD, &pf.rOUT}) r.push_back(h);
    return r;
}
size_t itf_serialize(const p3itf::TfProof& pf, uint8_t* out, size_t cap) {
    std::vector<uint8_t> b;
    auto app = [&](const void* s, size_t n) { const uint8_t* q = (const uint8_t*)s; b.insert(b.end(), q, q + n); };
    uint32_t hdr[6] = {pf.seq, pf.d, pf.nh, pf.dh, pf.dff, pf.batch};
    app(hdr, 24);
    SubIO io; io.b = &b;
    itf_walk(io, pf, true);
    for (auto* h : itf_roots(const_cast<p3itf::TfProof&>(pf))) app(h->data(), 32);
    p3ig::Tail t; t.lug = pf.lug;
    uint32_t ng = (uint32_t)pf.lug.size();
    app(&ng, 4);
    for (auto& g : pf.lug) { uint32_t n = (uint32_t)lu_serialize(g, io.tmp.data(), io.tmp.size()); app(&n, 4); app(io.tmp.data(), n); }
    app(&pf.ioin, 8); app(&pf.ioout, 8);
    uint32_t nb = (uint32_t)pf.batches.size();
    app(&nb, 4);
    for (auto& bp : pf.batches) { uint32_t n = (uint32_t)bo_serialize(bp, io.tmp.data(), io.tmp.size()); app(&n, 4); app(io.tmp.data(), n); }
    return emit(b, out, cap);
}
bool itf_deserialize(const uint8_t* in, size_t len, p3itf::TfProof& pf) {
    if (len < 24) return false;
    uint32_t hdr[6]; memcpy(hdr, in, 24);
    pf.seq = hdr[0]; pf.d = hdr[1]; pf.nh = hdr[2]; pf.dh = hdr[3]; pf.dff = hdr[4]; pf.batch = hdr[5];
    if (pf.nh == 0 || pf.batch == 0 || (uint64_t)pf.nh * pf.batch > 4096) return false;
    SubIO io; io.p = in + 24; io.end = in + len;
    itf_walk(io, pf, false);
    if (!io.ok) return false;
    const uint8_t* p = io.p; const uint8_t* end = io.end;
    auto need = [&](size_t n) { return (size_t)(end - p) >= n; };
    for (auto* h : itf_roots(pf)) { if (!need(32)) return false; memcpy(h->data(), p, 32); p += 32; }
    uint32_t ng;
    if (!need(4)) return false;
    memcpy(&ng, p, 4); p += 4;
    if (ng > 64) return false;
    pf.lug.resize(ng);
    for (auto& g : pf.lug) {
        uint32_t n;
        if (!need(4)) return false;
        memcpy(&n, p, 4); p += 4;
        if (!need(n) || !lu_deserialize(p, n, g)) return false;
        p += n;
    }
    if (!need(20)) return false;
    memcpy(&pf.ioin, p, 8); memcpy(&pf.ioout, p + 8, 8); p += 16;
    uint32_t nb; memcpy(&nb, p, 4); p += 4;
    if (nb > 64) return false;
    pf.batches.resize(nb);
    for (auto& bp : pf.batches) {
        uint32_t n;
        if (!need(4)) return false;
        memcpy(&n, p, 4); p += 4;
        if (!need(n) || !bo_deserialize(p, n, bp)) return false;
        p += n;
    }
    return p == end;
}
p3itf::Weights itf_weights(const p3itf::Config& cfg, const uint64_t* const* w7, const uint64_t* g1, const uint64_t* g2,
                           const int32_t* ct, const int32_t* sn) {
    p3itf::Weights W; W.cfg = cfg;
    for (int i = 0; i < p3itf::NW; i++) {
        uint32_t K, N; p3itf::wshape(cfg, i, K, N);
        W.w[i].assign(w7[i], w7[i] + (size_t)K * N);
    }
    W.g1.assign(g1, g1 + cfg.d); W.g2.assign(g2, g2 + cfg.d);
    W.rp = rope_pub(ct, sn, cfg.lseq(), cfg.ldh());
    return W;
}
// p3hwl::LayerProof <-> bytes (non-zk fields, declaration order):
//   u32 B K N | roots rdp[10] rdg[29] rdo[46] rdb[6] rdn[6] | u32 groups (len, GroupProof)* |
//   mDp yDp[10] yDpG | mDg yDg[29] | mCh yCh[8] | yGSc yGSa | mGS yGSal yGSsel | mDo yDo[46] | yDbBC[5] yDnBC[5] |
//   mDb yDb[6] yXsb | mDn yDn[6] yWsb | ySlA ySlE ySlS ySlF ySlBE ySlSG | mY yY | u32 batches (len, BatchProof)*
// every message list is u32 rounds + rounds*40 bytes
template <typename IO>
void hwl_walk(IO& io, p3hwl::LayerProof& pf) {
    using namespace p3hwl;
    io.u32(pf.B); io.u32(pf.K); io.u32(pf.N);
    for (int c = 0; c < NDP; c++) io.raw(pf.rdp[c].data(), 32);
    for (int c = 0; c < NDG; c++) io.raw(pf.rdg[c].data(), 32);
    for (int c = 0; c < NDO; c++) io.raw(pf.rdo[c].data(), 32);
    for (int c = 0; c < NDS; c++) io.raw(pf.rdb[c].data(), 32);
    for (int c = 0; c < NDS; c++) io.raw(pf.rdn[c].data(), 32);
    io.groups(pf.lug);
    io.msgs(pf.mDp); io.raw(pf.yDp, sizeof pf.yDp); io.raw(&pf.yDpG, 8);
    io.msgs(pf.mDg); io.raw(pf.yDg, sizeof pf.yDg);
    io.msgs(pf.mCh); io.raw(pf.yCh, sizeof pf.yCh);
    io.raw(&pf.yGSc, 8); io.raw(&pf.yGSa, 8);
    io.msgs(pf.mGS); io.raw(&pf.yGSal, 8); io.raw(&pf.yGSsel, 8);
    io.msgs(pf.mDo); io.raw(pf.yDo, sizeof pf.yDo);
    io.raw(pf.yDbBC, sizeof pf.yDbBC); io.raw(pf.yDnBC, sizeof pf.yDnBC);
    io.msgs(pf.mDb); io.raw(pf.yDb, sizeof pf.yDb); io.raw(&pf.yXsb, 8);
    io.msgs(pf.mDn); io.raw(pf.yDn, sizeof pf.yDn); io.raw(&pf.yWsb, 8);
    io.raw(&pf.ySlA, 8); io.raw(&pf.ySlE, 8); io.raw(&pf.ySlS, 8); io.raw(&pf.ySlF, 8); io.raw(&pf.ySlBE, 8); io.raw(&pf.ySlSG, 8);
    io.msgs(pf.mY); io.raw(&pf.yY, 8);
    io.batches(pf.batches);
}
struct HwlWriter {
    std::vector<uint8_t> b;
    std::vector<uint8_t> tmp = std::vector<uint8_t>((size_t)256 << 20);
    void raw(const void* s, size_t n) { const uint8_t* q = (const uint8_t*)s; b.insert(b.end(), q, q + n); }
    void fail() {}
    void u32(uint32_t& v) { raw(&v, 4); }
    void msgs(std::vector<p3hwl::Msg5>& m) { uint32_t n = (uint32_t)m.size(); raw(&n, 4); raw(m.data(), (size_t)n * 40); }
    void vec(std::vector<gl_t>& v) { uint32_t n = (uint32_t)v.size(); raw(&n, 4); raw(v.data(), (size_t)n * 8); }
    void vec16(std::vector<uint16_t>& v) { uint32_t n = (uint32_t)v.size(); raw(&n, 4); raw(v.data(), (size_t)n * 2); }
    template <typename PF, typename WALK> void sub(PF& pf, WALK walk) {      // length-prefixed nested proof
        HwlWriter w2;
        walk(w2, pf);
        uint32_t n = (uint32_t)w2.b.size(); raw(&n, 4); raw(w2.b.data(), n);
    }
    void groups(std::vector<p3lu::GroupProof>& g) {
        uint32_t ng = (uint32_t)g.size(); raw(&ng, 4);
        for (auto& x : g) { uint32_t n = (uint32_t)lu_serialize(x, tmp.data(), tmp.size()); raw(&n, 4); raw(tmp.data(), n); }
    }
    void batches(std::vector<p3bo::BatchProof>& v) {
        uint32_t nb = (uint32_t)v.size(); raw(&nb, 4);
        for (auto& x : v) { uint32_t n = (uint32_t)bo_serialize(x, tmp.data(), tmp.size()); raw(&n, 4); raw(tmp.data(), n); }
    }
};
struct HwlReader {
    const uint8_t* p; const uint8_t* end; bool ok = true;
    bool need(size_t n) { if (!ok || (size_t)(end - p) < n) ok = false; return ok; }
    void fail() { ok = false; }
    void raw(void* d, size_t n) { if (need(n)) { memcpy(d, p, n); p += n; } }
    void u32(uint32_t& v) { raw(&v, 4); }
    void msgs(std::vector<p3hwl::Msg5>& m) {
        uint32_t n = 0; u32(n);
        if (!ok || n > 64 || !need((size_t)n * 40)) { ok = false; return; }
        m.resize(n); raw(m.data(), (size_t)n * 40);
    }
    void vec(std::vector<gl_t>& v) {
        uint32_t n = 0; u32(n);
        if (!ok || n > (1u << 20) || !need((size_t)n * 8)) { ok = false; return; }
        v.resize(n); raw(v.data(), (size_t)n * 8);
    }
    void vec16(std::vector<uint16_t>& v) {
        uint32_t n = 0; u32(n);
        if (!ok || !need((size_t)n * 2)) { ok = false; return; }
        v.resize(n); raw(v.data(), (size_t)n * 2);
    }
    template <typename PF, typename WALK> void sub(PF& pf, WALK walk) {
        uint32_t n = 0; u32(n);
        if (!need(n)) return;
        HwlReader r2{p, p + n};
        walk(r2, pf);
        if (!r2.ok || r2.p != r2.end) { ok = false; return; }
        p += n;
    }
    void groups(std::vector<p3lu::GroupProof>& g) {
        uint32_t ng = 0; u32(ng);
        if (!ok || ng > 256) { ok = false; return; }
        g.resize(ng);
        for (auto& x : g) { uint32_t n = 0; u32(n); if (!need(n) || !lu_deserialize(p, n, x)) { ok = false; return; } p += n; }
    }
    void batches(std::vector<p3bo::BatchProof>& v) {
        uint32_t nb = 0; u32(nb);
        if (!ok || nb > 64) { ok = false; return; }
        v.resize(nb);
        for (auto& x : v) { uint32_t n = 0; u32(n); if (!need(n) || !bo_deserialize(p, n, x)) { ok = false; return; } p += n; }
    }
};
size_t hwl_serialize(const p3hwl::LayerProof& pf, uint8_t* out, size_t cap) {
    HwlWriter w;
    hwl_walk(w, const_cast<p3hwl::LayerProof&>(pf));
    return emit(w.b, out, cap);
}
bool hwl_deserialize(const uint8_t* in, size_t len, p3hwl::LayerProof& pf) {
    HwlReader r{in, in + len};
    hwl_walk(r, pf);
    return r.ok && r.p == r.end;
}
const p3hwl::Tables& hwl_tables() {
    static p3hwl::Tables T = p3hwl::build_tables();
    return T;
}
const p3lu::Table* hwl_table_at(int which) {
    const p3hwl::Tables& T = hwl_tables();
    const p3lu::Table* tabs[16] = {&T.DM, &T.SH, &T.RM, &T.R15, &T.ASH, &T.WIDTH, &T.R10, &T.R11,
                                   &T.R12, &T.R16, &T.FH, &T.REXP, &T.SE, &T.CREM13, &T.CREM12, &T.CTH};
    return (which >= 0 && which < 16) ? tabs[which] : nullptr;
}
p3hwl::Golden hwl_golden(uint32_t B, uint32_t K, uint32_t N, const uint8_t* x, const uint8_t* w, const uint32_t* xs,
                         const uint32_t* ws) {
    p3hwl::Golden L; L.B = B; L.K = K; L.N = N;
    L.x.assign(x, x + (size_t)B * K); L.w.assign(w, w + (size_t)N * K);
    L.xs.assign(xs, xs + B); L.ws.assign(ws, ws + N);
    L.y.assign((size_t)B * N, 0);
    return L;
}
// ---- bf16 gadgets of the fp8 transformer layer: the pinned table artefact and per-gadget proof walks ----
p3rms::Art& tf_art() { static p3rms::Art a; return a; }
// p3swg::SwgProof <-> bytes: u32 n | rws[14] | u32 groups (len, GroupProof)* | mE | yE[14] yUP yM | u32 batches (len, BatchProof)*
template <typename IO>
void swg_walk(IO& io, p3swg::SwgProof& pf) {
    io.u32(pf.n);
    for (int c = 0; c < p3swg::NDS; c++) io.raw(pf.rws[c].data(), 32);
    io.groups(pf.lug);
    io.msgs(pf.mE); io.raw(pf.yE, sizeof pf.yE); io.raw(&pf.yUP, 8); io.raw(&pf.yM, 8);
    io.batches(pf.batches);
}
const p3swg::Tables& swg_tables() {
    static p3swg::Tables T = p3swg::build_tables(tf_art());
    return T;
}
// p3bfa::BfaProof <-> bytes: u32 n | rws[55] | groups | mE | yE[55] yX1 yX2 yOUT | batches
template <typename IO>
void bfa_walk(IO& io, p3bfa::BfaProof& pf) {
    io.u32(pf.n);
    for (int c = 0; c < p3bfa::NBA; c++) io.raw(pf.rws[c].data(), 32);
    io.groups(pf.lug);
    io.msgs(pf.mE); io.raw(pf.yE, sizeof pf.yE); io.raw(&pf.yX1, 8); io.raw(&pf.yX2, 8); io.raw(&pf.yOUT, 8);
    io.batches(pf.batches);
}
const p3bfa::Tables& bfa_tables() {
    static p3bfa::Tables T = p3bfa::build_tables();
    return T;
}
// p3qnt::QntProof <-> bytes: u32 B ld | rde[8] rdb[3] | groups | mDe yDe[8] yDeX yDeC yDeE | mDb yDb[3] yDbS | yBF | mBind yBSEL | batches
template <typename IO>
void qnt_walk(IO& io, p3qnt::QntProof& pf) {
    io.u32(pf.B); io.u32(pf.ld);
    for (int c = 0; c < p3qnt::NDE; c++) io.raw(pf.rde[c].data(), 32);
    for (int c = 0; c < p3qnt::NDB; c++) io.raw(pf.rdb[c].data(), 32);
    io.groups(pf.lug);
    io.msgs(pf.mDe); io.raw(pf.yDe, sizeof pf.yDe); io.raw(&pf.yDeX, 8); io.raw(&pf.yDeC, 8); io.raw(&pf.yDeE, 8);
    io.msgs(pf.mDb); io.raw(pf.yDb, sizeof pf.yDb); io.raw(&pf.yDbS, 8);
    io.raw(&pf.yBF, 8);
    io.msgs(pf.mBind); io.raw(&pf.yBSEL, 8);
    io.batches(pf.batches);
}
const p3qnt::Tables& qnt_tables() { static p3qnt::Tables T = p3qnt::build_tables(tf_art()); return T; }
// p3rope::RopeProof <-> bytes: u32 lp lh | rws[NDR] | groups | mE | u32 count, yE.. | yQA yQB yOA yOB | batches
template <typename IO>
void rope_walk(IO& io, p3rope::RopeProof& pf) {
    io.u32(pf.lp); io.u32(pf.lh);
    for (int c = 0; c < p3rope::NDR; c++) io.raw(pf.rws[c].data(), 32);
    io.groups(pf.lug);
    io.msgs(pf.mE); io.vec(pf.yE);
    io.raw(&pf.yQA, 8); io.raw(&pf.yQB, 8); io.raw(&pf.yOA, 8); io.raw(&pf.yOB, 8);
    io.batches(pf.batches);
}
const p3rope::Tables& rope_tables() { static p3rope::Tables T = p3rope::build_tables(tf_art()); return T; }
// p3rms::RmsProof <-> bytes: u32 B ld | rde rdb rdw | groups | mDe yDe yDeX yDeY yDeE yDeTEB yDeGS yDeGEB yDeGZ | mDb yDb |
//   mDw yDw yDwG | yBS yBF | mBind yBXZ yBQ yBSEL | batches
template <typename IO>
void rms_walk(IO& io, p3rms::RmsProof& pf) {
    io.u32(pf.B); io.u32(pf.ld);
    for (int c = 0; c < p3rms::NDE; c++) io.raw(pf.rde[c].data(), 32);
    for (int c = 0; c < p3rms::NDB; c++) io.raw(pf.rdb[c].data(), 32);
    for (int c = 0; c < p3rms::NDW; c++) io.raw(pf.rdw[c].data(), 32);
    io.groups(pf.lug);
    io.msgs(pf.mDe); io.raw(pf.yDe, sizeof pf.yDe);
    io.raw(&pf.yDeX, 8); io.raw(&pf.yDeY, 8); io.raw(&pf.yDeE, 8); io.raw(&pf.yDeTEB, 8); io.raw(&pf.yDeGS, 8);
    io.raw(&pf.yDeGEB, 8); io.raw(&pf.yDeGZ, 8);
    io.msgs(pf.mDb); io.raw(pf.yDb, sizeof pf.yDb);
    io.msgs(pf.mDw); io.raw(pf.yDw, sizeof pf.yDw); io.raw(&pf.yDwG, 8);
    io.raw(&pf.yBS, 8); io.raw(&pf.yBF, 8);
    io.msgs(pf.mBind); io.raw(&pf.yBXZ, 8); io.raw(&pf.yBQ, 8); io.raw(&pf.yBSEL, 8);
    io.batches(pf.batches);
}
// p3smx::SmxProof <-> bytes: u32 B ln | rde[NDE2] rdb[NDB2] | groups | mDe | u32 count, yDe.. | yDeS yDeP yDeKM yDeMX yDeE yDeRB |
//   mDb yDb | yBF yBS | mBind yBSEL1 yBSEL2 yBQ2 | batches
template <typename IO>
void smx_walk(IO& io, p3smx::SmxProof& pf) {
    io.u32(pf.B); io.u32(pf.ln);
    for (int c = 0; c < p3smx::NDE2; c++) io.raw(pf.rde[c].data(), 32);
    for (int c = 0; c < p3smx::NDB2; c++) io.raw(pf.rdb[c].data(), 32);
    io.groups(pf.lug);
    io.msgs(pf.mDe); io.vec(pf.yDe);
    io.raw(&pf.yDeS, 8); io.raw(&pf.yDeP, 8); io.raw(&pf.yDeKM, 8); io.raw(&pf.yDeMX, 8); io.raw(&pf.yDeE, 8); io.raw(&pf.yDeRB, 8);
    io.msgs(pf.mDb); io.raw(pf.yDb, sizeof pf.yDb);
    io.raw(&pf.yBF, 8); io.raw(&pf.yBS, 8);
    io.msgs(pf.mBind); io.raw(&pf.yBSEL1, 8); io.raw(&pf.yBSEL2, 8); io.raw(&pf.yBQ2, 8);
    io.batches(pf.batches);
}
// p3tf::TfProof <-> bytes: 6 x u32 dims | length-prefixed sub-proofs in proving order | roots rX0 rRmsY[2] rCodes[] rScales[]
//   rMX[] rMW[] rRopeQ[] rRopeO[] rSmP[] rVtX[] rAtX rRes1 rSwM rOut | per matmul u32 count + bf16 outputs | groups |
//   u32 count + seam values | batches
template <typename IO>
void tf_walk(IO& io, p3tf::TfProof& pf, bool reading) {
    io.u32(pf.seq); io.u32(pf.d); io.u32(pf.nh); io.u32(pf.dh); io.u32(pf.dff); io.u32(pf.batch);
    p3tf::Config c; c.seq = pf.seq; c.d = pf.d; c.nh = pf.nh; c.dh = pf.dh; c.dff = pf.dff; c.batch = pf.batch;
    if (reading) {
        if (!c.pow2() || c.A() > 4096) { io.fail(); return; }
        pf.qn.resize(c.nqn()); pf.mm.resize(c.nmm()); pf.rp.resize(2 * c.A()); pf.sm.resize(c.A());
        pf.rCodes.resize(c.nqn()); pf.rScales.resize(c.nqn()); pf.rMX.resize(c.nmm()); pf.rMW.resize(c.nmm());
        pf.rRopeQ.resize(2 * c.A()); pf.rRopeO.resize(2 * c.A()); pf.rSmP.resize(c.A()); pf.rVtX.resize(c.A());
        pf.mmY.resize(c.nmm());
    }
    auto RMS = [&](p3rms::RmsProof& x) { io.sub(x, [](auto& i2, p3rms::RmsProof& y) { rms_walk(i2, y); }); };
    auto QN = [&](p3qnt::QntProof& x) { io.sub(x, [](auto& i2, p3qnt::QntProof& y) { qnt_walk(i2, y); }); };
    auto MM = [&](p3hwl::LayerProof& x) { io.sub(x, [](auto& i2, p3hwl::LayerProof& y) { hwl_walk(i2, y); }); };
    auto RP = [&](p3rope::RopeProof& x) { io.sub(x, [](auto& i2, p3rope::RopeProof& y) { rope_walk(i2, y); }); };
    auto SMX = [&](p3smx::SmxProof& x) { io.sub(x, [](auto& i2, p3smx::SmxProof& y) { smx_walk(i2, y); }); };
    auto BFA = [&](p3bfa::BfaProof& x) { io.sub(x, [](auto& i2, p3bfa::BfaProof& y) { bfa_walk(i2, y); }); };
    auto SWG = [&](p3swg::SwgProof& x) { io.sub(x, [](auto& i2, p3swg::SwgProof& y) { swg_walk(i2, y); }); };
    RMS(pf.rms[0]); QN(pf.qn[p3tf::QN_H1]);
    MM(pf.mm[p3tf::MM_WQ]); MM(pf.mm[p3tf::MM_WK]); MM(pf.mm[p3tf::MM_WV]);
    for (uint32_t a = 0; a < c.A(); a++) {
        RP(pf.rp[2 * a]); RP(pf.rp[2 * a + 1]);
        QN(pf.qn[c.qnRQ(a)]); QN(pf.qn[c.qnRK(a)]); MM(pf.mm[c.mmQK(a)]);
        SMX(pf.sm[a]);
        QN(pf.qn[c.qnPB(a)]); QN(pf.qn[c.qnVT(a)]); MM(pf.mm[c.mmPV(a)]);
    }
    QN(pf.qn[c.qnAT()]); MM(pf.mm[c.mmWO()]); BFA(pf.res[0]); RMS(pf.rms[1]); QN(pf.qn[c.qnH2()]);
    MM(pf.mm[c.mmWG()]); MM(pf.mm[c.mmWU()]); SWG(pf.sw); QN(pf.qn[c.qnSW()]); MM(pf.mm[c.mmWD()]); BFA(pf.res[1]);
    auto H = [&](p3fri::Hash& h) { io.raw(h.data(), 32); };
    H(pf.rX0); H(pf.rRmsY[0]); H(pf.rRmsY[1]);
    for (auto& h : pf.rCodes) H(h);
    for (auto& h : pf.rScales) H(h);
    for (auto& h : pf.rMX) H(h);
    for (auto& h : pf.rMW) H(h);
    for (auto& h : pf.rRopeQ) H(h);
    for (auto& h : pf.rRopeO) H(h);
    for (auto& h : pf.rSmP) H(h);
    for (auto& h : pf.rVtX) H(h);
    H(pf.rAtX); H(pf.rRes1); H(pf.rSwM); H(pf.rOut);
    for (auto& y : pf.mmY) io.vec16(y);
    io.groups(pf.lug);
    io.vec(pf.seam);
    io.batches(pf.batches);
}
// p3mdl::MdlProof <-> bytes: u32 nlayers vocab seq d batch | per layer u32 len + TfProof | rEmb | u32 len + rmsF, qnF, mmH |
//   rRmsFY rCodesF rScalesF rMXH rMWH | u32 count + logits | u32 count + seam values | groups | batches
template <typename IO>
void mdl_walk(IO& io, p3mdl::MdlProof& pf, bool reading) {
    io.u32(pf.nlayers); io.u32(pf.vocab); io.u32(pf.seq); io.u32(pf.d); io.u32(pf.batch);
    if (reading) {
        if (pf.nlayers < 1 || pf.nlayers > 256) { io.fail(); return; }
        pf.lay.resize(pf.nlayers);
    }
    for (auto& l : pf.lay) io.sub(l, [reading](auto& i2, p3tf::TfProof& y) { tf_walk(i2, y, reading); });
    io.raw(pf.rEmb.data(), 32);
    io.sub(pf.rmsF, [](auto& i2, p3rms::RmsProof& y) { rms_walk(i2, y); });
    io.sub(pf.qnF, [](auto& i2, p3qnt::QntProof& y) { qnt_walk(i2, y); });
    io.sub(pf.mmH, [](auto& i2, p3hwl::LayerProof& y) { hwl_walk(i2, y); });
    for (auto* h : {&pf.rRmsFY, &pf.rCodesF, &pf.rScalesF, &pf.rMXH, &pf.rMWH}) io.raw(h->data(), 32);
    io.vec16(pf.mmYH);
    io.vec(pf.seam);
    io.groups(pf.lug);
    io.batches(pf.batches);
}
// the integer layer's public tables, built once per (d, btop) by the reference's own build_tables
const p3ig::Tables& ig_tables(uint32_t d, uint32_t btop) {
    static std::map<std::pair<uint32_t, uint32_t>, p3ig::Tables> cache;
    auto key = std::make_pair(d, btop);
    auto it = cache.find(key);
    if (it == cache.end()) it = cache.emplace(key, p3ig::build_tables(d, btop)).first;
    return it->second;
}
p3fri::Hash hash_from(const uint8_t* p) { p3fri::Hash h; memcpy(h.data(), p, 32); return h; }
p3lu::Col col_from(const uint64_t* v, size_t n, const uint8_t* root, uint32_t vreal) {
    p3lu::Col c;
    c.v.assign(v, v + n);
    if (root) memcpy(c.root.data(), root, 32);
    c.vreal = vreal;
    return c;
}
// p3irs::Proof (non-zk) <-> bytes: u32 le, sf, nl, rng | limb roots nl*32 | messages le*40 | yX yY yL[nl] |
//   u32 groups, each u32 len + GroupProof | u32 batches, each u32 len + BatchProof
size_t irs_serialize(const p3irs::Proof& pf, uint8_t* out, size_t cap) {
    std::vector<uint8_t> b;
    auto app = [&](const void* s, size_t n) { const uint8_t* q = (const uint8_t*)s; b.insert(b.end(), q, q + n); };
    app(&pf.le, 4); app(&pf.sf, 4); app(&pf.nl, 4); app(&pf.rng, 4);
    for (uint32_t l = 0; l < pf.nl; l++) app(pf.rL[l].data(), 32);
    for (auto& m : pf.m) app(&m, 40);
    app(&pf.yX, 8); app(&pf.yY, 8);
    for (uint32_t l = 0; l < pf.nl; l++) app(&pf.yL[l], 8);
    if (p3zkc::G.on) blind_serialize(pf.bl, b);
    std::vector<uint8_t> t((size_t)64 << 20);
    uint32_t ng = (uint32_t)pf.tail.lug.size();
    app(&ng, 4);
    for (auto& g : pf.tail.lug) {
        uint32_t n = (uint32_t)lu_serialize(g, t.data(), t.size());
        app(&n, 4); app(t.data(), n);
    }
    uint32_t nb = (uint32_t)pf.tail.batches.size();
    app(&nb, 4);
    for (auto& bp : pf.tail.batches) {
        uint32_t n = (uint32_t)bo_serialize(bp, t.data(), t.size());
        app(&n, 4); app(t.data(), n);
    }
    if (b.size() > cap) return 0;
    memcpy(out, b.data(), b.size());
    return b.size();
}
bool irs_deserialize(const uint8_t* in, size_t len, p3irs::Proof& pf) {
    const uint8_t* p = in; const uint8_t* end = in + len;
    auto need = [&](size_t n) { return (size_t)(end - p) >= n; };
    if (!need(16)) return false;
    memcpy(&pf.le, p, 4); memcpy(&pf.sf, p + 4, 4); memcpy(&pf.nl, p + 8, 4); memcpy(&pf.rng, p + 12, 4); p += 16;
    if (pf.le > 40 || pf.nl < 1 || pf.nl > 2) return false;
    const uint32_t lch = p3zkc::vfull(pf.le);
    if (!need((size_t)pf.nl * 40 + (size_t)lch * 40 + 16 + 4)) return false;
    for (uint32_t l = 0; l < pf.nl; l++) { memcpy(pf.rL[l].data(), p, 32); p += 32; }
    pf.m.resize(lch);
    for (auto& m : pf.m) { memcpy(&m, p, 40); p += 40; }
    memcpy(&pf.yX, p, 8); memcpy(&pf.yY, p + 8, 8); p += 16;
    for (uint32_t l = 0; l < pf.nl; l++) { memcpy(&pf.yL[l], p, 8); p += 8; }
    if (p3zkc::G.on && !blind_deserialize(p, end, pf.bl)) return false;
    if (!need(4)) return false;
    uint32_t ng; memcpy(&ng, p, 4); p += 4;
    if (ng > 64) return false;
    pf.tail.lug.resize(ng);
    for (auto& g : pf.tail.lug) {
        uint32_t n;
        if (!need(4)) return false;
        memcpy(&n, p, 4); p += 4;
        if (!need(n) || !lu_deserialize(p, n, g)) return false;
        p += n;
    }
    if (!need(4)) return false;
    uint32_t nb; memcpy(&nb, p, 4); p += 4;
    if (nb > 64) return false;
    pf.tail.batches.resize(nb);
    for (auto& bp : pf.tail.batches) {
        uint32_t n;
        if (!need(4)) return false;
        memcpy(&n, p, 4); p += 4;
        if (!need(n) || !bo_deserialize(p, n, bp)) return false;
        p += n;
    }
    return p == end;
}
// the five range tables the rescale gadget looks up into (p3_int_gadgets.cuh:60-75)
p3ig::Tables irs_tables(uint32_t sf) {
    p3ig::Tables T;
    T.btop = sf > 16 && sf < 32 ? sf - 16 : 1;
    T.R16 = p3ig::range_table(16, 0);
    T.R14 = p3ig::range_table(14, 0);
    T.RTOP = p3ig::range_table(T.btop, 0);
    T.RS16 = p3ig::range_table(16, -(1LL << 15));
    T.RS20 = p3ig::range_table(20, -(1LL << 19));
    return T;
}
struct FProd2 { static __device__ gl_t eval(const gl_t* c, const gl_t*) { return gl_mul(c[0], c[1]); } };
struct M3 { gl_t s[3]; };
struct M4 { gl_t s[4]; };
struct M5 { gl_t s[5]; };
}  // namespace

static const char* g_last_why = "";

extern "C" {

// ---- field ----
uint64_t ref_gl_add(uint64_t a, uint64_t b) { return gl_add(a, b); }
uint64_t ref_gl_sub(uint64_t a, uint64_t b) { return gl_sub(a, b); }
uint64_t ref_gl_mul(uint64_t a, uint64_t b) { return gl_mul(a, b); }
uint64_t ref_gl_pow(uint64_t a, uint64_t e) { return gl_pow(a, e); }
uint64_t ref_gl_inv(uint64_t a) { return gl_inv(a); }
uint64_t ref_gl_root_of_unity(uint32_t logn) { return gl_root_of_unity(logn); }

// ---- hashing / transcript ----
void ref_sha256(const void* d, size_t n, uint8_t out[32]) { fs::sha256(d, n, out); }
void ref_sha256_compress64(const uint8_t in[64], uint8_t out[32]) { p3_sha256_compress64(in, out); }
void ref_tr_init(uint8_t st[32], const void* seed, size_t n) {
    fs::Transcript tr(std::string((const char*)seed, n));
    memcpy(st, tr.state, 32);
}
void ref_tr_absorb(uint8_t st[32], const char* label, const void* data, uint64_t len) {
    fs::Transcript tr = tr_from(st);
    tr.absorb(label, data, (size_t)len);
    memcpy(st, tr.state, 32);
}
void ref_tr_challenge_bytes(uint8_t st[32], uint8_t out[32]) {
    fs::Transcript tr = tr_from(st);
    tr.challenge_bytes(out);
    memcpy(st, tr.state, 32);
}
uint64_t ref_tr_chal(uint8_t st[32]) {
    fs::Transcript tr = tr_from(st);
    gl_t a = p3sg::chal(tr);
    memcpy(st, tr.state, 32);
    return a;
}
uint64_t ref_tr_idx(uint8_t st[32], uint64_t mod) {
    fs::Transcript tr = tr_from(st);
    uint64_t a = p3fri::idx_from(tr, mod);
    memcpy(st, tr.state, 32);
    return a;
}

// ---- multilinear helpers ----
void ref_build_eq(const uint64_t* z, uint32_t v, uint64_t* out) {
    std::vector<gl_t> zz(z, z + v);
    auto w = p3bf::build_eq(zz);
    memcpy(out, w.data(), w.size() * 8);
}
uint64_t ref_eval_h(const uint64_t* c, const uint64_t* eq, size_t n) {
    return p3bf::eval_h(std::vector<gl_t>(c, c + n), std::vector<gl_t>(eq, eq + n));
}
uint64_t ref_quad_eval(uint64_t s0, uint64_t s1, uint64_t s2, uint64_t t) {
    return p3bf::quad_eval(s0, s1, s2, t);
}
uint64_t ref_cubic_eval(uint64_t s0, uint64_t s1, uint64_t s2, uint64_t s3, uint64_t t) {
    return p3lu::cubic_eval(s0, s1, s2, s3, t);
}
uint64_t ref_quartic_eval(const uint64_t s[5], uint64_t t) {
    p3hwl::Msg5 m{s[0], s[1], s[2], s[3], s[4]};
    return p3hwl::quartic_eval(m, t);
}
uint64_t ref_eq_point(const uint64_t* a, const uint64_t* z, uint32_t v) {
    return p3bf::eq_point(std::vector<gl_t>(a, a + v), std::vector<gl_t>(z, z + v));
}

// ---- encode / merkle / fold (host paths) ----
void ref_rs_encode_horner(const uint64_t* c, uint32_t v, uint32_t R, uint64_t* cw) {
    auto w = p3bf::rs_encode(std::vector<gl_t>(c, c + ((size_t)1 << v)), R);
    memcpy(cw, w.data(), w.size() * 8);
}
void ref_merkle_build(const uint64_t* cw, size_t M, uint8_t* tree) {
    p3fri::g_gpu_merkle = false;
    p3fri::Merkle mk; mk.build(std::vector<gl_t>(cw, cw + M));
    uint8_t* p = tree;
    for (auto& lv : mk.levels) for (auto& h : lv) put(p, h.data(), 32);
}
void ref_merkle_root(const uint64_t* cw, size_t M, uint8_t root[32]) {
    p3fri::g_gpu_merkle = false;
    p3fri::Merkle mk; mk.build(std::vector<gl_t>(cw, cw + M));
    memcpy(root, mk.root().data(), 32);
}
void ref_fold(const uint64_t* f, size_t M, uint64_t wM, uint64_t beta, int mle, uint64_t* out) {
    auto o = p3fri::fold(std::vector<gl_t>(f, f + M), wM, beta, mle != 0);
    memcpy(out, o.data(), o.size() * 8);
}

// ---- Basefold opening (host path) + verifier ----
size_t ref_bf_prove_eval(const uint64_t* c, const uint64_t* z, uint32_t v, uint64_t y, uint32_t R,
                         uint32_t Q, const uint64_t* cw0, const char* seed, uint8_t* out, size_t cap) {
    p3fri::g_gpu_merkle = false;
    size_t N = (size_t)1 << v, M0 = (size_t)1 << (v + R);
    auto pf = p3bf::prove_eval(std::vector<gl_t>(c, c + N), std::vector<gl_t>(z, z + v), y, R, Q,
                               std::vector<gl_t>(cw0, cw0 + M0), seed);
    return bf_serialize(pf, out, cap);
}
int ref_bf_verify_eval(const uint8_t* proof, size_t len, const char* seed) {
    p3bf::EvalProof pf;
    if (!bf_deserialize(proof, len, pf)) return 0;
    return p3bf::verify_eval(pf, seed) ? 1 : 0;
}

// ---- GKR (host path) ----
size_t ref_gkr_prove(uint8_t st[32], const char* tag, const uint64_t* p, const uint64_t* q,
                     uint32_t L, int combine_last, uint64_t* rfin, uint64_t cpq[2], uint8_t* out,
                     size_t cap, int gpu) {
    fs::Transcript tr = tr_from(st);
    size_t N = (size_t)1 << L;
    std::vector<gl_t> rf;
    gl_t cp = 0, cq = 0;
    p3gkr::Proof pf;
    try {
        pf = p3gkr::prove(tr, tag, std::vector<gl_t>(p, p + N), std::vector<gl_t>(q, q + N),
                          combine_last != 0, rf, &cp, &cq, gpu != 0);
    } catch (...) { return 0; }
    memcpy(st, tr.state, 32);
    memcpy(rfin, rf.data(), rf.size() * 8);
    if (cpq) { cpq[0] = cp; cpq[1] = cq; }
    return gkr_serialize(pf, out, cap);
}
int ref_gkr_verify(uint8_t st[32], const char* tag, uint32_t L, const uint8_t* proof, size_t len,
                   int combine_last, uint64_t* rfin, uint64_t out4[4]) {
    p3gkr::Proof pf;
    if (!gkr_deserialize(proof, len, L, pf)) return 0;
    fs::Transcript tr = tr_from(st);
    std::vector<gl_t> rf;
    const char* why = nullptr;
    bool ok = p3gkr::verify(tr, tag, L, pf, combine_last != 0, rf, out4, &why);
    memcpy(st, tr.state, 32);
    if (ok) memcpy(rfin, rf.data(), rf.size() * 8);
    return ok ? 1 : 0;
}

// ---- host sumchecks: cubic logUp chain (Msg4) and generic quartic chain (Msg5) ----
int ref_lu_sc_prove(uint8_t st[32], const char* tag, const uint64_t* H, const uint64_t* V,
                    const uint64_t* E, const uint64_t* D, uint32_t logn, uint64_t lam, uint64_t beta,
                    uint64_t* msgs, uint64_t* chals) {
    fs::Transcript tr = tr_from(st);
    size_t n = (size_t)1 << logn;
    std::vector<p3lu::Msg4> m;
    auto r = p3lu::sc_prove(std::vector<gl_t>(H, H + n), std::vector<gl_t>(V, V + n),
                            std::vector<gl_t>(E, E + n), std::vector<gl_t>(D, D + n), lam, beta, tr,
                            tag, m);
    memcpy(st, tr.state, 32);
    memcpy(msgs, m.data(), m.size() * 32);
    memcpy(chals, r.data(), r.size() * 8);
    return 0;
}
// functor: 0 = c0*c1, 1 = c0*c1*c2 (message always 5 points: p3_hawkeye.cuh:659-695)
int ref_sc5_prove(uint8_t st[32], const char* tag, int functor, const uint64_t* const* cols, int nc,
                  uint32_t logn, uint64_t* msgs, uint64_t* chals) {
    fs::Transcript tr = tr_from(st);
    size_t n = (size_t)1 << logn;
    std::vector<std::vector<gl_t>> cc(nc);
    for (int k = 0; k < nc; k++) cc[k].assign(cols[k], cols[k] + n);
    p3hwl::CFn F;
    if (functor == 0) F = [](const gl_t* v) { return gl_mul(v[0], v[1]); };
    else if (functor == 1) F = [](const gl_t* v) { return gl_mul(v[0], gl_mul(v[1], v[2])); };
    else return -1;
    std::vector<p3hwl::Msg5> m;
    auto r = p3hwl::sc5_prove(tr, tag, std::move(cc), F, m);
    memcpy(st, tr.state, 32);
    memcpy(msgs, m.data(), m.size() * 40);
    memcpy(chals, r.data(), r.size() * 8);
    return 0;
}

// quartic zero-checks of the fp8 gadget on host cores: p3hwl::sc5_prove with the reference's own
// constraint functions (p3_hawkeye.cuh:850-1010).  functor 6..11 = F_dp, F_dg, F_ch, F_gs, F_ds, F_do.
int ref_sc5_prove_lam(uint8_t st[32], const char* tag, int functor, const uint64_t* const* cols, int nc,
                      uint32_t logn, const uint64_t* lam, int nlam, uint64_t* msgs, uint64_t* chals) {
    fs::Transcript tr = tr_from(st);
    size_t n = (size_t)1 << logn;
    std::vector<std::vector<gl_t>> cc(nc);
    for (int k = 0; k < nc; k++) cc[k].assign(cols[k], cols[k] + n);
    std::vector<gl_t> L(lam, lam + nlam);
    L.resize(64, 0);
    p3hwl::CFn F;
    if (functor == 6) F = [L](const gl_t* v) { return p3hwl::F_dp(v, L.data()); };
    else if (functor == 7) F = [L](const gl_t* v) { return p3hwl::F_dg(v, L.data()); };
    else if (functor == 8) F = [L](const gl_t* v) { return p3hwl::F_ch(v, L.data()); };
    else if (functor == 9) F = [L](const gl_t* v) { return p3hwl::F_gs(v, L.data()); };
    else if (functor == 10) F = [L](const gl_t* v) { return p3hwl::F_ds(v, L.data()); };
    else if (functor == 11) F = [L](const gl_t* v) { return p3hwl::F_do(v, L.data()); };
    else return -1;
    std::vector<p3hwl::Msg5> m;
    auto r = p3hwl::sc5_prove(tr, tag, std::move(cc), F, m);
    memcpy(st, tr.state, 32);
    memcpy(msgs, m.data(), m.size() * 40);
    memcpy(chals, r.data(), r.size() * 8);
    return 0;
}

// ---- logUp primitives ----
int ref_inv_all_add(const uint64_t* A, size_t n, uint64_t beta, uint64_t* out) {
    try {
        auto o = p3lu::inv_all_add(std::vector<gl_t>(A, A + n), beta);
        memcpy(out, o.data(), n * 8);
    } catch (...) { return -1; }
    return 0;
}
void ref_combine(const uint64_t* const* cols, int c, size_t n, uint64_t g, uint64_t* out) {
    std::vector<std::vector<gl_t>> cc(c);
    std::vector<const std::vector<gl_t>*> pp(c);
    for (int k = 0; k < c; k++) { cc[k].assign(cols[k], cols[k] + n); pp[k] = &cc[k]; }
    auto o = p3lu::combine(pp, g);
    memcpy(out, o.data(), n * 8);
}

// ---- the zk switch of the reference (p3zkc::G, p3_zkc.cuh:83-97): on/off, query budget, master seed, structured-blind
// threshold; the draw counter restarts.  While it is on, the (de)serialisers above read and write the zk fields. ----
void ref_zk_set(int on, uint32_t Q, uint64_t seed, uint32_t sblind_min) {
    p3zkc::G = p3zkc::Ctx();
    p3zkc::G.on = on != 0;
    p3zkc::G.Q = Q;
    p3zkc::G.seed = seed;
    p3zkc::G.ctr = 0;
    p3zkc::G.sblind_min = sblind_min;
}
uint64_t ref_zk_next_seed() { return p3zkc::next_seed(); }
uint32_t ref_zk_e_of(uint32_t v) { return p3zkc::e_of(v); }

// ---- batched opening: the reference's host-only verifier (p3_batchopen.cuh:1149-1302) ----
int ref_bo_verify_class(uint8_t st[32], uint32_t v, const uint64_t* pts, uint32_t T, const uint8_t* roots,
                        const uint32_t* zid, const uint64_t* y, uint32_t k, uint32_t R, uint32_t Q,
                        const char* label, const uint8_t* proof, size_t len) {
    p3bo::BatchProof pf;
    if (!bo_deserialize(proof, len, pf)) return 0;
    p3bo::VLedger::Cls C;
    C.v = v;
    for (uint32_t t = 0; t < T; t++) C.pts.push_back(std::vector<gl_t>(pts + (size_t)t * v, pts + (size_t)(t + 1) * v));
    for (uint32_t j = 0; j < k; j++) {
        p3fri::Hash h; memcpy(h.data(), roots + (size_t)j * 32, 32);
        C.ents.push_back({h, zid[j], y[j]});
    }
    fs::Transcript tr = tr_from(st);
    const char* why = nullptr;
    bool ok = p3bo::verify_class(tr, C, pf, Q, R, label, &why);
    memcpy(st, tr.state, 32);
    return ok ? 1 : 0;
}

// ---- merged lookup: the reference's host-only verifier (p3_logup.cuh:1958-2086 verify_super) ----
// Members are listed in flush order, subgroup after subgroup (K = sum of sub_k); wit_committed[j*c+t]
// tells whether column t of member j is a committed column (its root at wit_roots) or virtual.
// The verifier's opening-ledger additions come back in insertion order.
int ref_lu_verify_super(uint8_t st[32], const uint64_t* const* tcols, uint32_t m, uint32_t c, uint32_t ns,
                        const uint32_t* sub_n, const uint32_t* sub_k, const uint8_t* wit_roots,
                        const uint8_t* wit_committed, uint32_t R, uint32_t Q, const uint8_t* proof, size_t len,
                        uint32_t* n_claims, uint8_t* claim_roots, uint32_t* claim_vlen, uint64_t* claim_pts,
                        uint64_t* claim_y, uint32_t max_claims) {
    p3lu::GroupProof pf;
    if (!lu_deserialize(proof, len, pf)) return 0;
    std::vector<std::vector<gl_t>> cols(c);
    for (uint32_t t = 0; t < c; t++) cols[t].assign(tcols[t], tcols[t] + ((size_t)1 << m));
    p3lu::Table T = p3lu::make_table(cols);
    uint32_t K = 0;
    for (uint32_t s = 0; s < ns; s++) K += sub_k[s];
    std::vector<p3fri::Hash> roots((size_t)K * c);
    for (size_t i = 0; i < roots.size(); i++) memcpy(roots[i].data(), wit_roots + i * 32, 32);
    p3lu::VCtx V;
    std::vector<std::vector<size_t>> smi(ns);
    std::vector<uint32_t> sns(sub_n, sub_n + ns);
    size_t j = 0;
    for (uint32_t s = 0; s < ns; s++)
        for (uint32_t i = 0; i < sub_k[s]; i++, j++) {
            std::vector<const p3fri::Hash*> rp(c);
            for (uint32_t t = 0; t < c; t++) rp[t] = wit_committed[j * c + t] ? &roots[j * c + t] : nullptr;
            p3lu::vdefer_v(V, rp, T, sub_n[s], "m");
            smi[s].push_back(j);
        }
    fs::Transcript tr = tr_from(st);
    const char* why = nullptr;
    bool ok = p3lu::verify_super(tr, V, smi, sns, pf, Q, R, &why);
    memcpy(st, tr.state, 32);
    if (!ok) return 0;
    uint32_t nc = 0;
    for (auto& cl : V.vlg.cls)
        for (auto& e : cl.ents) (void)e, nc++;
    // ledger classes are keyed by size; return entries class by class, in class creation order
    uint32_t w = 0;
    for (auto& cl : V.vlg.cls)
        for (auto& e : cl.ents) {
            if (w >= max_claims) return 0;
            memcpy(claim_roots + (size_t)w * 32, e.root.data(), 32);
            claim_vlen[w] = cl.v;
            memcpy(claim_pts + (size_t)w * 64, cl.pts[e.zid].data(), (size_t)cl.v * 8);
            claim_y[w] = e.y;
            w++;
        }
    *n_claims = w;
    return 1;
}

// ---- standalone logUp (p3_logup.cuh:932-1163 prove_v, :1170-1350 verify_v), non-zk, per-instance openings.
// committed[k] != 0: column k is committed (root given / produced); else virtual.  gpu = 0 runs everything on
// host cores (Horner encode: small instances only).
size_t ref_lu_prove_v(uint8_t st[32], const uint64_t* const* tcols, uint32_t m, uint32_t c, const uint64_t* const* wcols,
                      const uint8_t* committed, const uint32_t* idx, uint32_t n, uint32_t R, uint32_t Q, const char* label,
                      int gpu, uint8_t* wroots_out, uint64_t* rA_out, uint8_t* out, size_t cap) {
    try {
        p3fri::g_gpu_merkle = gpu != 0;
        std::vector<std::vector<gl_t>> tc(c);
        for (uint32_t t = 0; t < c; t++) tc[t].assign(tcols[t], tcols[t] + ((size_t)1 << m));
        p3lu::Table T = p3lu::make_table(tc);
        std::vector<p3lu::Col> cols(c);
        std::vector<std::vector<gl_t>> virt(c);
        std::vector<p3lu::LuColSpec> W;
        for (uint32_t k = 0; k < c; k++) {
            std::vector<gl_t> v(wcols[k], wcols[k] + ((size_t)1 << n));
            if (committed[k]) {
                cols[k] = p3lu::commit_col(v, R, gpu != 0);
                memcpy(wroots_out + (size_t)k * 32, cols[k].root.data(), 32);
                W.push_back(p3lu::LC(&cols[k]));
            } else {
                virt[k] = v;
                W.push_back(p3lu::LV(&virt[k]));
            }
        }
        std::vector<uint32_t> ix(idx, idx + ((size_t)1 << n));
        fs::Transcript tr = tr_from(st);
        std::vector<gl_t> rA;
        auto pf = p3lu::prove_v(tr, W, ix, T, R, Q, label, gpu != 0, true, &rA);
        p3fri::g_gpu_merkle = false;
        memcpy(st, tr.state, 32);
        memcpy(rA_out, rA.data(), rA.size() * 8);
        return lup_serialize(pf, out, cap);
    } catch (...) { p3fri::g_gpu_merkle = false; return 0; }
}
int ref_lu_verify_v(uint8_t st[32], const uint64_t* const* tcols, uint32_t m, uint32_t c, const uint8_t* wroots,
                    const uint8_t* committed, uint32_t R, uint32_t Q, const char* label, const uint8_t* proof, size_t len,
                    uint64_t* rA_out, uint64_t* yvirt_out) {
    p3lu::LookupProof pf;
    if (!lup_deserialize(proof, len, pf)) return 0;
    std::vector<std::vector<gl_t>> tc(c);
    for (uint32_t t = 0; t < c; t++) tc[t].assign(tcols[t], tcols[t] + ((size_t)1 << m));
    p3lu::Table T = p3lu::make_table(tc);
    std::vector<p3fri::Hash> roots(c);
    std::vector<const p3fri::Hash*> rp(c);
    for (uint32_t k = 0; k < c; k++) {
        memcpy(roots[k].data(), wroots + (size_t)k * 32, 32);
        rp[k] = committed[k] ? &roots[k] : nullptr;
    }
    fs::Transcript tr = tr_from(st);
    const char* why = nullptr;
    std::vector<gl_t> rA, yv;
    bool ok = p3lu::verify_v(tr, rp, T, pf, Q, R, label, &why, &rA, &yv);
    memcpy(st, tr.state, 32);
    if (ok) {
        memcpy(rA_out, rA.data(), rA.size() * 8);
        memcpy(yvirt_out, yv.data(), yv.size() * 8);
    }
    return ok ? 1 : 0;
}

// ---- integer-layer tables: columns of the reference's build_tables (which: 0 EXPT, 1 SILU, 2 ISQ, 3 EXP4) ----
int ref_ig_table(uint32_t d, uint32_t btop, int which, uint64_t* const* cols_out, uint8_t id_out[32]) {
    const p3ig::Tables& T = ig_tables(d, btop);
    const p3lu::Table* t = which == 0 ? &T.EXPT : which == 1 ? &T.SILU : which == 2 ? &T.ISQ : which == 3 ? &T.EXP4 : nullptr;
    if (!t) return -1;
    for (size_t c = 0; c < t->cols.size(); c++) memcpy(cols_out[c], t->cols[c].data(), t->cols[c].size() * 8);
    memcpy(id_out, t->id.data(), 32);
    return (int)t->cols.size();
}
// ---- residual add / SwiGLU gadgets: host-only verifiers (p3_int_gadgets.cuh:739-773, :1834-1872) ----
int ref_iadd_verify(uint8_t st[32], const uint8_t* rA, const uint8_t* rB, const uint8_t* rO, uint32_t le, uint32_t R, uint32_t Q,
                    const uint8_t* proof, size_t len) {
    p3iadd::Proof pf;
    if (!iadd_deserialize(proof, len, pf)) return 0;
    fs::Transcript tr = tr_from(st);
    const char* why = nullptr;
    bool ok = p3iadd::verify(tr, ig_tables(64, 12), pf, hash_from(rA), hash_from(rB), hash_from(rO), le, Q, R, &why);
    memcpy(st, tr.state, 32);
    return ok ? 1 : 0;
}
int ref_iswg_verify(uint8_t st[32], const uint8_t* rG, const uint8_t* rU, const uint8_t* rM, uint32_t le, uint32_t R, uint32_t Q,
                    const uint8_t* proof, size_t len) {
    p3iswg::Proof pf;
    if (!iswg_deserialize(proof, len, pf)) return 0;
    fs::Transcript tr = tr_from(st);
    const char* why = nullptr;
    bool ok = p3iswg::verify(tr, ig_tables(64, 12), pf, hash_from(rG), hash_from(rU), hash_from(rM), le, Q, R, &why);
    memcpy(st, tr.state, 32);
    return ok ? 1 : 0;
}

int ref_irope_verify(uint8_t st[32], const int32_t* ct, const int32_t* sn, uint32_t lseq, uint32_t ldh, const uint8_t* rQ,
                     const uint8_t* rY, uint32_t lT, uint32_t ld, uint32_t R, uint32_t Q, const uint8_t* proof, size_t len) {
    p3irope::Proof pf;
    if (!irope_deserialize(proof, len, pf)) return 0;
    fs::Transcript tr = tr_from(st);
    const char* why = nullptr;
    bool ok = p3irope::verify(tr, ig_tables(64, 12), rope_pub(ct, sn, lseq, ldh), pf, hash_from(rQ), hash_from(rY), lT, ld, Q, R, &why);
    memcpy(st, tr.state, 32);
    return ok ? 1 : 0;
}

int ref_irms_verify(uint8_t st[32], const uint8_t* rX, const uint8_t* rG, const uint8_t* rY, uint32_t lT, uint32_t ld, uint32_t R,
                    uint32_t Q, const uint8_t* proof, size_t len) {
    p3irms::Proof pf;
    if (!irms_deserialize(proof, len, pf)) return 0;
    fs::Transcript tr = tr_from(st);
    const char* why = nullptr;
    bool ok = p3irms::verify(tr, ig_tables(1u << ld, 12), pf, hash_from(rX), hash_from(rG), hash_from(rY), lT, ld, Q, R, &why);
    memcpy(st, tr.state, 32);
    return ok ? 1 : 0;
}

int ref_ismx_verify(uint8_t st[32], const uint8_t* rZ, const uint8_t* rP, uint32_t la, uint32_t lseq, uint32_t R, uint32_t Q,
                    const uint8_t* proof, size_t len) {
    p3ismx::Proof pf;
    if (!ismx_deserialize(proof, len, pf)) return 0;
    fs::Transcript tr = tr_from(st);
    const char* why = nullptr;
    bool ok = p3ismx::verify(tr, ig_tables(64, 12), pf, hash_from(rZ), hash_from(rP), la, lseq, Q, R, &why);
    memcpy(st, tr.state, 32);
    return ok ? 1 : 0;
}

// ---- decoder layer: the reference's host-only verifier (p3_int_layer.cuh:584-737) ----
// wroots: the 7 weight roots then g1, g2 (9 x 32 bytes); x0 / outp: the public input and output grids
int ref_itf_verify(uint8_t st[32], const uint32_t dims[6], const uint64_t* x0, const uint8_t* rX0, const uint8_t* wroots,
                   const int32_t* ct, const int32_t* sn, const uint64_t* outp, uint32_t R, uint32_t Q, const uint8_t* proof,
                   size_t len) {
    p3itf::TfProof pf;
    g_last_why = "proof bytes do not parse";
    if (!itf_deserialize(proof, len, pf)) return 0;
    p3itf::Config cfg;
    cfg.seq = dims[0]; cfg.d = dims[1]; cfg.nh = dims[2]; cfg.dh = dims[3]; cfg.dff = dims[4]; cfg.batch = dims[5];
    if (!cfg.pow2()) return 0;
    const size_t Ne = (size_t)cfg.T() * cfg.d;
    std::vector<gl_t> x0v(x0, x0 + Ne), outv(outp, outp + Ne);
    p3itf::WeightRoots wr;
    for (int i = 0; i < p3itf::NW; i++) wr.Wc[i] = hash_from(wroots + 32 * i);
    wr.G1 = hash_from(wroots + 32 * 7); wr.G2 = hash_from(wroots + 32 * 8);
    fs::Transcript tr = tr_from(st);
    const char* why = nullptr;
    bool ok = p3itf::verify(tr, pf, ig_tables(cfg.d, cfg.btop()), cfg, x0v, hash_from(rX0), wr,
                            rope_pub(ct, sn, cfg.lseq(), cfg.ldh()), outv, Q, R, &why);
    g_last_why = why ? why : "";
    memcpy(st, tr.state, 32);
    return ok ? 1 : 0;
}
// the reason string of the last ref_itf_verify call (the reference's `why`), for test diagnostics
const char* ref_last_why() { return g_last_why; }

// ---- integer matmul gadget: the reference's host-only verifier (p3_int_gadgets.cuh:608-655) ----
int ref_imm_verify(uint8_t st[32], const uint8_t rootX[32], const uint8_t rootW[32], const uint8_t rootY[32],
                   uint32_t lj, uint32_t lk, uint32_t li, uint32_t R, uint32_t Q, const uint8_t* proof, size_t len) {
    p3imm::Proof pf;
    if (!imm_deserialize(proof, len, pf)) return 0;
    p3imm::OpView xv = p3imm::direct_x(nullptr, lj, li), wv = p3imm::direct_w(nullptr, lj, lk),
                  yv = p3imm::direct_y(nullptr, lk, li);
    memcpy(xv.root.data(), rootX, 32); memcpy(wv.root.data(), rootW, 32); memcpy(yv.root.data(), rootY, 32);
    fs::Transcript tr = tr_from(st);
    const char* why = nullptr;
    bool ok = p3imm::verify(tr, pf, xv, wv, yv, lj, lk, li, Q, R, &why);
    memcpy(st, tr.state, 32);
    return ok ? 1 : 0;
}

// ---- rescale gadget: the reference's host-only verifier (p3_int_gadgets.cuh:342-388) ----
int ref_irs_verify(uint8_t st[32], const uint8_t rootX[32], const uint8_t rootY[32], uint32_t le, uint32_t sf,
                   int rng, uint32_t R, uint32_t Q, const uint8_t* proof, size_t len) {
    p3irs::Proof pf;
    if (!irs_deserialize(proof, len, pf)) return 0;
    p3ig::Tables T = irs_tables(sf);
    p3fri::Hash rX, rY;
    memcpy(rX.data(), rootX, 32); memcpy(rY.data(), rootY, 32);
    fs::Transcript tr = tr_from(st);
    const char* why = nullptr;
    bool ok = p3irs::verify(tr, T, pf, rX, rY, le, sf, rng, Q, R, &why);
    memcpy(st, tr.state, 32);
    return ok ? 1 : 0;
}
// p3irs::gen_witness (p3_int_gadgets.cuh:234-281): y, limbs and lookup indices from the accumulator
int ref_irs_witness(const uint64_t* acc, uint32_t le, uint32_t sf, int rng, uint64_t* y, uint64_t* L0, uint64_t* L1,
                    uint32_t* iL0, uint32_t* iL1, uint32_t* iY) {
    try {
        std::vector<gl_t> a(acc, acc + ((size_t)1 << le));
        p3irs::Wit w = p3irs::gen_witness(le, sf, rng, a);
        size_t N = (size_t)1 << le;
        memcpy(y, w.y.data(), N * 8); memcpy(L0, w.L[0].data(), N * 8); memcpy(iL0, w.idxL[0].data(), N * 4);
        if (w.nl == 2) { memcpy(L1, w.L[1].data(), N * 8); memcpy(iL1, w.idxL[1].data(), N * 4); }
        memcpy(iY, w.idxY.data(), N * 4);
        return (int)w.nl;
    } catch (...) { return 0; }
}

// =====================================================================
// GPU entry points: the reference's own CUDA paths (need a GPU).
// =====================================================================
// how many sumchecks the reference's gadget code sent through libzkh (only in the build that force-includes
// include/p3_scgpu_zkh.cuh; -1 in the plain build)
long long ref_zkh_sumcheck_calls() {
#ifdef sc_prove_gpu
    return (long long)p3sg::zkh_shim_calls().load();
#else
    return -1;
#endif
}
int ref_gpu_available() {
    int n = 0;
    return cudaGetDeviceCount(&n) == cudaSuccess && n > 0;
}
void ref_gpu_setup() { p3bf::p3_enable_mempool(); }
// p3sg::sc_prove_gpu over host columns (uploaded here, outside any timing the
// caller does with ref_sc_prove_gpu_dev).  functor: 0 c0*c1, 1 c0*c1*c2,
// 2 GKR (par = lam), 3 logUp (par = lam,beta).
static int sc_gpu_run(fs::Transcript& tr, const char* tag, int functor, int nt,
                      std::vector<gl_t*>& d, uint32_t N, const uint64_t* par, uint32_t npar,
                      uint64_t* msgs, uint64_t* chals) {
    std::vector<gl_t> r;
#define RUN(FF, MT, NT)                                                                   \
    { std::vector<MT> m; r = p3sg::sc_prove_gpu<FF, MT, NT, 8>(tr, tag, d, N, par, npar, m); \
      memcpy(msgs, m.data(), m.size() * sizeof(MT)); }
    if (functor == 0 && nt == 3) RUN(FProd2, M3, 3)
    else if (functor == 1 && nt == 4) RUN(p3imm::FImmGpu, M4, 4)
    else if (functor == 1 && nt == 5) RUN(p3imm::FImmGpu, M5, 5)
    else if (functor == 2 && nt == 4) RUN(p3gkr::FGkrGpu, M4, 4)
    else if (functor == 3 && nt == 4) RUN(p3lu::FLuGpu, M4, 4)
    else if (functor >= 6 && functor <= 9 && nt == 5) {
        std::vector<M5> m;
        if (functor == 6) r = p3sg::sc_prove_gpu<p3hwl::FFdp, M5, 5, 40>(tr, tag, d, N, par, npar, m);
        else if (functor == 7) r = p3sg::sc_prove_gpu<p3hwl::FFdg, M5, 5, 40>(tr, tag, d, N, par, npar, m);
        else if (functor == 8) r = p3sg::sc_prove_gpu<p3hwl::FFch, M5, 5, 40>(tr, tag, d, N, par, npar, m);
        else r = p3sg::sc_prove_gpu<p3hwl::FFgs, M5, 5, 40>(tr, tag, d, N, par, npar, m);
        memcpy(msgs, m.data(), m.size() * sizeof(M5));
    }
    else return -1;
#undef RUN
    memcpy(chals, r.data(), r.size() * 8);
    return 0;
}
int ref_sc_prove_gpu(uint8_t st[32], const char* tag, int functor, int nt,
                     const uint64_t* const* cols, int nc, uint32_t logn, const uint64_t* par,
                     uint32_t npar, uint64_t* msgs, uint64_t* chals, double* ms_out) {
    fs::Transcript tr = tr_from(st);
    uint32_t N = 1u << logn;
    std::vector<gl_t*> d(nc);
    for (int k = 0; k < nc; k++) {
        if (cudaMallocAsync(&d[k], (size_t)N * 8, 0) != cudaSuccess) return -2;
        cudaMemcpy(d[k], cols[k], (size_t)N * 8, cudaMemcpyHostToDevice);
    }
    cudaDeviceSynchronize();
    double t0 = p3bf::bf_now_ms();
    int rc = sc_gpu_run(tr, tag, functor, nt, d, N, par, npar, msgs, chals);
    cudaDeviceSynchronize();
    if (ms_out) *ms_out = p3bf::bf_now_ms() - t0;
    for (auto p : d) cudaFreeAsync(p, 0);
    cudaDeviceSynchronize();
    memcpy(st, tr.state, 32);
    return cudaGetLastError() == cudaSuccess ? rc : -3;
}
int ref_commit_gpu_rootonly(const uint64_t* c, uint32_t v, uint32_t R, uint8_t root[32], double* ms_out) {
    try {
        std::vector<gl_t> cc(c, c + ((size_t)1 << v));
        cudaDeviceSynchronize();
        double t0 = p3bf::bf_now_ms();
        auto h = p3bf::commit_gpu_rootonly(cc, R);
        cudaDeviceSynchronize();
        if (ms_out) *ms_out = p3bf::bf_now_ms() - t0;
        memcpy(root, h.data(), 32);
    } catch (...) { return -1; }
    return 0;
}
int ref_rs_encode_gpu(const uint64_t* c, uint32_t v, uint32_t R, uint64_t* cw) {
    auto w = p3bf::rs_encode_gpu(std::vector<gl_t>(c, c + ((size_t)1 << v)), R);
    memcpy(cw, w.data(), w.size() * 8);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
size_t ref_bf_prove_eval_dev(const uint64_t* c, const uint64_t* z, uint32_t v, uint64_t y, uint32_t R,
                             uint32_t Q, const uint64_t* cw0, const char* seed, uint8_t* out,
                             size_t cap, double* ms_out) {
    size_t N = (size_t)1 << v, M0 = (size_t)1 << (v + R);
    std::vector<gl_t> cc(c, c + N), zz(z, z + v), cw(cw0, cw0 + M0);
    cudaDeviceSynchronize();
    double t0 = p3bf::bf_now_ms();
    auto pf = p3bf::prove_eval_dev(cc, zz, y, R, Q, cw, seed);
    cudaDeviceSynchronize();
    if (ms_out) *ms_out = p3bf::bf_now_ms() - t0;
    return bf_serialize(pf, out, cap);
}

// p3bo::prove_class (GPU): cols[j] = host values of entry j (entries with equal roots share values)
size_t ref_bo_prove_class(uint8_t st[32], uint32_t v, const uint64_t* pts, uint32_t T,
                          const uint64_t* const* cols, const uint8_t* roots, const uint32_t* zid, uint32_t k,
                          uint32_t R, uint32_t Q, const char* label, uint8_t* out, size_t cap, double* ms_out) {
    p3fri::g_gpu_merkle = true;
    size_t N = (size_t)1 << v;
    std::vector<std::vector<gl_t>> vals(k);
    p3bo::PLedger::Cls C;
    C.v = v;
    for (uint32_t t = 0; t < T; t++) C.pts.push_back(std::vector<gl_t>(pts + (size_t)t * v, pts + (size_t)(t + 1) * v));
    for (uint32_t j = 0; j < k; j++) {
        vals[j].assign(cols[j], cols[j] + N);
        p3fri::Hash h; memcpy(h.data(), roots + (size_t)j * 32, 32);
        C.ents.push_back({&vals[j], h, zid[j], 0, 0, {}, {}});
    }
    fs::Transcript tr = tr_from(st);
    size_t n = 0;
    try {
        cudaDeviceSynchronize();
        double t0 = p3bf::bf_now_ms();
        auto pf = p3bo::prove_class(tr, C, R, Q, label);
        cudaDeviceSynchronize();
        if (ms_out) *ms_out = p3bf::bf_now_ms() - t0;
        n = bo_serialize(pf, out, cap);
    } catch (...) { n = 0; }
    p3fri::g_gpu_merkle = false;
    memcpy(st, tr.state, 32);
    return n;
}

// p3lu::prove_super (GPU): all columns committed (roots given), host values; idx per member
size_t ref_lu_prove_super(uint8_t st[32], const uint64_t* const* tcols, uint32_t m, uint32_t c, uint32_t ns,
                          const uint32_t* sub_n, const uint32_t* sub_k, const uint64_t* const* wit_cols,
                          const uint8_t* wit_roots, const uint32_t* const* idx, uint32_t R, uint32_t Q,
                          uint8_t* out, size_t cap, double* ms_out) {
    p3fri::g_gpu_merkle = true;
    std::vector<std::vector<gl_t>> cols(c);
    for (uint32_t t = 0; t < c; t++) cols[t].assign(tcols[t], tcols[t] + ((size_t)1 << m));
    p3lu::Table T = p3lu::make_table(cols);
    uint32_t K = 0;
    for (uint32_t s = 0; s < ns; s++) K += sub_k[s];
    std::vector<p3lu::Col> wc((size_t)K * c);
    std::vector<std::vector<uint32_t>> ix(K);
    p3lu::XCtx xc;
    std::vector<std::vector<size_t>> smi(ns);
    std::vector<uint32_t> sns(sub_n, sub_n + ns);
    size_t j = 0;
    for (uint32_t s = 0; s < ns; s++)
        for (uint32_t i = 0; i < sub_k[s]; i++, j++) {
            size_t N = (size_t)1 << sub_n[s];
            std::vector<p3lu::LuColSpec> W;
            for (uint32_t t = 0; t < c; t++) {
                p3lu::Col& col = wc[j * c + t];
                col.v.assign(wit_cols[j * c + t], wit_cols[j * c + t] + N);
                memcpy(col.root.data(), wit_roots + (j * c + t) * 32, 32);
                col.vreal = sub_n[s];
                W.push_back(p3lu::LC(&col));
            }
            ix[j].assign(idx[j], idx[j] + N);
            p3lu::defer_v(xc, W, ix[j], T, "m");
            smi[s].push_back(j);
        }
    fs::Transcript tr = tr_from(st);
    size_t n = 0;
    try {
        cudaDeviceSynchronize();
        double t0 = p3bf::bf_now_ms();
        auto pf = p3lu::prove_super(tr, xc, smi, sns, R, Q, true, true);
        cudaDeviceSynchronize();
        if (ms_out) *ms_out = p3bf::bf_now_ms() - t0;
        n = lu_serialize(pf, out, cap);
    } catch (...) { n = 0; }
    p3fri::g_gpu_merkle = false;
    memcpy(st, tr.state, 32);
    return n;
}

// p3imm::prove (GPU): host values + given commitment roots of X [j | i<<lj], W [k | j<<lk], Y [k | i<<lk]
size_t ref_imm_prove(uint8_t st[32], const uint64_t* X, const uint64_t* W, const uint64_t* Y, const uint8_t rootX[32],
                     const uint8_t rootW[32], const uint8_t rootY[32], uint32_t lj, uint32_t lk, uint32_t li,
                     uint32_t R, uint32_t Q, uint8_t* out, size_t cap, double* ms_out) {
    p3fri::g_gpu_merkle = true;
    p3lu::Col cx, cw, cy;
    cx.v.assign(X, X + ((size_t)1 << (lj + li))); memcpy(cx.root.data(), rootX, 32); cx.vreal = lj + li;
    cw.v.assign(W, W + ((size_t)1 << (lj + lk))); memcpy(cw.root.data(), rootW, 32); cw.vreal = lj + lk;
    cy.v.assign(Y, Y + ((size_t)1 << (lk + li))); memcpy(cy.root.data(), rootY, 32); cy.vreal = lk + li;
    fs::Transcript tr = tr_from(st);
    size_t n = 0;
    try {
        cudaDeviceSynchronize();
        double t0 = p3bf::bf_now_ms();
        auto pf = p3imm::prove(tr, p3imm::direct_x(&cx, lj, li), p3imm::direct_w(&cw, lj, lk),
                               p3imm::direct_y(&cy, lk, li), lj, lk, li, R, Q);
        cudaDeviceSynchronize();
        if (ms_out) *ms_out = p3bf::bf_now_ms() - t0;
        n = imm_serialize(pf, out, cap);
    } catch (...) { n = 0; }
    p3fri::g_gpu_merkle = false;
    memcpy(st, tr.state, 32);
    return n;
}

// p3irs::prove with the zk switch on (GPU): X = acc and Y = the rescaled output committed by the reference (fresh masks),
// limb commitments, deferred range lookups, blinded zero-check, flush and blinded batched openings.  roots_out: X, Y.
size_t ref_irs_prove_zk(uint8_t st[32], const uint64_t* acc, uint32_t le, uint32_t sf, int rng, uint32_t R, uint32_t Q,
                        uint64_t seed, uint32_t sblind_min, uint8_t* out, size_t cap, uint8_t* roots_out, double* ms_out) {
    p3fri::g_gpu_merkle = true;
    ref_zk_set(1, Q, seed, sblind_min);
    fs::Transcript tr = tr_from(st);
    size_t n = 0;
    try {
        std::vector<gl_t> a(acc, acc + ((size_t)1 << le));
        p3irs::Wit w = p3irs::gen_witness(le, sf, rng, a);
        p3ig::Tables T = irs_tables(sf);
        p3lu::Col CX = p3lu::commit_col_nc(w.acc, R), CY = p3lu::commit_col_nc(w.y, R);
        memcpy(roots_out, CX.root.data(), 32); memcpy(roots_out + 32, CY.root.data(), 32);
        p3irs::Operands o{&CX, &CY};
        cudaDeviceSynchronize();
        double t0 = p3bf::bf_now_ms();
        p3irs::Proof pf = p3irs::prove(tr, w, T, o, R, Q);
        cudaDeviceSynchronize();
        if (ms_out) *ms_out = p3bf::bf_now_ms() - t0;
        n = irs_serialize(pf, out, cap);
    } catch (...) { n = 0; }
    p3fri::g_gpu_merkle = false;
    ref_zk_set(0, 24, 1, 22);
    memcpy(st, tr.state, 32);
    return n;
}

// p3imm::prove with the zk switch on (GPU): operands committed by the reference (fresh masks, salted leaves), Y with the
// mask linkage of its selftest (p3_int_selftest.cu:89-100); roots_out: X, W, Y.  The switch is off again on return.
size_t ref_imm_prove_zk(uint8_t st[32], const uint64_t* X, const uint64_t* W, uint32_t lj, uint32_t lk, uint32_t li,
                        uint32_t R, uint32_t Q, uint64_t seed, uint32_t sblind_min, uint8_t* out, size_t cap,
                        uint8_t* roots_out, double* ms_out) {
    p3fri::g_gpu_merkle = true;
    ref_zk_set(1, Q, seed, sblind_min);
    fs::Transcript tr = tr_from(st);
    size_t n = 0;
    try {
        std::vector<gl_t> xv_((size_t)1 << (lj + li)), wv_((size_t)1 << (lj + lk));
        memcpy(xv_.data(), X, xv_.size() * 8); memcpy(wv_.data(), W, wv_.size() * 8);
        p3lu::Col cx = p3lu::commit_col_nc(xv_, R), cw = p3lu::commit_col_nc(wv_, R);
        p3imm::OpView xv = p3imm::direct_x(&cx, lj, li), wv = p3imm::direct_w(&cw, lj, lk);
        std::vector<gl_t> Y = p3imm::compute_y(xv_, xv, wv_, wv, lj, lk, li);
        p3imm::OpView yv = p3imm::direct_y(nullptr, lk, li);
        std::vector<gl_t> m1((size_t)1 << (lk + li), 0);
        p3imm::accum_mask1(m1, xv, wv, yv, lj, lk, li);
        std::vector<gl_t> mask = p3zkc::mk_linked(lk + li, m1);
        p3lu::Col cy = p3lu::commit_col_nc(Y, R, &mask);
        yv.c = &cy; yv.root = cy.root;
        memcpy(roots_out, cx.root.data(), 32); memcpy(roots_out + 32, cw.root.data(), 32); memcpy(roots_out + 64, cy.root.data(), 32);
        cudaDeviceSynchronize();
        double t0 = p3bf::bf_now_ms();
        auto pf = p3imm::prove(tr, xv, wv, yv, lj, lk, li, R, Q);
        cudaDeviceSynchronize();
        if (ms_out) *ms_out = p3bf::bf_now_ms() - t0;
        n = imm_serialize(pf, out, cap);
    } catch (...) { n = 0; }
    p3fri::g_gpu_merkle = false;
    ref_zk_set(0, 24, 1, 22);
    memcpy(st, tr.state, 32);
    return n;
}

// p3irs::prove (commitments, lookup flush and batched openings on the GPU): host accumulator values and
// the commitment roots of X (= acc) and Y (= the rescaled output, as gen_witness computes it)
size_t ref_irs_prove(uint8_t st[32], const uint64_t* acc, const uint8_t rootX[32], const uint8_t rootY[32],
                     uint32_t le, uint32_t sf, int rng, uint32_t R, uint32_t Q, uint8_t* out, size_t cap,
                     double* ms_out) {
    p3fri::g_gpu_merkle = true;
    fs::Transcript tr = tr_from(st);
    size_t n = 0;
    try {
        std::vector<gl_t> a(acc, acc + ((size_t)1 << le));
        p3ig::Tables T = irs_tables(sf);
        cudaDeviceSynchronize();
        double t0 = p3bf::bf_now_ms();
        p3irs::Wit w = p3irs::gen_witness(le, sf, rng, a);
        p3lu::Col cx, cy;
        cx.v = w.acc; memcpy(cx.root.data(), rootX, 32); cx.vreal = le;
        cy.v = w.y;   memcpy(cy.root.data(), rootY, 32); cy.vreal = le;
        p3irs::Operands ops{&cx, &cy};
        auto pf = p3irs::prove(tr, w, T, ops, R, Q);
        cudaDeviceSynchronize();
        if (ms_out) *ms_out = p3bf::bf_now_ms() - t0;
        n = irs_serialize(pf, out, cap);
    } catch (...) { n = 0; }
    p3fri::g_gpu_merkle = false;
    memcpy(st, tr.state, 32);
    return n;
}

// p3iadd::prove / p3iswg::prove with the reference's own witness replay; commitments, lookups and openings on the GPU
size_t ref_iadd_prove(uint8_t st[32], const uint64_t* a, const uint64_t* b, const uint8_t* rA, const uint8_t* rB,
                      const uint8_t* rO, uint32_t le, uint32_t R, uint32_t Q, uint8_t* out, size_t cap, double* ms_out) {
    p3fri::g_gpu_merkle = true;
    fs::Transcript tr = tr_from(st);
    size_t n = 0;
    try {
        const size_t N = (size_t)1 << le;
        std::vector<gl_t> av(a, a + N), bv(b, b + N);
        const p3ig::Tables& T = ig_tables(64, 12);
        cudaDeviceSynchronize();
        double t0 = p3bf::bf_now_ms();
        p3iadd::Wit w = p3iadd::gen_witness(le, av, bv);
        p3lu::Col ca = col_from(a, N, rA, le), cb = col_from(b, N, rB, le), co = col_from(w.out.data(), N, rO, le);
        p3iadd::Operands ops{&ca, &cb, &co};
        auto pf = p3iadd::prove(tr, w, T, ops, R, Q);
        cudaDeviceSynchronize();
        if (ms_out) *ms_out = p3bf::bf_now_ms() - t0;
        n = iadd_serialize(pf, out, cap);
    } catch (...) { n = 0; }
    p3fri::g_gpu_merkle = false;
    memcpy(st, tr.state, 32);
    return n;
}
size_t ref_iswg_prove(uint8_t st[32], const uint64_t* g, const uint64_t* u, const uint8_t* rG, const uint8_t* rU,
                      const uint8_t* rM, uint32_t le, uint32_t R, uint32_t Q, uint8_t* out, size_t cap, double* ms_out) {
    p3fri::g_gpu_merkle = true;
    fs::Transcript tr = tr_from(st);
    size_t n = 0;
    try {
        const size_t N = (size_t)1 << le;
        std::vector<gl_t> gv(g, g + N), uv(u, u + N);
        const p3ig::Tables& T = ig_tables(64, 12);
        cudaDeviceSynchronize();
        double t0 = p3bf::bf_now_ms();
        p3iswg::Wit w = p3iswg::gen_witness(le, gv, uv, T);
        p3lu::Col cg = col_from(g, N, rG, le), cu = col_from(u, N, rU, le), cm = col_from(w.mo.data(), N, rM, le);
        p3iswg::Operands ops{&cg, &cu, &cm};
        auto pf = p3iswg::prove(tr, w, T, ops, R, Q);
        cudaDeviceSynchronize();
        if (ms_out) *ms_out = p3bf::bf_now_ms() - t0;
        n = iswg_serialize(pf, out, cap);
    } catch (...) { n = 0; }
    p3fri::g_gpu_merkle = false;
    memcpy(st, tr.state, 32);
    return n;
}

size_t ref_irope_prove(uint8_t st[32], const uint64_t* q, const int32_t* ct, const int32_t* sn, uint32_t lseq, uint32_t ldh,
                       const uint8_t* rQ, const uint8_t* rY, uint32_t lT, uint32_t ld, uint32_t R, uint32_t Q, uint8_t* out,
                       size_t cap, double* ms_out) {
    p3fri::g_gpu_merkle = true;
    fs::Transcript tr = tr_from(st);
    size_t n = 0;
    try {
        const size_t N = (size_t)1 << (lT + ld);
        std::vector<gl_t> qv(q, q + N);
        const p3ig::Tables& T = ig_tables(64, 12);
        p3irope::Pub P = rope_pub(ct, sn, lseq, ldh);
        cudaDeviceSynchronize();
        double t0 = p3bf::bf_now_ms();
        p3irope::Wit w = p3irope::gen_witness(lT, ld, P, qv);
        p3lu::Col cq = col_from(q, N, rQ, lT + ld), cy = col_from(w.y.data(), N, rY, lT + ld);
        p3irope::Operands ops{&cq, &cy};
        auto pf = p3irope::prove(tr, w, T, P, ops, R, Q);
        cudaDeviceSynchronize();
        if (ms_out) *ms_out = p3bf::bf_now_ms() - t0;
        n = irope_serialize(pf, out, cap);
    } catch (...) { n = 0; }
    p3fri::g_gpu_merkle = false;
    memcpy(st, tr.state, 32);
    return n;
}

size_t ref_irms_prove(uint8_t st[32], const uint64_t* x, const uint64_t* g, const uint8_t* rX, const uint8_t* rG, const uint8_t* rY,
                      uint32_t lT, uint32_t ld, uint32_t R, uint32_t Q, uint8_t* out, size_t cap, double* ms_out) {
    p3fri::g_gpu_merkle = true;
    fs::Transcript tr = tr_from(st);
    size_t n = 0;
    try {
        const size_t N = (size_t)1 << (lT + ld), D = (size_t)1 << ld;
        std::vector<gl_t> xv(x, x + N), gv(g, g + D);
        const p3ig::Tables& T = ig_tables(1u << ld, 12);
        cudaDeviceSynchronize();
        double t0 = p3bf::bf_now_ms();
        p3irms::Wit w = p3irms::gen_witness(lT, ld, xv, gv, T);
        p3lu::Col cx = col_from(x, N, rX, lT + ld), cg = col_from(g, D, rG, ld), cy = col_from(w.y.data(), N, rY, lT + ld);
        p3irms::Operands ops{&cx, &cg, &cy};
        auto pf = p3irms::prove(tr, w, T, ops, R, Q);
        cudaDeviceSynchronize();
        if (ms_out) *ms_out = p3bf::bf_now_ms() - t0;
        n = irms_serialize(pf, out, cap);
    } catch (...) { n = 0; }
    p3fri::g_gpu_merkle = false;
    memcpy(st, tr.state, 32);
    return n;
}

size_t ref_ismx_prove(uint8_t st[32], const uint64_t* z, const uint8_t* rZ, const uint8_t* rP, uint32_t la, uint32_t lseq,
                      uint32_t R, uint32_t Q, uint8_t* out, size_t cap, double* ms_out) {
    p3fri::g_gpu_merkle = true;
    fs::Transcript tr = tr_from(st);
    size_t n = 0;
    try {
        const uint32_t le = la + 2 * lseq;
        const size_t N = (size_t)1 << le;
        std::vector<gl_t> zv(z, z + N);
        const p3ig::Tables& T = ig_tables(64, 12);
        cudaDeviceSynchronize();
        double t0 = p3bf::bf_now_ms();
        p3ismx::Wit w = p3ismx::gen_witness(la, lseq, zv, T);
        p3lu::Col cz = col_from(z, N, rZ, le), cp = col_from(w.p.data(), N, rP, le);
        p3ismx::Operands ops{&cz, &cp};
        auto pf = p3ismx::prove(tr, w, T, ops, R, Q);
        cudaDeviceSynchronize();
        if (ms_out) *ms_out = p3bf::bf_now_ms() - t0;
        n = ismx_serialize(pf, out, cap);
    } catch (...) { n = 0; }
    p3fri::g_gpu_merkle = false;
    memcpy(st, tr.state, 32);
    return n;
}

// p3itf: build_witness (host) + commit_all + prove (GPU) of one decoder layer; ms_out[0] witness, [1] commit, [2] prove
size_t ref_itf_prove(uint8_t st[32], const uint32_t dims[6], const uint64_t* x0, const uint64_t* const* w7, const uint64_t* g1,
                     const uint64_t* g2, const int32_t* ct, const int32_t* sn, uint32_t R, uint32_t Q, uint8_t* out, size_t cap,
                     uint64_t* out_grid, double* ms_out) {
    p3fri::g_gpu_merkle = true;
    p3bf::p3_enable_mempool();
    fs::Transcript tr = tr_from(st);
    size_t n = 0;
    try {
        p3itf::Config cfg;
        cfg.seq = dims[0]; cfg.d = dims[1]; cfg.nh = dims[2]; cfg.dh = dims[3]; cfg.dff = dims[4]; cfg.batch = dims[5];
        const size_t Ne = (size_t)cfg.T() * cfg.d;
        p3itf::Weights W = itf_weights(cfg, w7, g1, g2, ct, sn);
        const p3ig::Tables& T = ig_tables(cfg.d, cfg.btop());
        std::vector<gl_t> x0v(x0, x0 + Ne);
        cudaDeviceSynchronize();
        double t0 = p3bf::bf_now_ms();
        p3itf::TfWit w = p3itf::build_witness(cfg, x0v, W, T);
        double t1 = p3bf::bf_now_ms();
        p3itf::TfOps o = p3itf::commit_all(w, W, R);
        cudaDeviceSynchronize();
        double t2 = p3bf::bf_now_ms();
        auto pf = p3itf::prove(tr, w, o, W, T, R, Q);
        cudaDeviceSynchronize();
        double t3 = p3bf::bf_now_ms();
        if (ms_out) { ms_out[0] = t1 - t0; ms_out[1] = t2 - t1; ms_out[2] = t3 - t2; }
        if (out_grid) memcpy(out_grid, w.out.data(), Ne * 8);
        n = itf_serialize(pf, out, cap);
    } catch (...) { n = 0; }
    p3fri::g_gpu_merkle = false;
    memcpy(st, tr.state, 32);
    return n;
}

// ---- p3hwl: the fp8 (Hawkeye) matmul gadget ----
// public table `which` (0..15 in the order the prover absorbs them): rows and column count, columns copied when given
int ref_hwl_table(int which, uint64_t* const* cols_out, uint32_t* rows_out, uint8_t id_out[32]) {
    const p3lu::Table* t = hwl_table_at(which);
    if (!t) return 0;
    if (rows_out) *rows_out = (uint32_t)t->cols[0].size();
    if (cols_out) for (size_t c = 0; c < t->cols.size(); c++) memcpy(cols_out[c], t->cols[c].data(), t->cols[c].size() * 8);
    if (id_out) memcpy(id_out, t->id.data(), 32);
    return (int)t->cols.size();
}
// p3hwl::gen_witness on the host.  dom: 0 dp, 1 dg, 2 dob, 3 db, 4 dn (column `col` copied to out64), 5 lookup indices of
// instance `col` (copied to out32), 6 the bf16 output (B*N uint16 to out32's memory).  Returns elements written, 0 on throw.
size_t ref_hwl_witness(uint32_t B, uint32_t K, uint32_t N, const uint8_t* x, const uint8_t* w, const uint32_t* xs, const uint32_t* ws,
                       int dom, int col, uint64_t* out64, uint32_t* out32) {
    try {
        static p3hwl::LayerWit wt; static std::vector<uint8_t> key;
        std::vector<uint8_t> k2;
        auto app = [&](const void* s, size_t n) { const uint8_t* q = (const uint8_t*)s; k2.insert(k2.end(), q, q + n); };
        uint32_t d3[3] = {B, K, N}; app(d3, 12); app(x, (size_t)B * K); app(w, (size_t)N * K); app(xs, 4 * B); app(ws, 4 * N);
        if (k2 != key) { wt = p3hwl::gen_witness(hwl_golden(B, K, N, x, w, xs, ws), true); key = k2; }
        const std::vector<gl_t>* v = nullptr;
        if (dom == 0 && col < p3hwl::NDP) v = &wt.dp[col];
        else if (dom == 1 && col < p3hwl::NDG) v = &wt.dg[col];
        else if (dom == 2 && col < p3hwl::NDO) v = &wt.dob[col];
        else if (dom == 3 && col < p3hwl::NDS) v = &wt.db[col];
        else if (dom == 4 && col < p3hwl::NDS) v = &wt.dn[col];
        if (v) { memcpy(out64, v->data(), v->size() * 8); return v->size(); }
        if (dom == 5 && col < p3hwl::NLU) { memcpy(out32, wt.lidx[col].data(), wt.lidx[col].size() * 4); return wt.lidx[col].size(); }
        if (dom == 6) { memcpy(out32, wt.Y.data(), wt.Y.size() * 2); return wt.Y.size(); }
    } catch (...) {}
    return 0;
}
// gen_witness + commit_operands + prove; roots4_out: X W XS WS roots; Y_out: B*N bf16 patterns; ms_out[0] witness,
// [1] operand commits, [2] prove
size_t ref_hwl_prove(uint8_t st[32], uint32_t B, uint32_t K, uint32_t N, const uint8_t* x, const uint8_t* w, const uint32_t* xs,
                     const uint32_t* ws, uint32_t R, uint32_t Q, int gpu, uint8_t* roots4_out, uint16_t* Y_out, uint8_t* out,
                     size_t cap, double* ms_out) {
    p3fri::g_gpu_merkle = gpu != 0;
    if (gpu) p3bf::p3_enable_mempool();
    fs::Transcript tr = tr_from(st);
    size_t n = 0;
    try {
        const p3hwl::Tables& T = hwl_tables();
        double t0 = p3bf::bf_now_ms();
        p3hwl::LayerWit wt = p3hwl::gen_witness(hwl_golden(B, K, N, x, w, xs, ws), false);
        double t1 = p3bf::bf_now_ms();
        p3hwl::Operands ops = p3hwl::commit_operands(wt, R, gpu != 0);
        if (gpu) cudaDeviceSynchronize();
        double t2 = p3bf::bf_now_ms();
        auto pf = p3hwl::prove(tr, wt, T, ops, R, Q, gpu != 0);
        if (gpu) cudaDeviceSynchronize();
        double t3 = p3bf::bf_now_ms();
        if (ms_out) { ms_out[0] = t1 - t0; ms_out[1] = t2 - t1; ms_out[2] = t3 - t2; }
        if (roots4_out) {
            memcpy(roots4_out, ops.X.root.data(), 32); memcpy(roots4_out + 32, ops.W.root.data(), 32);
            memcpy(roots4_out + 64, ops.XS.root.data(), 32); memcpy(roots4_out + 96, ops.WS.root.data(), 32);
        }
        if (Y_out) memcpy(Y_out, wt.Y.data(), wt.Y.size() * 2);
        n = hwl_serialize(pf, out, cap);
    } catch (...) { n = 0; }
    p3fri::g_gpu_merkle = false;
    memcpy(st, tr.state, 32);
    return n;
}
// p3hwl::verify (host only) on the serialised proof
int ref_hwl_verify(uint8_t st[32], uint32_t B, uint32_t K, uint32_t N, const uint8_t* roots4, const uint16_t* Y, uint32_t R,
                   uint32_t Q, const uint8_t* proof, size_t len) {
    fs::Transcript tr = tr_from(st);
    int ok = 0;
    try {
        p3hwl::LayerProof pf;
        if (hwl_deserialize(proof, len, pf)) {
            p3fri::Hash r[4];
            for (int i = 0; i < 4; i++) memcpy(r[i].data(), roots4 + 32 * i, 32);
            std::vector<uint16_t> Yv(Y, Y + (size_t)B * N);
            ok = p3hwl::verify(tr, hwl_tables(), pf, r[0], r[1], r[2], r[3], Yv, B, K, N, Q, R) ? 1 : 0;
        }
    } catch (...) { ok = 0; }
    memcpy(st, tr.state, 32);
    return ok;
}

// ---- bf16 gadgets of the fp8 transformer layer ----
// load the pinned table artefact (the file p3rms::load_art reads); call once before any gadget entry point below
int ref_tf_load_art(const char* path) { return p3rms::load_art(path, tf_art()) ? 1 : 0; }
// p3swg::verify (host only)
int ref_swg_verify(uint8_t st[32], const uint8_t* rG, const uint8_t* rU, const uint8_t* rM, uint32_t n, uint32_t R, uint32_t Q,
                   const uint8_t* proof, size_t len) {
    fs::Transcript tr = tr_from(st);
    int ok = 0;
    try {
        p3swg::SwgProof pf;
        HwlReader rd{proof, proof + len};
        swg_walk(rd, pf);
        if (rd.ok && rd.p == rd.end) {
            p3fri::Hash h[3];
            memcpy(h[0].data(), rG, 32); memcpy(h[1].data(), rU, 32); memcpy(h[2].data(), rM, 32);
            ok = p3swg::verify(tr, swg_tables(), pf, h[0], h[1], h[2], n, Q, R) ? 1 : 0;
        }
    } catch (...) { ok = 0; }
    memcpy(st, tr.state, 32);
    return ok;
}
// p3swg: gen_witness + commit_operands + prove; roots3_out: GATE UP M roots; M_out: n bf16 patterns
size_t ref_swg_prove(uint8_t st[32], const uint16_t* gate, const uint16_t* up, uint32_t n, uint32_t R, uint32_t Q, int gpu,
                     uint8_t* roots3_out, uint16_t* M_out, uint8_t* out, size_t cap) {
    p3fri::g_gpu_merkle = gpu != 0;
    if (gpu) p3bf::p3_enable_mempool();
    fs::Transcript tr = tr_from(st);
    size_t w = 0;
    try {
        p3swg::Golden L; L.n = n; L.gate.assign(gate, gate + n); L.up.assign(up, up + n); L.m.assign(n, 0);
        p3swg::Wit wt = p3swg::gen_witness(L, tf_art());
        p3swg::Operands ops = p3swg::commit_operands(wt, R);
        auto pf = p3swg::prove(tr, wt, swg_tables(), ops, R, Q);
        if (roots3_out) {
            memcpy(roots3_out, ops.GATE.root.data(), 32); memcpy(roots3_out + 32, ops.UP.root.data(), 32);
            memcpy(roots3_out + 64, ops.M.root.data(), 32);
        }
        if (M_out) memcpy(M_out, wt.M.data(), (size_t)n * 2);
        HwlWriter wr;
        swg_walk(wr, pf);
        w = emit(wr.b, out, cap);
    } catch (...) { w = 0; }
    p3fri::g_gpu_merkle = false;
    memcpy(st, tr.state, 32);
    return w;
}

// p3bfa::verify (host only)
int ref_bfa_verify(uint8_t st[32], const uint8_t* r1, const uint8_t* r2, const uint8_t* ro, uint32_t n, uint32_t R, uint32_t Q,
                   const uint8_t* proof, size_t len) {
    fs::Transcript tr = tr_from(st);
    int ok = 0;
    try {
        p3bfa::BfaProof pf;
        HwlReader rd{proof, proof + len};
        bfa_walk(rd, pf);
        if (rd.ok && rd.p == rd.end) {
            p3fri::Hash h[3];
            memcpy(h[0].data(), r1, 32); memcpy(h[1].data(), r2, 32); memcpy(h[2].data(), ro, 32);
            ok = p3bfa::verify(tr, bfa_tables(), pf, h[0], h[1], h[2], n, Q, R) ? 1 : 0;
        }
    } catch (...) { ok = 0; }
    memcpy(st, tr.state, 32);
    return ok;
}
// p3bfa: gen_witness + commit_operands + prove; roots3_out: X1 X2 OUT roots; O_out: n bf16 patterns
size_t ref_bfa_prove(uint8_t st[32], const uint16_t* a, const uint16_t* b, uint32_t n, uint32_t R, uint32_t Q, int gpu,
                     uint8_t* roots3_out, uint16_t* O_out, uint8_t* out, size_t cap) {
    p3fri::g_gpu_merkle = gpu != 0;
    if (gpu) p3bf::p3_enable_mempool();
    fs::Transcript tr = tr_from(st);
    size_t w = 0;
    try {
        p3bfa::Golden L; L.n = n; L.a.assign(a, a + n); L.b.assign(b, b + n); L.o.assign(n, 0);
        p3bfa::Wit wt = p3bfa::gen_witness(L);
        p3bfa::Operands ops = p3bfa::commit_operands(wt, R);
        auto pf = p3bfa::prove(tr, wt, bfa_tables(), ops, R, Q);
        if (roots3_out) {
            memcpy(roots3_out, ops.X1.root.data(), 32); memcpy(roots3_out + 32, ops.X2.root.data(), 32);
            memcpy(roots3_out + 64, ops.OUT.root.data(), 32);
        }
        if (O_out) memcpy(O_out, wt.O.data(), (size_t)n * 2);
        HwlWriter wr;
        bfa_walk(wr, pf);
        w = emit(wr.b, out, cap);
    } catch (...) { w = 0; }
    p3fri::g_gpu_merkle = false;
    memcpy(st, tr.state, 32);
    return w;
}

// p3qnt::verify (host only): roots X CODES SCALES
int ref_qnt_verify(uint8_t st[32], const uint8_t* roots3, uint32_t B, uint32_t ld, uint32_t R, uint32_t Q, const uint8_t* proof, size_t len) {
    fs::Transcript tr = tr_from(st);
    int ok = 0;
    try {
        p3qnt::QntProof pf;
        HwlReader rd{proof, proof + len};
        qnt_walk(rd, pf);
        if (rd.ok && rd.p == rd.end) {
            p3fri::Hash h[3];
            for (int i = 0; i < 3; i++) memcpy(h[i].data(), roots3 + 32 * i, 32);
            ok = p3qnt::verify(tr, qnt_tables(), pf, h[0], h[1], h[2], B, ld, Q, R) ? 1 : 0;
        }
    } catch (...) { ok = 0; }
    memcpy(st, tr.state, 32);
    return ok;
}
// p3qnt: gen_witness + commit_operands + prove; codes_out: B*d codes, scales_out: B fp32 bit patterns
size_t ref_qnt_prove(uint8_t st[32], const uint16_t* x, uint32_t B, uint32_t ld, uint32_t R, uint32_t Q, int gpu, uint8_t* roots3_out,
                     uint8_t* codes_out, uint32_t* scales_out, uint8_t* out, size_t cap) {
    p3fri::g_gpu_merkle = gpu != 0;
    if (gpu) p3bf::p3_enable_mempool();
    fs::Transcript tr = tr_from(st);
    size_t w = 0;
    try {
        p3qnt::Golden L; L.B = B; L.d = 1u << ld;
        const size_t n = (size_t)B << ld;
        L.x.assign(x, x + n); L.codes.assign(n, 0); L.scales.assign(B, 0);
        p3qnt::Wit wt = p3qnt::gen_witness(L, tf_art());
        p3qnt::Operands ops = p3qnt::commit_operands(wt, R);
        auto pf = p3qnt::prove(tr, wt, qnt_tables(), ops, R, Q);
        if (roots3_out) {
            memcpy(roots3_out, ops.X.root.data(), 32); memcpy(roots3_out + 32, ops.CODES.root.data(), 32);
            memcpy(roots3_out + 64, ops.SCALES.root.data(), 32);
        }
        if (codes_out) memcpy(codes_out, wt.C.data(), n);
        if (scales_out) memcpy(scales_out, wt.S.data(), (size_t)B * 4);
        HwlWriter wr;
        qnt_walk(wr, pf);
        w = emit(wr.b, out, cap);
    } catch (...) { w = 0; }
    p3fri::g_gpu_merkle = false;
    memcpy(st, tr.state, 32);
    return w;
}
// p3rope::verify (host only): cos / sin bf16 tables of seq * dh/2 patterns, roots Q OUT
int ref_rope_verify(uint8_t st[32], const uint16_t* cosp, const uint16_t* sinp, const uint8_t* roots2, uint32_t seq, uint32_t dh,
                    uint32_t R, uint32_t Q, const uint8_t* proof, size_t len) {
    fs::Transcript tr = tr_from(st);
    int ok = 0;
    try {
        p3rope::RopeProof pf;
        HwlReader rd{proof, proof + len};
        rope_walk(rd, pf);
        if (rd.ok && rd.p == rd.end) {
            p3fri::Hash h[2];
            for (int i = 0; i < 2; i++) memcpy(h[i].data(), roots2 + 32 * i, 32);
            const size_t nh = (size_t)seq * (dh / 2);
            std::vector<uint16_t> c(cosp, cosp + nh), s2(sinp, sinp + nh);
            ok = p3rope::verify(tr, rope_tables(), pf, c, s2, h[0], h[1], seq, dh, Q, R) ? 1 : 0;
        }
    } catch (...) { ok = 0; }
    memcpy(st, tr.state, 32);
    return ok;
}
// p3rms::verify (host only): roots X G Y
int ref_rms_verify(uint8_t st[32], const uint8_t* roots3, uint32_t B, uint32_t ld, uint32_t R, uint32_t Q, const uint8_t* proof, size_t len) {
    fs::Transcript tr = tr_from(st);
    int ok = 0;
    try {
        p3rms::RmsProof pf;
        HwlReader rd{proof, proof + len};
        rms_walk(rd, pf);
        if (rd.ok && rd.p == rd.end) {
            static p3rms::Tables T; static int64_t t_ld = -1;
            if (t_ld != tf_art().ld) { T = p3rms::build_tables(tf_art()); t_ld = tf_art().ld; }
            p3fri::Hash h[3];
            for (int i = 0; i < 3; i++) memcpy(h[i].data(), roots3 + 32 * i, 32);
            ok = p3rms::verify(tr, T, tf_art(), pf, h[0], h[1], h[2], B, ld, Q, R) ? 1 : 0;
        }
    } catch (...) { ok = 0; }
    memcpy(st, tr.state, 32);
    return ok;
}
// p3smx::verify (host only): mask of B*n bytes, roots S P
int ref_smx_verify(uint8_t st[32], const uint8_t* mask, const uint8_t* roots2, uint32_t B, uint32_t n, uint32_t wmax, uint32_t R,
                   uint32_t Q, const uint8_t* proof, size_t len) {
    fs::Transcript tr = tr_from(st);
    int ok = 0;
    try {
        p3smx::SmxProof pf;
        HwlReader rd{proof, proof + len};
        smx_walk(rd, pf);
        if (rd.ok && rd.p == rd.end) {
            static p3smx::Tables T; static uint32_t t_w = 0;
            if (t_w != wmax) { T = p3smx::build_tables(tf_art(), wmax); t_w = wmax; }
            p3fri::Hash h[2];
            for (int i = 0; i < 2; i++) memcpy(h[i].data(), roots2 + 32 * i, 32);
            std::vector<uint8_t> m(mask, mask + (size_t)B * n);
            ok = p3smx::verify(tr, T, tf_art(), pf, m, h[0], h[1], B, n, Q, R) ? 1 : 0;
        }
    } catch (...) { ok = 0; }
    memcpy(st, tr.state, 32);
    return ok;
}

// p3tf::verify (host only) of one composed fp8 transformer layer.  dims: seq d nh dh dff batch; x0 / out: T*d bf16 patterns;
// rX0: root of the committed input; wroots: 16 roots (7 weight codes, 7 weight scales, g1, g2); cos / sin: seq*dh/2 patterns
int ref_tf_verify(uint8_t st[32], const uint32_t dims[6], const uint16_t* x0, const uint8_t* rX0, const uint8_t* wroots,
                  const uint16_t* cosp, const uint16_t* sinp, const uint16_t* outp, uint32_t smx_wmax, uint32_t R, uint32_t Q,
                  const uint8_t* proof, size_t len) {
    fs::Transcript tr = tr_from(st);
    int ok = 0;
    try {
        p3tf::TfProof pf;
        HwlReader rd{proof, proof + len};
        tf_walk(rd, pf, true);
        if (rd.ok && rd.p == rd.end) {
            p3tf::Config c; c.seq = dims[0]; c.d = dims[1]; c.nh = dims[2]; c.dh = dims[3]; c.dff = dims[4]; c.batch = dims[5];
            static p3tf::TfTables T; static int64_t t_ld = -1; static uint32_t t_w = 0;
            if (t_ld != tf_art().ld || t_w != smx_wmax) { T = p3tf::build_tables(tf_art(), smx_wmax); t_ld = tf_art().ld; t_w = smx_wmax; }
            p3tf::WeightRoots wr;
            for (int i = 0; i < p3tf::NW; i++) {
                memcpy(wr.Wc[i].data(), wroots + 32 * i, 32);
                memcpy(wr.Ws[i].data(), wroots + 32 * (p3tf::NW + i), 32);
            }
            memcpy(wr.G1.data(), wroots + 32 * 14, 32); memcpy(wr.G2.data(), wroots + 32 * 15, 32);
            p3fri::Hash hx; memcpy(hx.data(), rX0, 32);
            const size_t n = (size_t)c.T() * c.d, nh2 = (size_t)c.seq * (c.dh / 2);
            std::vector<uint16_t> xv(x0, x0 + n), ov(outp, outp + n), cv(cosp, cosp + nh2), sv(sinp, sinp + nh2);
            ok = p3tf::verify(tr, pf, T, tf_art(), c, xv, hx, wr, cv, sv, ov, Q, R) ? 1 : 0;
        }
    } catch (...) { ok = 0; }
    memcpy(st, tr.state, 32);
    return ok;
}

// p3mdl::verify_model (host only).  roots: E, GF, WHc, WHs, then 16 per layer (7 weight codes, 7 weight scales, g1, g2);
// ids: T token ids; logits: T*vocab bf16 patterns
int ref_mdl_verify(uint8_t st[32], const uint32_t dims[6], uint32_t nlayers, uint32_t vocab, const uint32_t* ids, const uint8_t* roots,
                   const uint16_t* cosp, const uint16_t* sinp, const uint16_t* logits, uint32_t smx_wmax, uint32_t R, uint32_t Q,
                   const uint8_t* proof, size_t len) {
    fs::Transcript tr = tr_from(st);
    int ok = 0;
    try {
        p3mdl::MdlProof pf;
        HwlReader rd{proof, proof + len};
        mdl_walk(rd, pf, true);
        if (rd.ok && rd.p == rd.end) {
            p3tf::Config c; c.seq = dims[0]; c.d = dims[1]; c.nh = dims[2]; c.dh = dims[3]; c.dff = dims[4]; c.batch = dims[5];
            static p3tf::TfTables T; static int64_t t_ld = -1; static uint32_t t_w = 0;
            if (t_ld != tf_art().ld || t_w != smx_wmax) { T = p3tf::build_tables(tf_art(), smx_wmax); t_ld = tf_art().ld; t_w = smx_wmax; }
            p3mdl::MdlRoots mr;
            auto H = [&](p3fri::Hash& h, size_t i) { memcpy(h.data(), roots + 32 * i, 32); };
            H(mr.E, 0); H(mr.GF, 1); H(mr.WHc, 2); H(mr.WHs, 3);
            mr.lw.resize(nlayers);
            for (uint32_t li = 0; li < nlayers; li++) {
                const size_t b = 4 + (size_t)16 * li;
                for (int i = 0; i < p3tf::NW; i++) { H(mr.lw[li].Wc[i], b + i); H(mr.lw[li].Ws[i], b + p3tf::NW + i); }
                H(mr.lw[li].G1, b + 14); H(mr.lw[li].G2, b + 15);
            }
            const size_t nh2 = (size_t)c.seq * (c.dh / 2);
            std::vector<uint32_t> idv(ids, ids + c.T());
            std::vector<uint16_t> cv(cosp, cosp + nh2), sv(sinp, sinp + nh2), lv(logits, logits + (size_t)c.T() * vocab);
            ok = p3mdl::verify_model(tr, pf, T, tf_art(), c, nlayers, vocab, idv, mr, cv, sv, lv, Q, R) ? 1 : 0;
        }
    } catch (...) { ok = 0; }
    memcpy(st, tr.state, 32);
    return ok;
}

// ---- hiding commitment (p3_zkc.cuh) ----
// host: p3zkc::salted_leaf(v, p3zkc::salt_of(sseed, i))
void ref_salted_leaf(uint64_t v, uint64_t sseed, uint64_t i, uint8_t out[32]) {
    p3fri::Hash h = p3zkc::salted_leaf(v, p3zkc::salt_of(sseed, i));
    memcpy(out, h.data(), 32);
}
// GPU: p3zkc::salted_commit_root_dev of 2^v values with salting on
int ref_salted_commit_root(const uint64_t* c, uint32_t v, uint32_t R, uint64_t sseed, uint8_t root[32]) {
    int rc = 0;
    const bool was = p3zkc::G.salt_on;
    try {
        p3fri::g_gpu_merkle = true;
        p3zkc::G.salt_on = true;
        const size_t n = (size_t)1 << v;
        gl_t* d = p3bf::dmalloc(n, "shim:salt");
        cudaMemcpy(d, c, n * 8, cudaMemcpyHostToDevice);
        p3fri::Hash h = p3zkc::salted_commit_root_dev(d, n, R, sseed);
        cudaFreeAsync(d, 0);
        cudaDeviceSynchronize();
        memcpy(root, h.data(), 32);
    } catch (...) { rc = -1; }
    p3zkc::G.salt_on = was;
    p3fri::g_gpu_merkle = false;
    return rc;
}

// host: p3zkc::zprng_fill (the mask chain) and p3zkc::zprng_at (the random-access stream)
void ref_zprng_fill(uint64_t s, uint64_t* out, size_t n) { p3zkc::zprng_fill(s, out, n); }
uint64_t ref_zprng_at(uint64_t seed, uint64_t i) { return p3zkc::zprng_at(seed, i); }

// p3tf: build_witness (host) + commit_all + prove (GPU) of one fp8 transformer layer.  wcodes[i] / wscales[i]: the 7 weight
// matrices (N*K codes, N fp32 bit patterns) in the order q k v o g u d; ms_out[0] witness, [1] commit, [2] prove
size_t ref_tf_prove(uint8_t st[32], const uint32_t dims[6], const uint16_t* x0, const uint8_t* const* wcodes, const uint32_t* const* wscales,
                    const uint16_t* g1, const uint16_t* g2, const uint16_t* cosp, const uint16_t* sinp, uint32_t smx_wmax, uint32_t R,
                    uint32_t Q, uint8_t* out, size_t cap, uint16_t* out_act, double* ms_out) {
    p3fri::g_gpu_merkle = true;
    p3bf::p3_enable_mempool();
    fs::Transcript tr = tr_from(st);
    size_t n = 0;
    try {
        p3tf::Config c; c.seq = dims[0]; c.d = dims[1]; c.nh = dims[2]; c.dh = dims[3]; c.dff = dims[4]; c.batch = dims[5];
        p3tf::Weights W; W.cfg = c;
        const uint32_t NK[7][2] = {{c.d, c.d}, {c.d, c.d}, {c.d, c.d}, {c.d, c.d}, {c.dff, c.d}, {c.dff, c.d}, {c.d, c.dff}};
        for (int i = 0; i < p3tf::NW; i++) {
            W.w[i].N = NK[i][0]; W.w[i].K = NK[i][1];
            W.w[i].codes.assign(wcodes[i], wcodes[i] + (size_t)NK[i][0] * NK[i][1]);
            W.w[i].scales.assign(wscales[i], wscales[i] + NK[i][0]);
        }
        const size_t nh2 = (size_t)c.seq * (c.dh / 2), ne = (size_t)c.T() * c.d;
        W.g1.assign(g1, g1 + c.d); W.g2.assign(g2, g2 + c.d);
        W.cos.assign(cosp, cosp + nh2); W.sin.assign(sinp, sinp + nh2);
        static p3tf::TfTables T; static int64_t t_ld = -1; static uint32_t t_w = 0;
        if (t_ld != tf_art().ld || t_w != smx_wmax) { T = p3tf::build_tables(tf_art(), smx_wmax); t_ld = tf_art().ld; t_w = smx_wmax; }
        std::vector<uint16_t> xv(x0, x0 + ne);
        cudaDeviceSynchronize();
        double t0 = p3bf::bf_now_ms();
        p3tf::TfWit w = p3tf::build_witness(c, xv, W, tf_art());
        double t1 = p3bf::bf_now_ms();
        p3tf::TfOps o = p3tf::commit_all(w, R);
        cudaDeviceSynchronize();
        double t2 = p3bf::bf_now_ms();
        auto pf = p3tf::prove(tr, w, o, T, tf_art(), R, Q);
        cudaDeviceSynchronize();
        double t3 = p3bf::bf_now_ms();
        if (ms_out) { ms_out[0] = t1 - t0; ms_out[1] = t2 - t1; ms_out[2] = t3 - t2; }
        if (out_act) memcpy(out_act, w.outp.data(), ne * 2);
        HwlWriter wr;
        tf_walk(wr, pf, false);
        n = emit(wr.b, out, cap);
    } catch (...) { n = 0; }
    p3fri::g_gpu_merkle = false;
    memcpy(st, tr.state, 32);
    return n;
}

}  // extern "C"
