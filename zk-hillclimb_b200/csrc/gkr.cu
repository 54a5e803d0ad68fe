// GKR fractional-sum tree prover over Goldilocks for sm_100a (logUp-GKR).
//
// Statement and schedule: zkllm-src/p3_gkr.cuh:200-364 (p3gkr::prove).  Leaves (p_i, q_i),
// levels combine (p', q') = (p1*q2 + p2*q1, q1*q2); the root (P, Q) is absorbed, then one cubic
// sumcheck per level reduces the claims to the leaves.
//
// The reference keeps levels above 2^13 nodes on the device and everything smaller on the
// host, copying partial sums to the host every round.  Here the whole tree and every layer
// sumcheck stay on the device with the transcript: the layer's challenges (lambda, mu and the
// round challenges) are drawn by device kernels and feed the next layer's eq table directly,
// and the children of a level are read in place (no split copy).  The host queues the whole
// proof and synchronises once.
#include "sumcheck.cuh"

namespace zkh {

// (op,oq)[y] = (cp[2y]*cq[2y+1] + cp[2y+1]*cq[2y], cq[2y]*cq[2y+1])   zkllm-src/p3_gkr.cuh:104-109
__global__ void __launch_bounds__(256)
gkr_comb_kernel(const gl_t* __restrict__ cp, const gl_t* __restrict__ cq, gl_t* __restrict__ op,
                gl_t* __restrict__ oq, size_t n) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        ulonglong2 p = ld2(cp + 2 * i), q = ld2(cq + 2 * i);
        Acc192 acc;
        acc.clear();
        acc.add_prod(p.x, q.y);
        acc.add_prod(p.y, q.x);
        op[i] = acc.reduce();
        oq[i] = gl_mul(q.x, q.y);
    }
}
// root pair -> pq[0..1]; a zero denominator raises the error flag (the reference throws)
__global__ void gkr_root_kernel(const gl_t* P, const gl_t* Q, gl_t* pq, ZkhCtl* ctl) {
    if (threadIdx.x == 0) {
        pq[0] = *P; pq[1] = *Q;
        if (*Q == 0) ctl->err = 1;
    }
}
// top layer: the two children of the root are published as they are
__global__ void gkr_top_kernel(const gl_t* cp, const gl_t* cq, gl_t* term) {
    if (threadIdx.x == 0) { term[0] = cp[0]; term[1] = cp[1]; term[2] = cq[0]; term[3] = cq[1]; }
}
// draw one field challenge from the device transcript into *dst
__global__ void tr_chal_kernel(ZkhCtl* ctl, gl_t* dst) {
    uint32_t st[8];
    for (int i = 0; i < 8; i++) st[i] = ctl->st[i];
    gl_t a = tr_warp_chal_gl(st);
    __syncwarp();
    if (threadIdx.x == 0) {
        *dst = a;
        for (int i = 0; i < 8; i++) ctl->st[i] = st[i];
    }
}

}  // namespace zkh

using namespace zkh;

static size_t gkr_proof_bytes(uint32_t L) {
    size_t s = 16;
    for (uint32_t h = L; h >= 1; h--) s += 4 + (size_t)(L - h) * 32 + 32;
    return s;
}
extern "C" size_t zkh_gkr_proof_size(uint32_t L) { return gkr_proof_bytes(L); }

extern "C" int zkh_gkr_prove(zkh_ctx* c, const uint64_t* p_dev, const uint64_t* q_dev, uint32_t L, int combine_last,
                             const char* tag, uint8_t state[32], uint64_t* rfin, uint64_t cpq[2], uint8_t* out,
                             size_t cap, size_t* written) {
    if (!c || !p_dev || !q_dev || !tag || !state || !rfin || !out || !written)
        return zkh_fail(c, ZKH_ERR_ARG, "gkr_prove: null pointer");
    if (L < 1 || L > 32) return zkh_fail(c, ZKH_ERR_ARG, "gkr_prove: need 1 <= L <= 32");
    if (strlen(tag) > ZKH_TR_MAX_LABEL) return zkh_fail(c, ZKH_ERR_LIMIT, "gkr_prove: tag longer than 48 bytes");
    const size_t need = gkr_proof_bytes(L);
    if (cap < need) return zkh_fail(c, ZKH_ERR_ARG, "gkr_prove: output buffer smaller than zkh_gkr_proof_size");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    const size_t N0 = (size_t)1 << L;

    // ---- workspace: levels 1..L of both trees, E column, sumcheck scratch, small result area ----
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off += zkh_align(bytes); return o; };
    const size_t o_lp = take(N0 * 8), o_lq = take(N0 * 8);  // sum_{h>=1} 2^(L-h) < 2^L
    const size_t o_E = take((N0 / 2) * 8);
    const size_t o_sc = take(sc_workspace_bytes(5, L - 1 ? L - 1 : 1));
    const size_t o_eq = take(eq_scratch_bytes(L));
    const size_t nmsg = (size_t)L * (L - 1) / 2;              // total rounds over all layers
    const size_t o_msgs = take((nmsg * 4 + 4) * 8);
    const size_t o_terms = take((size_t)L * 5 * 8);
    const size_t o_z = take((size_t)(L + 2) * 8);
    const size_t o_pq = take(16);
    const size_t res_bytes = off - o_msgs;
    ZKH_TRY(zkh_ws_reserve(c, off));
    char* ws = (char*)c->ws;
    auto lvl = [&](size_t base_off, const uint64_t* leaves, uint32_t h) -> const gl_t* {
        if (h == 0) return leaves;
        return (const gl_t*)(ws + base_off) + (N0 - (N0 >> (h - 1)));  // level h starts after levels 1..h-1
    };
    gl_t* E = (gl_t*)(ws + o_E);
    gl_t* d_msgs = (gl_t*)(ws + o_msgs);
    gl_t* d_terms = (gl_t*)(ws + o_terms);
    gl_t* d_z = (gl_t*)(ws + o_z);
    gl_t* d_pq = (gl_t*)(ws + o_pq);
    cudaStream_t s = c->stream;

    ZkhCtl* hc = c->h_ctl;
    digest_from_bytes(state, hc->st);
    hc->counter = 0;
    hc->err = 0;
    for (int i = 0; i < 8; i++) hc->par[i] = 0;
    ZKH_CUDA(c, cudaMemcpyAsync(c->d_ctl, hc, offsetof(ZkhCtl, local), cudaMemcpyHostToDevice, s));

    // ---- tree ----
    for (uint32_t h = 1; h <= L; h++) {
        size_t n = N0 >> h, blocks = (n + 255) / 256, capb = (size_t)c->sm_count * 8;
        gkr_comb_kernel<<<(unsigned)(blocks < capb ? blocks : capb), 256, 0, s>>>(
            lvl(o_lp, p_dev, h - 1), lvl(o_lq, q_dev, h - 1), (gl_t*)lvl(o_lp, p_dev, h), (gl_t*)lvl(o_lq, q_dev, h), n);
    }
    gkr_root_kernel<<<1, 32, 0, s>>>(lvl(o_lp, p_dev, L), lvl(o_lq, q_dev, L), d_pq, c->d_ctl);
    ZKH_CUDA(c, cudaGetLastError());
    ZKH_TRY(tr_absorb_enqueue(c, tag, d_pq, 2));

    // ---- layers ----
    const ZkhTag ztag = zkh_make_tag(tag);
    size_t moff = 0;
    for (uint32_t h = L; h >= 1; h--) {
        gl_t* term5 = d_terms + (size_t)(L - h) * 5;  // [E_final, p0, p1, q0, q1]
        const gl_t* cp = lvl(o_lp, p_dev, h - 1);
        const gl_t* cq = lvl(o_lq, q_dev, h - 1);
        const uint32_t nr = L - h;
        if (h == L) {
            gkr_top_kernel<<<1, 32, 0, s>>>(cp, cq, term5 + 1);
        } else {
            tr_chal_kernel<<<1, 32, 0, s>>>(c->d_ctl, &c->d_ctl->par[0]);   // lambda
            ZKH_TRY(eq_enqueue(c, d_z, nr, E, ws + o_eq, /*z_on_device=*/true));
            const gl_t* in[3] = {E, cp, cq};
            ScOut so{d_msgs + moff * 4, d_z + 1, term5};  // round challenges become z[1..] of the next layer
            ZKH_TRY(sc_enqueue(c, ZKH_F_GKR, 4, LD_GKR, in, nr, ztag, ws + o_sc, so));
            moff += nr;
        }
        ZKH_TRY(tr_absorb_enqueue(c, tag, term5 + 1, 4));
        if (h > 1 || combine_last) tr_chal_kernel<<<1, 32, 0, s>>>(c->d_ctl, d_z);  // mu = z[0] of the next layer
        ZKH_CUDA(c, cudaGetLastError());
    }
    // ---- one download: transcript state + results ----
    std::string hres(res_bytes, '\0');
    ZKH_CUDA(c, cudaMemcpyAsync(hc, c->d_ctl, offsetof(ZkhCtl, par), cudaMemcpyDeviceToHost, s));
    ZKH_CUDA(c, cudaMemcpyAsync(&hres[0], ws + o_msgs, res_bytes, cudaMemcpyDeviceToHost, s));
    ZKH_CUDA(c, cudaStreamSynchronize(s));
    if (hc->err) return zkh_fail(c, ZKH_ERR_DOMAIN, "gkr_prove: zero leaf denominator");
    const gl_t* hm = (const gl_t*)&hres[0];
    const gl_t* ht = (const gl_t*)(&hres[0] + (o_terms - o_msgs));
    const gl_t* hz = (const gl_t*)(&hres[0] + (o_z - o_msgs));
    const gl_t* hpq = (const gl_t*)(&hres[0] + (o_pq - o_msgs));
    uint8_t* p = out;
    memcpy(p, hpq, 16); p += 16;
    size_t mo = 0;
    for (uint32_t h = L; h >= 1; h--) {
        uint32_t nr = L - h;
        memcpy(p, &nr, 4); p += 4;
        memcpy(p, hm + mo * 4, (size_t)nr * 32); p += (size_t)nr * 32;
        mo += nr;
        memcpy(p, ht + (size_t)(L - h) * 5 + 1, 32); p += 32;
    }
    *written = (size_t)(p - out);
    const gl_t* last = ht + (size_t)(L - 1) * 5 + 1;
    if (combine_last) {
        memcpy(rfin, hz, (size_t)L * 8);
        if (cpq) {
            cpq[0] = gl_lerp(last[0], last[1], hz[0]);
            cpq[1] = gl_lerp(last[2], last[3], hz[0]);
        }
    } else {
        memcpy(rfin, hz + 1, (size_t)(L - 1) * 8);
        if (cpq) { cpq[0] = 0; cpq[1] = 0; }
    }
    digest_to_bytes(hc->st, state);
    return ZKH_OK;
}
