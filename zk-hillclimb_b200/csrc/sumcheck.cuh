// Internal interface of the sumcheck engine (shared by the sumcheck, GKR and
// Basefold translation units).
#pragma once
#include "common.cuh"

namespace zkh {

// how the nc logical columns are laid out in memory
enum { LD_PLAIN = 0,  // in[k] = column k
       LD_GKR = 1 };  // in[0] = E (n), in[1] = P (2n), in[2] = Q (2n) with children interleaved:
                      // A0[j]=P[2j] A1[j]=P[2j+1] B0[j]=Q[2j] B1[j]=Q[2j+1]
                      // (replaces the split copy of zkllm-src/p3_gkr.cuh:111-115)

struct ScPtrs {
    const gl_t* in[8];
    gl_t* out[8];
};

// where one sumcheck writes its public outputs (all device pointers)
struct ScOut {
    gl_t* msgs;    // rounds*nt
    gl_t* chals;   // rounds
    gl_t* finals;  // nc
};

// largest column length (after the pending bind) that the single-CTA tail handles
constexpr uint32_t SC_TAIL_LOG = 11;

int functor_nc(int functor);
size_t sc_workspace_bytes(int nc, uint32_t logn);

// Queue all rounds of one sumcheck on ctx->stream.  Nothing is read back.
//   in       source columns (layout ld), untouched
//   scratch  sc_workspace_bytes(nc, logn) bytes
//   out      device destinations
// The transcript state and parameters live in ctx->d_ctl.
int sc_enqueue(zkh_ctx* ctx, int functor, int nt, int ld, const gl_t* const* in, uint32_t logn,
               const ZkhTag& tag, void* scratch, const ScOut& out);


// One round on explicit plain-layout buffers; see sumcheck.cu.
int sc_enqueue_round(zkh_ctx* ctx, int functor, int nt, bool first, const gl_t* const* in, gl_t* const* out,
                     size_t n_in, const gl_t* chal_prev, gl_t* msg_out, gl_t* chal_out, const ZkhTag& tag,
                     int mode = 0);
int sc_enqueue_tail(zkh_ctx* ctx, int functor, int nt, const gl_t* const* in, uint32_t n, int nrounds, gl_t* msg_out,
                    gl_t* chal_out, gl_t* finals_out, const ZkhTag& tag, int pending = 0, const gl_t* chal_prev = nullptr,
                    int mode = 0, int resid = 0);
// Absorb nwords 64-bit words of device data under `tag` into the device transcript.
int tr_absorb_enqueue(zkh_ctx* ctx, const char* tag, const uint64_t* vals_dev, uint32_t nwords);

// ------------------------------------------------------------------ peer exchange
// All-gather of nv (<= 8) words per GPU through the peer mailboxes (ctl->xchg): publish this GPU's words into slot
// [seq & 1][rank] of every mailbox, system fence, publish the flag, wait (a bounded number of polls) until this GPU's own
// mailbox holds every rank's flag for this sequence number, then copy the G x nv words to all[g * 8 + t] (shared memory).
// A GPU whose device error flag is already set publishes its flag with the poison bit: the GPUs that read it set their own
// error flag too, so a wait that ran out on one GPU ends the proof with an error status on every GPU instead of leaving the
// others with sums that no longer match.  Called by all 32 lanes of one warp; mine[] must be visible to the warp.
// Returns G.
#define ZKH_XCHG_POISON (1ull << 63)
static __device__ __noinline__ uint32_t xchg_allgather(ZkhCtl* ctl, const gl_t* mine, int nv, gl_t* all) {
    ZkhXchg* x = static_cast<ZkhXchg*>(ctl->xchg);
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t G = x->G, me = x->rank;
    const unsigned long long seq = x->seq + 1;
    const int slot = (int)(seq & 1);
    const unsigned int err0 = ctl->err;
    __syncwarp();
    if (lane < (uint32_t)nv)
        for (uint32_t p = 0; p < G; p++)
            *reinterpret_cast<volatile gl_t*>(&x->mbox[p]->data[slot][me][lane]) = mine[lane];
    __threadfence_system();
    __syncwarp();
    if (lane < G)
        *reinterpret_cast<volatile unsigned long long*>(&x->mbox[lane]->flag[slot][me]) = seq | (err0 ? ZKH_XCHG_POISON : 0ull);
    bool ok = true;
    if (lane < G) {
        volatile unsigned long long* f = &x->mbox[me]->flag[slot][lane];
        const uint32_t limit = err0 ? 0u : (1u << 21);   // about a second, then give up with an error flag
        uint32_t it = 0;
        unsigned long long v = *f;
        while ((v & ~ZKH_XCHG_POISON) != seq && it < limit) { __nanosleep(128); it++; v = *f; }
        ok = (v == seq);                                 // arrived, and the sender had no error
    }
    ok = __all_sync(0xffffffffu, ok);
    __threadfence_system();
    for (uint32_t i = lane; i < G * (uint32_t)nv; i += 32) {
        const uint32_t g = i / (uint32_t)nv, t = i % (uint32_t)nv;
        all[g * 8 + t] = *reinterpret_cast<volatile gl_t*>(&x->mbox[me]->data[slot][g][t]);
    }
    if (lane == 0) {
        x->seq = seq;
        if (!ok) atomicOr(&ctl->err, 4u);
    }
    __syncwarp();
    return G;
}

// ------------------------------------------------------------------ round end
// mode 0: absorb the message under `tag` and draw the challenge on the device.
// mode 1: write this GPU's sums to msg_out and stop (another step combines the GPUs).
// mode 2: exchange the sums with the other GPUs through the peer mailboxes (ctl->xchg), add them in
//         rank order, then absorb and draw the challenge as in mode 0: the whole round is one kernel.
// Called by all 32 lanes of warp 0; the sums s are valid on lane 0.
template <int NT>
__device__ __noinline__ void finish_round(const gl_t (&s)[NT], ZkhCtl* ctl, gl_t* msg_out, gl_t* chal_out,
                                          const ZkhTag& tag, int mode) {
    __shared__ uint32_t trbuf[ZKH_TRBUF_WORDS];
    __shared__ gl_t mvals[NT];
    const uint32_t lane = threadIdx.x & 31;
    if (lane == 0) {
#pragma unroll
        for (int t = 0; t < NT; t++) { msg_out[t] = s[t]; mvals[t] = s[t]; }
    }
    if (mode == 1) return;
    if (mode == 2) {
        // sum over the GPUs through the peer mailboxes, in rank order
        __shared__ gl_t xall[ZKH_XCHG_MAXG * 8];
        __syncwarp();
        const uint32_t G = xchg_allgather(ctl, mvals, NT, xall);
        if (lane < NT) {
            gl_t a = 0;
            for (uint32_t g = 0; g < G; g++) a = gl_add(a, xall[g * 8 + lane]);
            mvals[lane] = a;
            msg_out[lane] = a;
        }
        __syncwarp();
    }
    // mode 3: structured Libra blind g(x) = sum_j g_j(x_j) of the hiding mode (zkllm-src/p3_hawkeye.cuh:1092-1110 sb_fix): the
    // message of round rd gains A_rd * (pref + g_rd(t)) + B_rd, and pref gains g_rd(a) once the challenge a is known.
    // Table at par[6]: word 0 = pref, then 8 words per round: the five coefficients of g_rd, A_rd, B_rd, unused.
    gl_t* fx = nullptr;
    const gl_t* fe = nullptr;
    if (mode == 3) {
        fx = reinterpret_cast<gl_t*>(ctl->par[6]);
        fe = fx + 8 + 8 * (size_t)((msg_out - ctl->msgs) / NT);
        if (lane < NT) {
            const gl_t t = (gl_t)lane;
            gl_t g = fe[4];
#pragma unroll
            for (int k = 3; k >= 0; k--) g = gl_add(gl_mul(g, t), fe[k]);
            const gl_t add = gl_add(gl_mul(fe[5], gl_add(fx[0], g)), fe[6]);
            mvals[lane] = gl_add(mvals[lane], add);
            msg_out[lane] = mvals[lane];
        }
        __syncwarp();
    }
    uint32_t st[8];
#pragma unroll
    for (int i = 0; i < 8; i++) st[i] = ctl->st[i];
    tr_warp_absorb(st, tag.s, tag.len, mvals, NT, trbuf);
    gl_t a = tr_warp_chal_gl(st);
    if (lane == 0) {
#pragma unroll
        for (int i = 0; i < 8; i++) ctl->st[i] = st[i];
        *chal_out = a;
        if (mode == 3) {
            gl_t g = fe[4];
#pragma unroll
            for (int k = 3; k >= 0; k--) g = gl_add(gl_mul(g, a), fe[k]);
            fx[0] = gl_add(fx[0], g);
        }
    }
}

// CTA sums -> grid sum by the last CTA to arrive -> finish_round.
template <int NT>
__device__ __forceinline__ void grid_finish(gl_t (&s)[NT], gl_t* sh, ZkhCtl* ctl, gl_t* partials,
                                            gl_t* msg_out, gl_t* chal_out, const ZkhTag& tag,
                                            int mode) {
    __shared__ int is_last;
    block_sum<NT>(s, sh);
    if (threadIdx.x == 0) {
#pragma unroll
        for (int t = 0; t < NT; t++) __stcg(&partials[(size_t)blockIdx.x * NT + t], s[t]);
        __threadfence();
        unsigned prev = atomicAdd(&ctl->counter, 1u);
        is_last = (prev == gridDim.x - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    gl_t v[NT];
#pragma unroll
    for (int t = 0; t < NT; t++) v[t] = 0;
    for (unsigned b = threadIdx.x; b < gridDim.x; b += blockDim.x) {
#pragma unroll
        for (int t = 0; t < NT; t++) v[t] = gl_add(v[t], __ldcg(&partials[(size_t)b * NT + t]));
    }
    block_sum<NT>(v, sh);
    if (threadIdx.x < 32) {
        if (threadIdx.x == 0) ctl->counter = 0;
        finish_round<NT>(v, ctl, msg_out, chal_out, tag, mode);
    }
}

}  // namespace zkh
