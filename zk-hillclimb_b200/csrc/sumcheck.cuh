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
                    gl_t* chal_out, gl_t* finals_out, const ZkhTag& tag);
// Absorb nwords 64-bit words of device data under `tag` into the device transcript.
int tr_absorb_enqueue(zkh_ctx* ctx, const char* tag, const uint64_t* vals_dev, uint32_t nwords);

}  // namespace zkh
