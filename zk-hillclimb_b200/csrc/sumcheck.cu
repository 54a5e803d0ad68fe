// Sumcheck prover rounds over Goldilocks for sm_100a.
//
// What the reference does per round (zkllm-src/p3_scgpu.cuh:107-156): a message
// kernel, a device-to-host copy of 256 partials per evaluation point, a host sum,
// a host SHA-256 absorb/challenge, nc device allocations and a bind kernel.
//
// What happens here per round: ONE kernel.  It binds the previous round's columns
// with the previous challenge (read from device memory), writes the halved
// columns, and accumulates this round's message from the values it just
// produced, all from 128-bit loads of adjacent pairs.  Partial sums are reduced
// with warp shuffles, then across CTAs by the last CTA to finish, which also runs
// the Fiat-Shamir absorb and derives the next challenge on the device.  The host
// queues every round up front and reads results back once.
//
// Sums are exact field sums, so any partition and any order give the same
// canonical values as the reference's accumulation.
#include "sumcheck.cuh"

namespace zkh {

// ------------------------------------------------------------------ summands
// Each summand F has degree DEG (2 or 3) in the round variable.  Its round polynomial is fixed
// by DEG+1 numbers; the kernels accumulate F at t = 0 .. DEG-1 and the leading coefficient
// (F's top-degree part applied to the pair differences), which needs no stepped operands, and
// derive the evaluations at t = DEG .. NT-1 by finite differences afterwards.  All of it is
// exact field arithmetic, so the message equals the reference's t = 0..NT-1 sums.
template <int F> struct Fn;
template <> struct Fn<ZKH_F_PROD2> {
    static constexpr int NC = 2, DEG = 2;
    static __device__ __forceinline__ void acc(Acc192& a, const gl_t* c, const gl_t*) {
        a.add_prod(c[0], c[1]);
    }
    static __device__ __forceinline__ void lead(Acc192& a, const gl_t* d, const gl_t*) {
        a.add_prod(d[0], d[1]);
    }
};
template <> struct Fn<ZKH_F_PROD3> {
    static constexpr int NC = 3, DEG = 3;
    static __device__ __forceinline__ void acc(Acc192& a, const gl_t* c, const gl_t*) {
        a.add_prod(c[0], gl_mul(c[1], c[2]));
    }
    static __device__ __forceinline__ void lead(Acc192& a, const gl_t* d, const gl_t*) {
        a.add_prod(d[0], gl_mul(d[1], d[2]));
    }
};
template <> struct Fn<ZKH_F_GKR> {
    static constexpr int NC = 5, DEG = 3;
    static __device__ __forceinline__ void acc(Acc192& a, const gl_t* c, const gl_t* p) {
        Acc192 in;
        in.clear();
        in.add_prod(c[1], c[4]);
        in.add_prod(c[2], c[3]);
        in.add_prod(p[0], gl_mul(c[3], c[4]));
        a.add_prod(c[0], in.reduce());
    }
    static __device__ __forceinline__ void lead(Acc192& a, const gl_t* d, const gl_t* p) { acc(a, d, p); }
};
template <> struct Fn<ZKH_F_LOGUP> {
    static constexpr int NC = 4, DEG = 3;
    static __device__ __forceinline__ void acc(Acc192& a, const gl_t* c, const gl_t* p) {
        a.add_prod(p[0], c[0]);
        a.add_prod(c[2], gl_sub(gl_mul(c[0], gl_add(c[1], p[1])), c[3]));
    }
    // the only cubic term of  p0*H + E*(H*(V+p1) - D)  is E*H*V
    static __device__ __forceinline__ void lead(Acc192& a, const gl_t* d, const gl_t*) {
        a.add_prod(d[2], gl_mul(d[0], d[1]));
    }
};

// rescale zero-check (zkllm-src/p3_int_gadgets.cuh:316-325):
//   E * (X + H - Y*2^sf - L0 [- 2^16*L1]),  par = [H, 2^sf]
template <int NL> struct FnIrs {
    static constexpr int NC = 3 + NL, DEG = 2;
    static __device__ __forceinline__ gl_t inner(const gl_t* c, const gl_t* p, gl_t h) {
        gl_t t = gl_sub(gl_add(c[1], h), gl_mul(c[2], p[1]));
        t = gl_sub(t, c[3]);
        if (NL == 2) t = gl_sub(t, gl_mul(c[4], 65536ULL));
        return t;
    }
    static __device__ __forceinline__ void acc(Acc192& a, const gl_t* c, const gl_t* p) {
        a.add_prod(c[0], inner(c, p, p[0]));
    }
    static __device__ __forceinline__ void lead(Acc192& a, const gl_t* d, const gl_t* p) {
        a.add_prod(d[0], inner(d, p, 0));   // the constant H has no part in the top coefficient
    }
};
template <> struct Fn<ZKH_F_IRS1> : FnIrs<1> {};
template <> struct Fn<ZKH_F_IRS2> : FnIrs<2> {};

int functor_nc(int functor) {
    switch (functor) {
        case ZKH_F_IRS1: return 4;
        case ZKH_F_IRS2: return 5;
        case ZKH_F_PROD2: return 2;
        case ZKH_F_PROD3: return 3;
        case ZKH_F_GKR: return 5;
        case ZKH_F_LOGUP: return 4;
    }
    return -1;
}

// ------------------------------------------------------------------ loaders
template <int LD, int NC>
__device__ __forceinline__ void load_pairs(const ScPtrs& P, size_t i, gl_t (&lo)[NC], gl_t (&hi)[NC]) {
    if (LD == LD_PLAIN) {
#pragma unroll
        for (int k = 0; k < NC; k++) {
            ulonglong2 v = ld2(P.in[k] + 2 * i);
            lo[k] = v.x; hi[k] = v.y;
        }
    } else {
        ulonglong2 e = ld2(P.in[0] + 2 * i);
        lo[0] = e.x; hi[0] = e.y;
#pragma unroll
        for (int s = 0; s < 2; s++) {
            ulonglong2 a = ld2(P.in[1 + s] + 4 * i), b = ld2(P.in[1 + s] + 4 * i + 2);
            lo[1 + 2 * s] = a.x; hi[1 + 2 * s] = b.x;  // even child
            lo[2 + 2 * s] = a.y; hi[2 + 2 * s] = b.y;  // odd child
        }
    }
}
template <int LD, int NC>
__device__ __forceinline__ void load_quads(const ScPtrs& P, size_t i, gl_t (&x)[NC][4]) {
    if (LD == LD_PLAIN) {
#pragma unroll
        for (int k = 0; k < NC; k++) {
            ulonglong2 a = ld2(P.in[k] + 4 * i), b = ld2(P.in[k] + 4 * i + 2);
            x[k][0] = a.x; x[k][1] = a.y; x[k][2] = b.x; x[k][3] = b.y;
        }
    } else {
        ulonglong2 a = ld2(P.in[0] + 4 * i), b = ld2(P.in[0] + 4 * i + 2);
        x[0][0] = a.x; x[0][1] = a.y; x[0][2] = b.x; x[0][3] = b.y;
#pragma unroll
        for (int s = 0; s < 2; s++) {
            const gl_t* src = P.in[1 + s] + 8 * i;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                ulonglong2 v = ld2(src + 2 * j);
                x[1 + 2 * s][j] = v.x;
                x[2 + 2 * s][j] = v.y;
            }
        }
    }
}

// message contribution of one pair per column (zkllm-src/p3_scgpu.cuh:63-72 computes
// F(lo + t*(hi-lo)) for every t; see the note above Fn for what is accumulated instead).
// acc[t], t < DEG: F at t;  acc[DEG]: leading coefficient;  acc[t > DEG]: unused.
template <int F, int NT>
__device__ __forceinline__ void msg_accum(Acc192 (&acc)[NT], const gl_t (&lo)[Fn<F>::NC],
                                          const gl_t (&hi)[Fn<F>::NC], const gl_t* par) {
    constexpr int NC = Fn<F>::NC, DEG = Fn<F>::DEG;
    static_assert(NT > DEG, "message must carry at least DEG+1 evaluations");
    gl_t dd[NC];
    Fn<F>::acc(acc[0], lo, par);
    Fn<F>::acc(acc[1], hi, par);
#pragma unroll
    for (int k = 0; k < NC; k++) dd[k] = gl_sub(hi[k], lo[k]);
    Fn<F>::lead(acc[DEG], dd, par);
    if (DEG == 3) {
        gl_t cur[NC];
#pragma unroll
        for (int k = 0; k < NC; k++) cur[k] = gl_add(hi[k], dd[k]);
        Fn<F>::acc(acc[2], cur, par);
    }
}
// per-thread: reduce the lazy sums and turn (F(0..DEG-1), lead) into evaluations at t = 0..NT-1.
// Linear in the accumulated quantities, so it commutes with the later summation over threads.
template <int F, int NT>
__device__ __forceinline__ void msg_reduce(const Acc192 (&acc)[NT], gl_t (&s)[NT]) {
    constexpr int DEG = Fn<F>::DEG;
#pragma unroll
    for (int t = 0; t <= DEG; t++) s[t] = acc[t].reduce();
    if (DEG == 2) {
        // g(2) = 2 g(1) - g(0) + 2 c2 ; third difference vanishes afterwards
        gl_t c2 = s[2];
        s[2] = gl_add(gl_sub(gl_dbl(s[1]), s[0]), gl_dbl(c2));
#pragma unroll
        for (int t = 3; t < NT; t++)
            s[t] = gl_add(gl_mul(3, gl_sub(s[t - 1], s[t - 2])), s[t - 3]);
    } else {
        // g(3) = 3 g(2) - 3 g(1) + g(0) + 6 c3 ; fourth difference vanishes afterwards
        gl_t c3 = s[3];
        s[3] = gl_add(gl_add(gl_mul(3, gl_sub(s[2], s[1])), s[0]), gl_mul(6, c3));
#pragma unroll
        for (int t = 4; t < NT; t++)
            s[t] = gl_sub(gl_add(gl_mul(4, gl_add(s[t - 1], s[t - 3])), 0), gl_add(gl_mul(6, s[t - 2]), s[t - 4]));
    }
}

// ------------------------------------------------------------------ kernels
// round 0: message only
template <int F, int NT, int LD>
__global__ void __launch_bounds__(256)
sc_first_kernel(ScPtrs P, size_t half, ZkhCtl* ctl, gl_t* partials, gl_t* msg_out, gl_t* chal_out,
                ZkhTag tag, int mode) {
    constexpr int NC = Fn<F>::NC;
    __shared__ gl_t sh[NT * 32];
    gl_t par[2] = {ctl->par[0], ctl->par[1]};
    Acc192 acc[NT];
#pragma unroll
    for (int t = 0; t < NT; t++) acc[t].clear();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < half; i += stride) {
        gl_t lo[NC], hi[NC];
        load_pairs<LD, NC>(P, i, lo, hi);
        msg_accum<F, NT>(acc, lo, hi, par);
    }
    gl_t s[NT];
    msg_reduce<F, NT>(acc, s);
    grid_finish<NT>(s, sh, ctl, partials, msg_out, chal_out, tag, mode);
}

// round r >= 1: bind with challenge r-1, store the halved columns, message of round r
template <int F, int NT, int LD>
__global__ void __launch_bounds__(256)
sc_fused_kernel(ScPtrs P, size_t quads, ZkhCtl* ctl, gl_t* partials, const gl_t* chal_prev,
                gl_t* msg_out, gl_t* chal_out, ZkhTag tag, int mode) {
    constexpr int NC = Fn<F>::NC;
    __shared__ gl_t sh[NT * 32];
    gl_t par[2] = {ctl->par[0], ctl->par[1]};
    const gl_t a = *chal_prev;
    Acc192 acc[NT];
#pragma unroll
    for (int t = 0; t < NT; t++) acc[t].clear();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < quads; i += stride) {
        gl_t x[NC][4], lo[NC], hi[NC];
        load_quads<LD, NC>(P, i, x);
#pragma unroll
        for (int k = 0; k < NC; k++) {
            lo[k] = gl_lerp(x[k][0], x[k][1], a);
            hi[k] = gl_lerp(x[k][2], x[k][3], a);
            st2(P.out[k] + 2 * i, lo[k], hi[k]);
        }
        msg_accum<F, NT>(acc, lo, hi, par);
    }
    gl_t s[NT];
    msg_reduce<F, NT>(acc, s);
    grid_finish<NT>(s, sh, ctl, partials, msg_out, chal_out, tag, mode);
}

// all remaining rounds of a small instance in one CTA, columns in shared memory.
// n_in: source column length; pending: bind the source with *chal_prev while loading.
// Column length in shared memory is at most 2*blockDim.x.
// resid > 0 (sharded proofs, mode 2): after the nrounds local rounds the GPUs all-gather their nc bound values through
// the peer mailboxes (one more exchange) and every GPU runs the last `resid` = log2(G) rounds on the G-element columns
// here, without further exchanges: the proof ends in this launch.
template <int F, int NT, int LD>
__global__ void __launch_bounds__(1024)
sc_tail_kernel(ScPtrs P, uint32_t n_in, int pending, ZkhCtl* ctl, const gl_t* chal_prev,
               gl_t* msg_out, gl_t* chal_out, gl_t* finals_out, int nrounds, ZkhTag tag, int mode = 0, int resid = 0) {
    constexpr int NC = Fn<F>::NC;
    extern __shared__ gl_t cols[];
    __shared__ gl_t sh[NT * 32];
    __shared__ gl_t sh_chal;
    const uint32_t tid = threadIdx.x;
    uint32_t n0 = pending ? n_in / 2 : n_in;
    gl_t par[2] = {ctl->par[0], ctl->par[1]};
    if (pending) {
        const gl_t a = *chal_prev;
        for (uint32_t j = tid; j < n0; j += blockDim.x) {
            gl_t lo[NC], hi[NC];
            load_pairs<LD, NC>(P, j, lo, hi);
#pragma unroll
            for (int k = 0; k < NC; k++) cols[k * n0 + j] = gl_lerp(lo[k], hi[k], a);
        }
    } else {
        for (uint32_t j = tid; j < n0 / 2; j += blockDim.x) {
            gl_t lo[NC], hi[NC];
            load_pairs<LD, NC>(P, j, lo, hi);
#pragma unroll
            for (int k = 0; k < NC; k++) { cols[k * n0 + 2 * j] = lo[k]; cols[k * n0 + 2 * j + 1] = hi[k]; }
        }
    }
    __syncthreads();
    for (int phase = 0; phase < 2; phase++) {
        uint32_t n = n0;
        for (int r = 0; r < nrounds; r++) {
            const uint32_t half = n / 2;
            Acc192 acc[NT];
#pragma unroll
            for (int t = 0; t < NT; t++) acc[t].clear();
            gl_t lo[NC], hi[NC];
            const bool active = tid < half;  // half <= blockDim.x
            if (active) {
#pragma unroll
                for (int k = 0; k < NC; k++) { lo[k] = cols[k * n0 + 2 * tid]; hi[k] = cols[k * n0 + 2 * tid + 1]; }
                msg_accum<F, NT>(acc, lo, hi, par);
            }
            gl_t s[NT];
            msg_reduce<F, NT>(acc, s);
            block_sum<NT>(s, sh);  // ends with a barrier: every pair has been read
            if (tid < 32) {
                finish_round<NT>(s, ctl, msg_out + (size_t)r * NT, chal_out + r, tag, mode);
                if (tid == 0) sh_chal = chal_out[r];
            }
            __syncthreads();
            const gl_t a = sh_chal;
            if (active) {
#pragma unroll
                for (int k = 0; k < NC; k++) cols[k * n0 + tid] = gl_lerp(lo[k], hi[k], a);
            }
            __syncthreads();
            n = half;
        }
        if (phase == 1 || resid == 0) break;
        // every GPU's bound values -> G-element columns, column k at cols[k * G ..]; the remaining rounds are local
        __shared__ gl_t xmine[8];
        __shared__ gl_t xall[ZKH_XCHG_MAXG * 8];
        __shared__ uint32_t xG;
        if (tid < NC) { xmine[tid] = cols[tid * n0]; if (finals_out) finals_out[tid] = xmine[tid]; }
        __syncthreads();
        if (tid < 32) {
            const uint32_t G = xchg_allgather(ctl, xmine, NC, xall);
            if (tid == 0) xG = G;
        }
        __syncthreads();
        const uint32_t G = xG;
        if (tid < NC * G) cols[(tid / G) * G + (tid % G)] = xall[(tid % G) * 8 + tid / G];
        __syncthreads();
        msg_out += (size_t)nrounds * NT;
        chal_out += nrounds;
        n0 = G;
        nrounds = resid;
        mode = 0;
        finals_out = ctl->finals;
    }
    if (tid < NC && finals_out) finals_out[tid] = cols[tid * n0];
}

// ------------------------------------------------------------------ host side
size_t sc_workspace_bytes(int nc, uint32_t logn) {
    if (logn <= SC_TAIL_LOG) return 256;
    size_t n = (size_t)1 << logn;
    return zkh_align((size_t)nc * (n / 2) * 8) + zkh_align((size_t)nc * (n / 4) * 8) + 256;
}

template <int F, int NT, int LD>
static int sc_enqueue_t(zkh_ctx* ctx, const gl_t* const* in, uint32_t logn, const ZkhTag& tag,
                        void* scratch, const ScOut& out) {
    constexpr int NC = Fn<F>::NC;
    const int nsrc = LD == LD_GKR ? 3 : NC;
    cudaStream_t s = ctx->stream;
    ZkhCtl* ctl = ctx->d_ctl;
    const size_t n = (size_t)1 << logn;
    ctx->prof_valid = false;
    ScPtrs P;
    memset(&P, 0, sizeof P);
    for (int k = 0; k < nsrc; k++) P.in[k] = in[k];

    struct Occ { int first, fused, fused_plain; };
    static const Occ occ = [] {                          // initialised once, by one thread (others wait)
        Occ o{0, 0, 0};
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&o.first, sc_first_kernel<F, NT, LD>, 256, 0);
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&o.fused, sc_fused_kernel<F, NT, LD>, 256, 0);
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&o.fused_plain, sc_fused_kernel<F, NT, LD_PLAIN>, 256, 0);
        if (o.first < 1) o.first = 1;
        if (o.fused < 1) o.fused = 1;
        if (o.fused_plain < 1) o.fused_plain = 1;
        return o;
    }();
    const int occ_first = occ.first, occ_fused = occ.fused, occ_fused_plain = occ.fused_plain;
    static ZkhOncePerDevice attr_set;                    // per device: the limit is a property of the device's function
    zkh_once_on_device(attr_set, ctx->device, [] {
        cudaFuncSetAttribute(sc_tail_kernel<F, NT, LD>, cudaFuncAttributeMaxDynamicSharedMemorySize, NC * (1 << SC_TAIL_LOG) * 8);
        cudaFuncSetAttribute(sc_tail_kernel<F, NT, LD_PLAIN>, cudaFuncAttributeMaxDynamicSharedMemorySize, NC * (1 << SC_TAIL_LOG) * 8);
    });
    auto grid_for = [&](size_t items, int occ) {
        size_t want = (items + 255) / 256, cap = (size_t)ctx->sm_count * occ;
        if (cap > ctx->partials_cap / 5) cap = ctx->partials_cap / 5;
        return (unsigned)(want < cap ? want : cap);
    };

    if (logn <= SC_TAIL_LOG) {
        sc_tail_kernel<F, NT, LD><<<1, 1024, NC * n * 8, s>>>(P, (uint32_t)n, 0, ctl, nullptr, out.msgs,
                                                              out.chals, out.finals, (int)logn, tag);
        return cudaGetLastError() == cudaSuccess ? ZKH_OK : zkh_fail(ctx, ZKH_ERR_CUDA, "sc_tail launch");
    }
    // round 0 on the caller's columns
    sc_first_kernel<F, NT, LD><<<grid_for(n / 2, occ_first), 256, 0, s>>>(
        P, n / 2, ctl, ctx->d_partials, out.msgs, out.chals, tag, 0);
    // ping-pong buffers for the bound columns
    gl_t* bufA = (gl_t*)scratch;
    gl_t* bufB = (gl_t*)((char*)scratch + zkh_align((size_t)NC * (n / 2) * 8));
    size_t cur_n = n;  // length of the columns the next kernel reads
    int r = 1;
    bool src_is_input = true;
    const gl_t* cur_in[8];
    for (int k = 0; k < nsrc; k++) cur_in[k] = in[k];
    gl_t* dst = bufA;
    while ((cur_n >> 1) > ((size_t)1 << SC_TAIL_LOG)) {
        const size_t out_n = cur_n / 2;
        for (int k = 0; k < 8; k++) { P.in[k] = nullptr; P.out[k] = nullptr; }
        for (int k = 0; k < (src_is_input ? nsrc : NC); k++) P.in[k] = cur_in[k];
        for (int k = 0; k < NC; k++) P.out[k] = dst + (size_t)k * out_n;
        const bool prof = (r == 1) && ctx->prof_ev[0];
        if (prof) cudaEventRecord(ctx->prof_ev[0], s);
        if (src_is_input)
            sc_fused_kernel<F, NT, LD><<<grid_for(cur_n / 4, occ_fused), 256, 0, s>>>(
                P, cur_n / 4, ctl, ctx->d_partials, out.chals + (r - 1), out.msgs + (size_t)r * NT,
                out.chals + r, tag, 0);
        else
            sc_fused_kernel<F, NT, LD_PLAIN><<<grid_for(cur_n / 4, occ_fused_plain), 256, 0, s>>>(
                P, cur_n / 4, ctl, ctx->d_partials, out.chals + (r - 1), out.msgs + (size_t)r * NT,
                out.chals + r, tag, 0);
        if (prof) {
            cudaEventRecord(ctx->prof_ev[1], s);
            ctx->prof_valid = true;
            ctx->prof_bytes = (uint64_t)12 * NC * cur_n;  // read 8, write 4 bytes per input element
            ctx->prof_kernel = "sc_fused_kernel";
        }
        for (int k = 0; k < NC; k++) cur_in[k] = P.out[k];
        src_is_input = false;
        dst = (dst == bufA) ? bufB : bufA;
        cur_n = out_n;
        r++;
    }
    for (int k = 0; k < 8; k++) { P.in[k] = nullptr; P.out[k] = nullptr; }
    for (int k = 0; k < (src_is_input ? nsrc : NC); k++) P.in[k] = cur_in[k];
    const size_t tail_n = cur_n / 2;
    if (src_is_input)
        sc_tail_kernel<F, NT, LD><<<1, 1024, NC * tail_n * 8, s>>>(
            P, (uint32_t)cur_n, 1, ctl, out.chals + (r - 1), out.msgs + (size_t)r * NT, out.chals + r,
            out.finals, (int)logn - r, tag);
    else
        sc_tail_kernel<F, NT, LD_PLAIN><<<1, 1024, NC * tail_n * 8, s>>>(
            P, (uint32_t)cur_n, 1, ctl, out.chals + (r - 1), out.msgs + (size_t)r * NT, out.chals + r,
            out.finals, (int)logn - r, tag);
    return cudaGetLastError() == cudaSuccess ? ZKH_OK : zkh_fail(ctx, ZKH_ERR_CUDA, "sumcheck launch");
}

// One round on explicit buffers (plain column layout).  first: message over `in` (n_in elements
// per column); otherwise bind `in` with *chal_prev into `out` (n_in/2 elements) and take the
// message of the bound columns.  n_in >= 2 (first) or >= 4 (fused).
template <int F, int NT>
static int sc_round_t(zkh_ctx* ctx, bool first, const gl_t* const* in, gl_t* const* out, size_t n_in,
                      const gl_t* chal_prev, gl_t* msg_out, gl_t* chal_out, const ZkhTag& tag, int mode) {
    constexpr int NC = Fn<F>::NC;
    ScPtrs P;
    memset(&P, 0, sizeof P);
    for (int k = 0; k < NC; k++) { P.in[k] = in[k]; P.out[k] = out ? out[k] : nullptr; }
    const size_t items = first ? n_in / 2 : n_in / 4;
    size_t want = (items + 255) / 256, cap = (size_t)ctx->sm_count * 4;
    if (cap > ctx->partials_cap / 5) cap = ctx->partials_cap / 5;
    unsigned grid = (unsigned)(want < cap ? want : cap);
    if (first)
        sc_first_kernel<F, NT, LD_PLAIN><<<grid, 256, 0, ctx->stream>>>(P, items, ctx->d_ctl, ctx->d_partials,
                                                                        msg_out, chal_out, tag, mode);
    else
        sc_fused_kernel<F, NT, LD_PLAIN><<<grid, 256, 0, ctx->stream>>>(P, items, ctx->d_ctl, ctx->d_partials,
                                                                        chal_prev, msg_out, chal_out, tag, mode);
    return cudaGetLastError() == cudaSuccess ? ZKH_OK : zkh_fail(ctx, ZKH_ERR_CUDA, "sumcheck round launch");
}
int sc_enqueue_round(zkh_ctx* ctx, int functor, int nt, bool first, const gl_t* const* in, gl_t* const* out,
                     size_t n_in, const gl_t* chal_prev, gl_t* msg_out, gl_t* chal_out, const ZkhTag& tag, int mode) {
#define CASE(F, NT) \
    if (functor == F && nt == NT) return sc_round_t<F, NT>(ctx, first, in, out, n_in, chal_prev, msg_out, chal_out, tag, mode);
    CASE(ZKH_F_PROD2, 3)
    CASE(ZKH_F_PROD2, 5)
    CASE(ZKH_F_PROD3, 4)
    CASE(ZKH_F_PROD3, 5)
    CASE(ZKH_F_GKR, 4)
    CASE(ZKH_F_LOGUP, 4)
    CASE(ZKH_F_IRS1, 5)
    CASE(ZKH_F_IRS2, 5)
#undef CASE
    return zkh_fail(ctx, ZKH_ERR_ARG, "sumcheck round: unsupported (functor, nt) combination");
}

// tail on explicit plain columns: nrounds rounds in one CTA.  pending == 0: columns of length n (<= 2^11);
// pending == 1: columns of length n (<= 2^12) still to be bound with *chal_prev first.
template <int F, int NT>
static int sc_tail_t(zkh_ctx* ctx, const gl_t* const* in, uint32_t n, int nrounds, gl_t* msg_out, gl_t* chal_out,
                     gl_t* finals_out, const ZkhTag& tag, int pending, const gl_t* chal_prev, int mode, int resid) {
    constexpr int NC = Fn<F>::NC;
    ScPtrs P;
    memset(&P, 0, sizeof P);
    for (int k = 0; k < NC; k++) P.in[k] = in[k];
    static ZkhOncePerDevice attr;
    zkh_once_on_device(attr, ctx->device, [] {
        cudaFuncSetAttribute(sc_tail_kernel<F, NT, LD_PLAIN>, cudaFuncAttributeMaxDynamicSharedMemorySize, NC * (1 << SC_TAIL_LOG) * 8);
    });
    size_t held = pending ? n / 2 : n;
    if (resid > 0 && held < ((size_t)1 << resid)) held = (size_t)1 << resid;   // room for the G-element residual columns
    sc_tail_kernel<F, NT, LD_PLAIN><<<1, 1024, (size_t)NC * held * 8, ctx->stream>>>(P, n, pending, ctx->d_ctl, chal_prev,
                                                                                msg_out, chal_out, finals_out, nrounds, tag,
                                                                                mode, resid);
    return cudaGetLastError() == cudaSuccess ? ZKH_OK : zkh_fail(ctx, ZKH_ERR_CUDA, "sumcheck tail launch");
}
int sc_enqueue_tail(zkh_ctx* ctx, int functor, int nt, const gl_t* const* in, uint32_t n, int nrounds, gl_t* msg_out,
                    gl_t* chal_out, gl_t* finals_out, const ZkhTag& tag, int pending, const gl_t* chal_prev, int mode,
                    int resid) {
#define CASE(F, NT) \
    if (functor == F && nt == NT) \
        return sc_tail_t<F, NT>(ctx, in, n, nrounds, msg_out, chal_out, finals_out, tag, pending, chal_prev, mode, resid);
    CASE(ZKH_F_PROD2, 3)
    CASE(ZKH_F_PROD2, 5)
    CASE(ZKH_F_PROD3, 4)
    CASE(ZKH_F_PROD3, 5)
    CASE(ZKH_F_GKR, 4)
    CASE(ZKH_F_LOGUP, 4)
    CASE(ZKH_F_IRS1, 5)
    CASE(ZKH_F_IRS2, 5)
#undef CASE
    return zkh_fail(ctx, ZKH_ERR_ARG, "sumcheck tail: unsupported (functor, nt) combination");
}

// sum the G ranks' round sums (rank-major [G][nt]), absorb, draw the challenge: the step every
// rank of a sharded sumcheck runs identically after the all-gather
__global__ void sc_combine_kernel(ZkhCtl* ctl, const gl_t* gathered, uint32_t G, int nt, ZkhTag tag, gl_t* msg_out,
                                  gl_t* chal_out) {
    __shared__ uint32_t buf[ZKH_TRBUF_WORDS];
    __shared__ gl_t m[5];
    if (threadIdx.x < (unsigned)nt) {
        gl_t a = 0;
        for (uint32_t g = 0; g < G; g++) a = gl_add(a, gathered[(size_t)g * nt + threadIdx.x]);
        m[threadIdx.x] = a;
        msg_out[threadIdx.x] = a;
    }
    uint32_t st[8];
    for (int i = 0; i < 8; i++) st[i] = ctl->st[i];
    tr_warp_absorb(st, tag.s, tag.len, m, nt, buf);
    gl_t a = tr_warp_chal_gl(st);
    if (threadIdx.x == 0) {
        *chal_out = a;
        for (int i = 0; i < 8; i++) ctl->st[i] = st[i];
    }
}
// out[k] = in[k][0] + a*(in[k][1]-in[k][0]): the last local bind of a sharded sumcheck
__global__ void sc_finals_kernel(ScPtrs P, int nc, const gl_t* chal, gl_t* out) {
    int k = threadIdx.x;
    if (k < nc) out[k] = gl_lerp(P.in[k][0], P.in[k][1], *chal);
}
// rank-major [G][nc] -> column-major [nc][G]
__global__ void sc_transpose_kernel(const gl_t* in, gl_t* out, uint32_t G, int nc) {
    uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t < G * nc) { uint32_t g = t / nc, k = t % nc; out[(size_t)k * G + g] = in[t]; }
}

// st = absorb(st, tag, vals[0..n)) on the device transcript (n 64-bit words of raw bytes)
__global__ void tr_absorb_kernel(ZkhCtl* ctl, ZkhTag tag, const uint64_t* vals, uint32_t n) {
    __shared__ uint32_t buf[ZKH_TRBUF_WORDS];
    uint32_t st[8];
    for (int i = 0; i < 8; i++) st[i] = ctl->st[i];
    tr_warp_absorb(st, tag.s, tag.len, vals, n, buf);
    if (threadIdx.x == 0)
        for (int i = 0; i < 8; i++) ctl->st[i] = st[i];
}
int tr_absorb_enqueue(zkh_ctx* ctx, const char* tag, const uint64_t* vals_dev, uint32_t nwords) {
    if (nwords * 8 > ZKH_TR_MAX_DATA) return zkh_fail(ctx, ZKH_ERR_LIMIT, "device absorb: more than 320 bytes");
    tr_absorb_kernel<<<1, 32, 0, ctx->stream>>>(ctx->d_ctl, zkh_make_tag(tag), vals_dev, nwords);
    return cudaGetLastError() == cudaSuccess ? ZKH_OK : zkh_fail(ctx, ZKH_ERR_CUDA, "absorb launch");
}

int sc_enqueue(zkh_ctx* ctx, int functor, int nt, int ld, const gl_t* const* in, uint32_t logn,
               const ZkhTag& tag, void* scratch, const ScOut& out) {
    if (logn < 1 || logn > 34) return zkh_fail(ctx, ZKH_ERR_ARG, "sumcheck: logn out of range");
#define CASE(F, NT, LD) \
    if (functor == F && nt == NT && ld == LD) return sc_enqueue_t<F, NT, LD>(ctx, in, logn, tag, scratch, out);
    CASE(ZKH_F_PROD2, 3, LD_PLAIN)
    CASE(ZKH_F_PROD2, 5, LD_PLAIN)
    CASE(ZKH_F_PROD3, 4, LD_PLAIN)
    CASE(ZKH_F_PROD3, 5, LD_PLAIN)
    CASE(ZKH_F_GKR, 4, LD_PLAIN)
    CASE(ZKH_F_GKR, 4, LD_GKR)
    CASE(ZKH_F_LOGUP, 4, LD_PLAIN)
    CASE(ZKH_F_IRS1, 5, LD_PLAIN)
    CASE(ZKH_F_IRS2, 5, LD_PLAIN)
#undef CASE
    return zkh_fail(ctx, ZKH_ERR_ARG, "sumcheck: unsupported (functor, nt) combination");
}

}  // namespace zkh

using namespace zkh;

// ------------------------------------------------------------------ C ABI
extern "C" size_t zkh_sumcheck_workspace(int nc, uint32_t logn) { return sc_workspace_bytes(nc, logn); }

static int sumcheck_common(zkh_ctx* ctx, int functor, int nt, const uint64_t* const* cols_dev, int nc,
                           uint32_t logn, const uint64_t* par, int npar, const char* tag,
                           uint8_t state[32], uint64_t* msgs, uint64_t* chals, uint64_t* finals,
                           void* scratch) {
    ZkhCtl* h = ctx->h_ctl;
    digest_from_bytes(state, h->st);
    h->counter = 0;
    h->err = 0;
    for (int i = 0; i < 8; i++) h->par[i] = i < npar ? par[i] : 0;
    ZKH_CUDA(ctx, cudaMemcpyAsync(ctx->d_ctl, h, offsetof(ZkhCtl, local), cudaMemcpyHostToDevice,
                                  ctx->stream));
    ScOut out{ctx->d_ctl->msgs, ctx->d_ctl->chals, ctx->d_ctl->finals};
    ZKH_TRY(sc_enqueue(ctx, functor, nt, LD_PLAIN, cols_dev, logn, zkh_make_tag(tag), scratch, out));
    ZKH_CUDA(ctx, cudaMemcpyAsync(h, ctx->d_ctl, sizeof(ZkhCtl), cudaMemcpyDeviceToHost, ctx->stream));
    ZKH_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (h->err) return zkh_fail(ctx, ZKH_ERR_DEVICE, "sumcheck: device error flag set");
    memcpy(msgs, h->msgs, (size_t)logn * nt * 8);
    memcpy(chals, h->chals, (size_t)logn * 8);
    if (finals) memcpy(finals, h->finals, (size_t)nc * 8);
    digest_to_bytes(h->st, state);
    return ZKH_OK;
}

static int sumcheck_check(zkh_ctx* ctx, int functor, int nt, const void* cols, int nc, uint32_t logn,
                          const uint64_t* par, int npar, const char* tag, const void* state,
                          const void* msgs, const void* chals) {
    if (!ctx) return ZKH_ERR_ARG;
    if (!cols || !tag || !state || !msgs || !chals) return zkh_fail(ctx, ZKH_ERR_ARG, "sumcheck: null pointer");
    if (functor_nc(functor) != nc) return zkh_fail(ctx, ZKH_ERR_ARG, "sumcheck: nc does not match the summand");
    if (nt < 3 || nt > 5) return zkh_fail(ctx, ZKH_ERR_ARG, "sumcheck: nt must be 3..5");
    if (logn < 1 || logn > 34) return zkh_fail(ctx, ZKH_ERR_ARG, "sumcheck: logn must be 1..34");
    if (logn > 80) return zkh_fail(ctx, ZKH_ERR_LIMIT, "sumcheck: too many rounds");
    if (npar < 0 || npar > 8 || (npar > 0 && !par)) return zkh_fail(ctx, ZKH_ERR_ARG, "sumcheck: bad par");
    if (strlen(tag) > ZKH_TR_MAX_LABEL) return zkh_fail(ctx, ZKH_ERR_LIMIT, "sumcheck: tag longer than 48 bytes");
    return ZKH_OK;
}

extern "C" int zkh_sumcheck(zkh_ctx* ctx, int functor, int nt, const uint64_t* const* cols_dev, int nc,
                            uint32_t logn, const uint64_t* par, int npar, const char* tag,
                            uint8_t state[32], uint64_t* msgs, uint64_t* chals, uint64_t* finals) {
    ZKH_TRY(sumcheck_check(ctx, functor, nt, cols_dev, nc, logn, par, npar, tag, state, msgs, chals));
    for (int k = 0; k < nc; k++)
        if (!cols_dev[k] || ((uintptr_t)cols_dev[k] & 15))
            return zkh_fail(ctx, ZKH_ERR_ARG, "sumcheck: columns must be non-null and 16-byte aligned (128-bit loads)");
    ZKH_CUDA(ctx, cudaSetDevice(ctx->device));
    ZKH_TRY(zkh_ws_reserve(ctx, sc_workspace_bytes(nc, logn)));
    return sumcheck_common(ctx, functor, nt, cols_dev, nc, logn, par, npar, tag, state, msgs, chals,
                           finals, ctx->ws);
}

extern "C" int zkh_sumcheck_host(zkh_ctx* ctx, int functor, int nt, const uint64_t* const* cols, int nc,
                                 uint32_t logn, const uint64_t* par, int npar, const char* tag,
                                 uint8_t state[32], uint64_t* msgs, uint64_t* chals, uint64_t* finals) {
    ZKH_TRY(sumcheck_check(ctx, functor, nt, cols, nc, logn, par, npar, tag, state, msgs, chals));
    ZKH_CUDA(ctx, cudaSetDevice(ctx->device));
    const size_t colb = zkh_align(((size_t)8) << logn);
    ZKH_TRY(zkh_ws_reserve(ctx, (size_t)nc * colb + sc_workspace_bytes(nc, logn)));
    const uint64_t* d[8];
    for (int k = 0; k < nc; k++) {
        d[k] = (const uint64_t*)((char*)ctx->ws + (size_t)k * colb);
        ZKH_CUDA(ctx, cudaMemcpyAsync((void*)d[k], cols[k], ((size_t)8) << logn, cudaMemcpyHostToDevice,
                                      ctx->stream));
    }
    return sumcheck_common(ctx, functor, nt, d, nc, logn, par, npar, tag, state, msgs, chals, finals,
                           (char*)ctx->ws + (size_t)nc * colb);
}

// ------------------------------------------------------------------ sharded sumcheck (multi-GPU)
// The hypercube is split on its top log2(G) variables: GPU g holds the slice [g*n, (g+1)*n) of
// every column.  LSB-first pairs never cross a slice, so rounds 0..log2(n)-1 are local apart from
// summing the nt round values of all GPUs (the caller all-gathers them between
// zkh_shard_round_local and zkh_shard_round_combine; every GPU runs the same transcript).
// After log2(n) rounds each GPU holds one value per column; the caller all-gathers those and
// every GPU finishes the last log2(G) rounds on the G-element residual.
extern "C" int zkh_shard_begin(zkh_ctx* c, int functor, int nt, const uint64_t* const* cols_dev, int nc,
                               uint32_t logn_local, const uint64_t* par, int npar, const char* tag,
                               const uint8_t state[32]) {
    static const uint64_t dummy = 0;
    ZKH_TRY(sumcheck_check(c, functor, nt, cols_dev, nc, logn_local, par, npar, tag, state, &dummy, &dummy));
    for (int k = 0; k < nc; k++)
        if (!cols_dev[k] || ((uintptr_t)cols_dev[k] & 15))
            return zkh_fail(c, ZKH_ERR_ARG, "shard_begin: columns must be non-null and 16-byte aligned (128-bit loads)");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    const size_t n = (size_t)1 << logn_local;
    const size_t a = zkh_align((size_t)nc * (n / 2 + 1) * 8), b = zkh_align((size_t)nc * (n / 4 + 1) * 8);
    ZKH_TRY(zkh_ws_reserve(c, a + b + zkh_align((size_t)nc * 2048 * 8)));
    zkh_ctx::Shard& sh = c->shard;
    sh.active = true;
    sh.functor = functor; sh.nt = nt; sh.nc = nc; sh.logn = logn_local; sh.next_round = 0;
    sh.tag = zkh_make_tag(tag);
    for (int k = 0; k < nc; k++) sh.cur_in[k] = cols_dev[k];
    sh.bufA = (gl_t*)c->ws;
    sh.bufB = (gl_t*)((char*)c->ws + a);
    sh.res = (gl_t*)((char*)c->ws + a + b);
    sh.dst = sh.bufA;
    ZkhCtl* h = c->h_ctl;
    digest_from_bytes(state, h->st);
    h->counter = 0;
    h->err = 0;
    for (int i = 0; i < 8; i++) h->par[i] = i < npar ? par[i] : 0;
    ZKH_CUDA(c, cudaMemcpyAsync(c->d_ctl, h, offsetof(ZkhCtl, local), cudaMemcpyHostToDevice, c->stream));
    return ZKH_OK;
}
// ------------------------------------------------------------------ peer-to-peer round exchange
// One process per GPU.  zkh_p2p_create allocates this GPU's mailbox and returns its CUDA IPC handle; the
// caller exchanges the handles between the ranks (any host channel) and calls zkh_p2p_connect with all of
// them in rank order.  After that zkh_shard_round_fused runs a whole sharded round as ONE kernel: local
// bind + sums, peer stores of the sums, bounded wait for the other ranks, combine, transcript step.
extern "C" int zkh_p2p_create(zkh_ctx* c, uint8_t handle_out[64]) {
    if (!c || !handle_out) return zkh_fail(c, ZKH_ERR_ARG, "p2p_create: null pointer");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    if (!c->p2p.mine) {
        ZKH_CUDA(c, cudaMalloc(&c->p2p.mine, sizeof(ZkhMailbox)));
        ZKH_CUDA(c, cudaMemset(c->p2p.mine, 0, sizeof(ZkhMailbox)));
    }
    cudaIpcMemHandle_t h;
    ZKH_CUDA(c, cudaIpcGetMemHandle(&h, c->p2p.mine));
    memcpy(handle_out, &h, 64);
    return ZKH_OK;
}
extern "C" int zkh_p2p_disconnect(zkh_ctx* c) {
    if (!c) return ZKH_ERR_ARG;
    cudaSetDevice(c->device);
    if (c->stream) cudaStreamSynchronize(c->stream);
    for (int g = 0; g < ZKH_XCHG_MAXG; g++)
        if (c->p2p.opened[g]) { cudaIpcCloseMemHandle(c->p2p.opened[g]); c->p2p.opened[g] = nullptr; }
    if (c->p2p.d_xchg) { cudaFree(c->p2p.d_xchg); c->p2p.d_xchg = nullptr; }
    if (c->d_ctl) cudaMemset(&c->d_ctl->xchg, 0, sizeof(void*));
    c->p2p.G = 0;
    return ZKH_OK;
}
extern "C" int zkh_p2p_connect(zkh_ctx* c, uint32_t rank, uint32_t G, const uint8_t* handles) {
    if (!c || !handles) return zkh_fail(c, ZKH_ERR_ARG, "p2p_connect: null pointer");
    if (G < 2 || G > ZKH_XCHG_MAXG || rank >= G) return zkh_fail(c, ZKH_ERR_ARG, "p2p_connect: 2..16 ranks");
    if (!c->p2p.mine) return zkh_fail(c, ZKH_ERR_ARG, "p2p_connect: call zkh_p2p_create first");
    zkh_p2p_disconnect(c);
    ZKH_CUDA(c, cudaSetDevice(c->device));
    ZkhXchg hx;
    memset(&hx, 0, sizeof hx);
    hx.rank = rank;
    hx.G = G;
    hx.seq = 0;
    for (uint32_t g = 0; g < G; g++) {
        if (g == rank) { hx.mbox[g] = c->p2p.mine; continue; }
        cudaIpcMemHandle_t h;
        memcpy(&h, handles + (size_t)g * 64, 64);
        void* ptr = nullptr;
        if (cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
            cudaGetLastError();
            zkh_p2p_disconnect(c);
            return zkh_fail(c, ZKH_ERR_CUDA, "p2p_connect: cannot map a peer mailbox (no peer access between these GPUs?)");
        }
        c->p2p.opened[g] = ptr;
        hx.mbox[g] = (ZkhMailbox*)ptr;
    }
    ZKH_CUDA(c, cudaMemset(c->p2p.mine, 0, sizeof(ZkhMailbox)));
    ZKH_CUDA(c, cudaMalloc(&c->p2p.d_xchg, sizeof(ZkhXchg)));
    ZKH_CUDA(c, cudaMemcpy(c->p2p.d_xchg, &hx, sizeof hx, cudaMemcpyHostToDevice));
    void* xp = c->p2p.d_xchg;
    ZKH_CUDA(c, cudaMemcpy(&c->d_ctl->xchg, &xp, sizeof xp, cudaMemcpyHostToDevice));
    c->p2p.rank = (int)rank;
    c->p2p.G = (int)G;
    return ZKH_OK;
}
extern "C" int zkh_shard_round_fused(zkh_ctx* c, uint32_t r) {
    if (!c) return ZKH_ERR_ARG;
    zkh_ctx::Shard& sh = c->shard;
    if (c->p2p.G < 2) return zkh_fail(c, ZKH_ERR_ARG, "shard_round_fused: peer exchange not connected");
    if (!sh.active || r != sh.next_round || r >= sh.logn)
        return zkh_fail(c, ZKH_ERR_ARG, "shard_round_fused: rounds must run in order 0..logn_local-1");
    gl_t* msg = c->d_ctl->msgs + (size_t)r * sh.nt;
    if (r == 0) {
        ZKH_TRY(sc_enqueue_round(c, sh.functor, sh.nt, true, sh.cur_in, nullptr, (size_t)1 << sh.logn, nullptr, msg,
                                 c->d_ctl->chals + r, sh.tag, 2));
    } else {
        const size_t n_in = (size_t)1 << (sh.logn - r + 1), n_out = n_in / 2;
        gl_t* outp[8];
        for (int k = 0; k < sh.nc; k++) outp[k] = sh.dst + (size_t)k * n_out;
        const bool prof = (r == 1) && c->prof_ev[0];
        if (prof) cudaEventRecord(c->prof_ev[0], c->stream);
        ZKH_TRY(sc_enqueue_round(c, sh.functor, sh.nt, false, sh.cur_in, outp, n_in, c->d_ctl->chals + (r - 1), msg,
                                 c->d_ctl->chals + r, sh.tag, 2));
        if (prof) {
            cudaEventRecord(c->prof_ev[1], c->stream);
            c->prof_valid = true;
            c->prof_bytes = (uint64_t)12 * sh.nc * n_in;
            c->prof_kernel = "sc_fused_kernel";
        }
        for (int k = 0; k < sh.nc; k++) sh.cur_in[k] = outp[k];
        sh.dst = (sh.dst == sh.bufA) ? sh.bufB : sh.bufA;
    }
    sh.next_round = r + 1;
    return ZKH_OK;
}

// all local rounds of the running sharded sumcheck with the peer exchange, the last ones (columns of at most
// 2^12 elements) inside one single-CTA kernel per GPU; this rank's bound column values go to finals_dev.
// whole: that last kernel also all-gathers the bound values through the mailboxes and runs the log2(G) residual rounds,
// so the proof is complete when it ends (no collective and no further launch).
static int shard_fused(zkh_ctx* c, uint64_t* finals_dev, bool whole) {
    zkh_ctx::Shard& sh = c->shard;
    if (c->p2p.G < 2) return zkh_fail(c, ZKH_ERR_ARG, "shard fused: peer exchange not connected");
    if (!sh.active || sh.next_round != 0) return zkh_fail(c, ZKH_ERR_ARG, "shard fused: must follow shard_begin");
    uint32_t k2 = 0;
    while ((1u << k2) < (uint32_t)c->p2p.G) k2++;
    if (whole && sh.logn + k2 > 80) return zkh_fail(c, ZKH_ERR_LIMIT, "shard fused: too many rounds");
    const int resid = whole ? (int)k2 : 0;
    uint32_t r = 0;
    if (sh.logn <= SC_TAIL_LOG) {
        ZKH_TRY(sc_enqueue_tail(c, sh.functor, sh.nt, sh.cur_in, 1u << sh.logn, (int)sh.logn, c->d_ctl->msgs, c->d_ctl->chals,
                                finals_dev, sh.tag, 0, nullptr, 2, resid));
    } else {
        ZKH_TRY(zkh_shard_round_fused(c, 0));
        for (r = 1; sh.logn - r + 1 > SC_TAIL_LOG + 1; r++) ZKH_TRY(zkh_shard_round_fused(c, r));
        // columns of 2^(logn-r+1) <= 2^12 elements, still to be bound with challenge r-1
        ZKH_TRY(sc_enqueue_tail(c, sh.functor, sh.nt, sh.cur_in, 1u << (sh.logn - r + 1), (int)(sh.logn - r),
                                c->d_ctl->msgs + (size_t)r * sh.nt, c->d_ctl->chals + r, finals_dev, sh.tag, 1,
                                c->d_ctl->chals + (r - 1), 2, resid));
    }
    sh.next_round = sh.logn + (whole ? k2 : 0);
    return ZKH_OK;
}
extern "C" int zkh_shard_local_fused(zkh_ctx* c, uint64_t* finals_dev) {
    if (!c || !finals_dev) return zkh_fail(c, ZKH_ERR_ARG, "shard_local_fused: null pointer");
    return shard_fused(c, finals_dev, false);
}
extern "C" int zkh_shard_prove_fused(zkh_ctx* c) {
    if (!c) return ZKH_ERR_ARG;
    return shard_fused(c, nullptr, true);
}

extern "C" int zkh_shard_round_local(zkh_ctx* c, uint32_t r, uint64_t* sums_dev) {
    if (!c || !sums_dev) return zkh_fail(c, ZKH_ERR_ARG, "shard_round_local: null pointer");
    zkh_ctx::Shard& sh = c->shard;
    if (!sh.active || r != sh.next_round || r >= sh.logn)
        return zkh_fail(c, ZKH_ERR_ARG, "shard_round_local: rounds must run in order 0..logn_local-1");
    if (r == 0)
        return sc_enqueue_round(c, sh.functor, sh.nt, true, sh.cur_in, nullptr, (size_t)1 << sh.logn, nullptr,
                                sums_dev, nullptr, sh.tag, 1);
    const size_t n_in = (size_t)1 << (sh.logn - r + 1), n_out = n_in / 2;
    gl_t* outp[8];
    for (int k = 0; k < sh.nc; k++) outp[k] = sh.dst + (size_t)k * n_out;
    const bool prof = (r == 1) && c->prof_ev[0];
    if (prof) cudaEventRecord(c->prof_ev[0], c->stream);
    ZKH_TRY(sc_enqueue_round(c, sh.functor, sh.nt, false, sh.cur_in, outp, n_in, c->d_ctl->chals + (r - 1), sums_dev,
                             nullptr, sh.tag, 1));
    if (prof) {
        cudaEventRecord(c->prof_ev[1], c->stream);
        c->prof_valid = true;
        c->prof_bytes = (uint64_t)12 * sh.nc * n_in;
        c->prof_kernel = "sc_fused_kernel";
    }
    for (int k = 0; k < sh.nc; k++) sh.cur_in[k] = outp[k];
    sh.dst = (sh.dst == sh.bufA) ? sh.bufB : sh.bufA;
    return ZKH_OK;
}
extern "C" int zkh_shard_round_combine(zkh_ctx* c, uint32_t r, const uint64_t* gathered_dev, uint32_t G) {
    if (!c || !gathered_dev) return zkh_fail(c, ZKH_ERR_ARG, "shard_round_combine: null pointer");
    zkh_ctx::Shard& sh = c->shard;
    if (!sh.active || r != sh.next_round || G < 1 || G > 1024)
        return zkh_fail(c, ZKH_ERR_ARG, "shard_round_combine: out of order, or G outside 1..1024");
    sc_combine_kernel<<<1, 32, 0, c->stream>>>(c->d_ctl, gathered_dev, G, sh.nt, sh.tag,
                                              c->d_ctl->msgs + (size_t)r * sh.nt, c->d_ctl->chals + r);
    ZKH_CUDA(c, cudaGetLastError());
    sh.next_round = r + 1;
    return ZKH_OK;
}
extern "C" int zkh_shard_finals(zkh_ctx* c, uint64_t* finals_dev) {
    if (!c || !finals_dev) return zkh_fail(c, ZKH_ERR_ARG, "shard_finals: null pointer");
    zkh_ctx::Shard& sh = c->shard;
    if (!sh.active || sh.next_round != sh.logn) return zkh_fail(c, ZKH_ERR_ARG, "shard_finals: local rounds not finished");
    ScPtrs P;
    memset(&P, 0, sizeof P);
    for (int k = 0; k < sh.nc; k++) P.in[k] = sh.cur_in[k];
    sc_finals_kernel<<<1, 32, 0, c->stream>>>(P, sh.nc, c->d_ctl->chals + (sh.logn - 1), finals_dev);
    ZKH_CUDA(c, cudaGetLastError());
    return ZKH_OK;
}
extern "C" int zkh_shard_residual(zkh_ctx* c, const uint64_t* gathered_finals_dev, uint32_t G) {
    if (!c || !gathered_finals_dev) return zkh_fail(c, ZKH_ERR_ARG, "shard_residual: null pointer");
    zkh_ctx::Shard& sh = c->shard;
    if (!sh.active || sh.next_round != sh.logn) return zkh_fail(c, ZKH_ERR_ARG, "shard_residual: local rounds not finished");
    if (G < 1 || G > 2048 || (G & (G - 1))) return zkh_fail(c, ZKH_ERR_ARG, "shard_residual: G must be a power of two <= 2048");
    uint32_t k2 = 0;
    while ((1u << k2) < G) k2++;
    if (G == 1) {
        ZKH_CUDA(c, cudaMemcpyAsync(c->d_ctl->finals, gathered_finals_dev, (size_t)sh.nc * 8, cudaMemcpyDeviceToDevice,
                                    c->stream));
    } else {
        sc_transpose_kernel<<<(G * sh.nc + 255) / 256, 256, 0, c->stream>>>(gathered_finals_dev, sh.res, G, sh.nc);
        const gl_t* in[8];
        for (int k = 0; k < sh.nc; k++) in[k] = sh.res + (size_t)k * G;
        ZKH_TRY(sc_enqueue_tail(c, sh.functor, sh.nt, in, G, (int)k2, c->d_ctl->msgs + (size_t)sh.logn * sh.nt,
                                c->d_ctl->chals + sh.logn, c->d_ctl->finals, sh.tag));
    }
    sh.next_round = sh.logn + k2;
    return ZKH_OK;
}
extern "C" int zkh_shard_end(zkh_ctx* c, uint8_t state[32], uint64_t* msgs, uint64_t* chals, uint64_t* finals) {
    if (!c || !state || !msgs || !chals) return zkh_fail(c, ZKH_ERR_ARG, "shard_end: null pointer");
    zkh_ctx::Shard& sh = c->shard;
    if (!sh.active) return zkh_fail(c, ZKH_ERR_ARG, "shard_end: no sharded sumcheck is running");
    ZkhCtl* h = c->h_ctl;
    ZKH_CUDA(c, cudaMemcpyAsync(h, c->d_ctl, sizeof(ZkhCtl), cudaMemcpyDeviceToHost, c->stream));
    ZKH_CUDA(c, cudaStreamSynchronize(c->stream));
    sh.active = false;
    if (h->err) return zkh_fail(c, ZKH_ERR_DEVICE, "shard_end: device error flag set");
    memcpy(msgs, h->msgs, (size_t)sh.next_round * sh.nt * 8);
    memcpy(chals, h->chals, (size_t)sh.next_round * 8);
    if (finals) memcpy(finals, h->finals, (size_t)sh.nc * 8);
    digest_to_bytes(h->st, state);
    return ZKH_OK;
}
