// Exact integer matrix products on the 5th-generation tensor cores (tcgen05, sm_100a): the tensor-core form of
// zkh_ig_matmul for the shapes of a full-size layer (rows a multiple of 128, columns and inner dimension multiples of 64,
// operands in (-2^20, 2^20)).
//
// Exactness: every operand v is split into three 7-bit limbs v = l0 + 2^7 l1 + 2^14 l2 with l0, l1 in [0, 128) and
// l2 = v >> 14 in [-64, 64), all signed 8-bit.  The nine limb products are accumulated in FIVE 32-bit integer accumulators
// by weight (acc[s] = sum over a + b = s of A_a . B_b^T; |acc| < 3 * 2^14 * 127^2 < 2^30 for an inner dimension of up to
// 2^14), and the epilogue forms C = sum_s acc[s] << 7s in 64-bit integers and writes it field-lifted.
//
// Data path:  limb planes (int8, inner dimension contiguous for BOTH operands, written by a split kernel that also
// transposes where an operand is stored the other way round)  ->  16-byte loads into shared memory in the canonical
// no-swizzle K-major core-matrix layout (8 rows x 16 bytes per core matrix)  ->  tcgen05.mma kind::i8, M = 128, N = 64,
// K = 32 per instruction, issued by one thread, accumulators in tensor memory (5 x 64 columns)  ->  tcgen05.commit onto
// an mbarrier per shared-memory stage (the stage may be refilled when the instructions reading it have retired)  ->
// tcgen05.ld of the accumulators by four warps (32 lanes each) for the epilogue.
// Every wait on an mbarrier is bounded: when it runs out the kernel raises the device error flag, skips the remaining
// work, frees its tensor memory and returns (the caller then gets ZKH_ERR_DEVICE).
#include "common.cuh"

namespace zkh {

struct TcView { long long sb0, sb1, sr, sc; };

constexpr int TC_BM = 128, TC_BN = 64, TC_BK = 64;          // CTA tile; TC_BK bytes of inner dimension per stage
constexpr int TC_STAGES = 2;
constexpr int TC_A_BYTES = TC_BM * TC_BK, TC_B_BYTES = TC_BN * TC_BK;
constexpr int TC_STAGE_BYTES = 3 * TC_A_BYTES + 3 * TC_B_BYTES;          // 36 KB
constexpr uint32_t TC_TMEM_COLS = 512;                                    // 5 accumulators of 64 columns -> next power of two
constexpr uint32_t TC_SPIN_LIMIT = 1u << 22;
constexpr int TC_SMEM_BYTES = 116 * 1024;     // more than half of an SM's shared memory: one CTA (and one 512-column allocation) per SM

// ---- operand split: field-lifted integers -> three int8 limb planes [limb][batch][row][k], k contiguous ----
// src(b0, b1, row, k) at src + b0*sb0 + b1*sb1 + row*sr + k*sc.  Tiles of 64 x 64 go through shared memory so that both the
// reads (along whichever source dimension has the smaller stride) and the writes (along k) are coalesced.
__global__ void __launch_bounds__(256)
ig_limbs_kernel(const gl_t* __restrict__ src, TcView v, uint32_t nb1, uint32_t rows, uint32_t K, int8_t* __restrict__ out,
                size_t plane, unsigned int* flags) {
    __shared__ __align__(16) int8_t sm[3][64][64 + 4];
    const uint32_t b0 = blockIdx.z / nb1, b1 = blockIdx.z % nb1;
    const uint32_t r0 = blockIdx.y * 64, k0 = blockIdx.x * 64;
    src += (long long)b0 * v.sb0 + (long long)b1 * v.sb1;
    const bool by_k = v.sc <= v.sr;
    bool big = false;
    for (uint32_t e = threadIdx.x; e < 64 * 64; e += blockDim.x) {
        const uint32_t r = by_k ? e / 64 : e % 64, k = by_k ? e % 64 : e / 64;
        long long s = 0;
        if (r0 + r < rows && k0 + k < K) {
            const gl_t x = src[(long long)(r0 + r) * v.sr + (long long)(k0 + k) * v.sc];
            s = (long long)(x >> 63 ? x + 0xFFFFFFFFull : x);
            big |= (s <= -(1ll << 20)) | (s >= (1ll << 20));
        }
        sm[0][r][k] = (int8_t)(s & 127);
        sm[1][r][k] = (int8_t)((s >> 7) & 127);
        sm[2][r][k] = (int8_t)(s >> 14);
    }
    __syncthreads();
    int8_t* dst = out + (size_t)blockIdx.z * rows * K;
    for (uint32_t e = threadIdx.x; e < 3 * 64 * 16; e += blockDim.x) {          // 4-byte words along k
        const uint32_t l = e / (64 * 16), r = (e / 16) % 64, kw = e % 16;
        if (r0 + r < rows && k0 + 4 * kw < K)
            *reinterpret_cast<int*>(dst + l * plane + (size_t)(r0 + r) * K + k0 + 4 * kw) = *reinterpret_cast<const int*>(&sm[l][r][4 * kw]);
    }
    if (big) atomicOr(flags, 1u);
}

// ---- PTX wrappers ----
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
// bounded wait for the completion of the phase with the given parity; false when the bound ran out
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t a = smem_u32(bar);
    for (uint32_t it = 0; it < TC_SPIN_LIMIT; it++) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(a), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
// shared-memory matrix descriptor, K-major, no swizzle: core matrices of 8 rows x 16 bytes; lbo = distance between the two
// 16-byte halves of an instruction's K = 32 bytes, sbo = distance between 8-row groups (both in bytes)
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)((lbo >> 4) & 0x3FFF) << 16) | ((uint64_t)((sbo >> 4) & 0x3FFF) << 32) |
           (1ull << 46);                                                 // descriptor version of this architecture
}
// instruction descriptor: signed 8-bit A and B (both K-major), 32-bit integer accumulator, M = 128, N = 64
constexpr uint32_t TC_IDESC = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TC_BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);

__device__ __forceinline__ void mma_i8(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t"
        "}\n"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(TC_IDESC), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n\t"
        "tcgen05.wait::ld.sync.aligned;\n"                      // in the same statement: no use of the registers can move above it
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

// One CTA = one 128 x 64 tile of C for one batch entry.  A limb planes: [3][batch][I][K], B limb planes: [3][batch][N][K].
__global__ void __launch_bounds__(256, 1)
ig_matmul_tc_kernel(const int8_t* __restrict__ Al, const int8_t* __restrict__ Bl, size_t planeA, size_t planeB, gl_t* __restrict__ C,
                    TcView vc, uint32_t nb1, uint32_t I, uint32_t K, uint32_t N, unsigned int* err) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ __align__(8) uint64_t bar_stage[TC_STAGES];
    __shared__ __align__(8) uint64_t bar_done;
    __shared__ uint32_t tmem_base_sh;
    __shared__ uint32_t failed_sh;
    const uint32_t tid = threadIdx.x, warp = tid >> 5;
    const uint32_t b0 = blockIdx.z / nb1, b1 = blockIdx.z % nb1;
    const uint32_t i0 = blockIdx.y * TC_BM, n0 = blockIdx.x * TC_BN;
    const int8_t* Ab = Al + (size_t)blockIdx.z * I * K + (size_t)i0 * K;
    const int8_t* Bb = Bl + (size_t)blockIdx.z * N * K + (size_t)n0 * K;
    C += (long long)b0 * vc.sb0 + (long long)b1 * vc.sb1;

    if (tid == 0) {
        for (int s = 0; s < TC_STAGES; s++) mbar_init(&bar_stage[s], 1);
        mbar_init(&bar_done, 1);
        failed_sh = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {       // one warp allocates the tensor memory of this CTA and gives the permit back
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_sh)), "r"(TC_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_base_sh;

    const uint32_t KT = K / TC_BK;
    bool ok = true;
    for (uint32_t kt = 0; kt < KT; kt++) {
        const uint32_t st = kt % TC_STAGES;
        uint8_t* sbuf = smem + (size_t)st * TC_STAGE_BYTES;
        if (kt >= TC_STAGES) {            // the instructions that read this stage two iterations ago must have retired
            const bool got = mbar_wait(&bar_stage[st], ((kt / TC_STAGES) - 1) & 1);
            ok = __syncthreads_and(got);  // one verdict for the whole CTA: nobody leaves the loop alone
            if (!ok) break;
        }
        // 16-byte chunks: row r, chunk kc of the stage -> core-matrix layout (r / 8) * 512 + kc * 128 + (r % 8) * 16
        for (uint32_t e = tid; e < 3 * (TC_BM + TC_BN) * 4; e += blockDim.x) {
            const uint32_t kc = e & 3, rr = e >> 2;
            uint32_t l, r;
            const int8_t* g;
            uint8_t* s;
            if (rr < 3 * TC_BM) { l = rr / TC_BM; r = rr % TC_BM; g = Ab + l * planeA + (size_t)r * K; s = sbuf + l * TC_A_BYTES; }
            else { const uint32_t q = rr - 3 * TC_BM; l = q / TC_BN; r = q % TC_BN; g = Bb + l * planeB + (size_t)r * K; s = sbuf + 3 * TC_A_BYTES + l * TC_B_BYTES; }
            const int4 val = __ldg(reinterpret_cast<const int4*>(g + (size_t)kt * TC_BK + kc * 16));
            *reinterpret_cast<int4*>(s + (r >> 3) * 512 + kc * 128 + (r & 7) * 16) = val;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // generic-proxy stores -> visible to the tensor core's reads
        __syncthreads();
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (ok) {
                const uint32_t sa = smem_u32(sbuf), sb = sa + 3 * TC_A_BYTES;
#pragma unroll
                for (int ks = 0; ks < TC_BK / 32; ks++) {
#pragma unroll
                    for (int a = 0; a < 3; a++) {
#pragma unroll
                        for (int b = 0; b < 3; b++) {
                            const uint64_t da = smem_desc(sa + a * TC_A_BYTES + ks * 256, 128, 512);
                            const uint64_t db = smem_desc(sb + b * TC_B_BYTES + ks * 256, 128, 512);
                            // the first product that reaches accumulator a + b overwrites it: pairs (0,0) (0,1) (0,2) (1,2) (2,2)
                            const bool first = kt == 0 && ks == 0 && (a == 0 || b == 2);
                            mma_i8(tmem + (uint32_t)(a + b) * TC_BN, da, db, first ? 0u : 1u);
                        }
                    }
                }
            }
            mma_commit(&bar_stage[st]);
            if (kt + 1 == KT) mma_commit(&bar_done);
        }
        // no barrier here: the next iteration fills the OTHER stage; this one is protected by its mbarrier
    }
    {
        const bool got = ok && mbar_wait(&bar_done, 0);
        ok = __syncthreads_and(got);
    }
    if (!ok && tid == 0) failed_sh = 1;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    __syncthreads();
    if (!failed_sh && warp < 4) {
        // warp w reads lanes 32w .. 32w + 31 (rows of the tile); 32 columns at a time from each of the five accumulators
        const uint32_t row = i0 + warp * 32 + (tid & 31);
#pragma unroll 1
        for (int half = 0; half < TC_BN / 32; half++) {
            long long sum[32];
#pragma unroll
            for (int j = 0; j < 32; j++) sum[j] = 0;
#pragma unroll
            for (int s = 0; s < 5; s++) {
                uint32_t r[32];
                tmem_ld32(tmem + ((warp * 32u) << 16) + (uint32_t)s * TC_BN + half * 32, r);
#pragma unroll
                for (int j = 0; j < 32; j++) sum[j] += (long long)(int)r[j] << (7 * s);
            }
            gl_t* crow = C + (long long)row * vc.sr + (long long)(n0 + half * 32) * vc.sc;
#pragma unroll
            for (int j = 0; j < 32; j++) crow[(long long)j * vc.sc] = sum[j] < 0 ? (gl_t)sum[j] - 0xFFFFFFFFull : (gl_t)sum[j];
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TC_TMEM_COLS) : "memory");
    if (tid == 0 && failed_sh) atomicOr(err, 64u);
}

// Returns ZKH_OK when the product ran on the tensor cores, 1 when the shapes or the operand range rule it out (nothing was
// written: the caller runs the integer-pipe kernel), or an error code.
int ig_matmul_tc(zkh_ctx* c, const gl_t* A, const long long sa[4], const gl_t* B, const long long sb[4], gl_t* Cc, const long long sc[4],
                 uint32_t nb0, uint32_t nb1, uint32_t I, uint32_t J, uint32_t K) {
    // J = inner dimension, K = columns of C (the caller's naming)
    if (I % TC_BM || K % TC_BN || J % TC_BK || J > (1u << 14)) return 1;
    const size_t nb = (size_t)nb0 * nb1;
    const size_t planeA = nb * I * J, planeB = nb * K * J;
    ZKH_TRY(zkh_ws_reserve(c, zkh_align(3 * planeA) + zkh_align(3 * planeB) + 256));
    int8_t* Al = (int8_t*)c->ws;
    int8_t* Bl = Al + zkh_align(3 * planeA);
    unsigned int* flags = &c->d_ctl->err;
    cudaStream_t s = c->stream;
    ZKH_CUDA(c, cudaMemsetAsync(flags, 0, 4, s));
    TcView va{sa[0], sa[1], sa[2], sa[3]};
    TcView vb{sb[0], sb[1], sb[3], sb[2]};        // B is addressed (j, k): its planes hold row = k (column of C), inner = j
    TcView vc{sc[0], sc[1], sc[2], sc[3]};
    ig_limbs_kernel<<<dim3(J / 64, I / 64, (unsigned)nb), 256, 0, s>>>(A, va, nb1, I, J, Al, planeA, flags);
    ig_limbs_kernel<<<dim3(J / 64, K / 64, (unsigned)nb), 256, 0, s>>>(B, vb, nb1, K, J, Bl, planeB, flags);
    ZKH_CUDA(c, cudaGetLastError());
    ZKH_CUDA(c, cudaMemcpyAsync(&c->h_ctl->err, flags, 4, cudaMemcpyDeviceToHost, s));
    ZKH_CUDA(c, cudaStreamSynchronize(s));
    if (c->h_ctl->err & 1u) return 1;             // an operand outside (-2^20, 2^20): three 7-bit limbs do not hold it
    static std::atomic<uint64_t> attr{0};
    if (zkh_first_on_device(attr, c->device))
        cudaFuncSetAttribute(ig_matmul_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_BYTES);
    static_assert(TC_STAGES * TC_STAGE_BYTES <= TC_SMEM_BYTES, "stages must fit the shared-memory request");
    ig_matmul_tc_kernel<<<dim3(K / TC_BN, I / TC_BM, (unsigned)nb), 256, TC_SMEM_BYTES, s>>>(
        Al, Bl, planeA, planeB, Cc, vc, nb1, I, J, K, flags);
    ZKH_CUDA(c, cudaGetLastError());
    ZKH_CUDA(c, cudaMemcpyAsync(&c->h_ctl->err, flags, 4, cudaMemcpyDeviceToHost, s));
    ZKH_CUDA(c, cudaStreamSynchronize(s));
    if (c->h_ctl->err & 64u) return zkh_fail(c, ZKH_ERR_DEVICE, "ig_matmul: a tensor-core stage did not complete within its wait bound");
    return ZKH_OK;
}

}  // namespace zkh
