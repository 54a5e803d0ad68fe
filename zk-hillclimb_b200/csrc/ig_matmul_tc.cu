// Exact integer matrix products on the 5th-generation tensor cores (tcgen05, sm_100a): the tensor-core form of
// zkh_ig_matmul for the shapes of a full-size layer (rows a multiple of 128, columns and inner dimension multiples of 64,
// operands in (-2^20, 2^20)).
//
// Exactness: every operand v is split into three 7-bit limbs v = l0 + 2^7 l1 + 2^14 l2 with l0, l1 in [0, 128) and
// l2 = v >> 14 in [-64, 64), all signed 8-bit.  The nine limb products are accumulated in FIVE 32-bit integer accumulators
// by weight (acc[s] = sum over a + b = s of A_a . B_b^T; |acc| < 3 * 2^14 * 127^2 < 2^30 for an inner dimension of up to
// 2^14), and the epilogue forms C = sum_s acc[s] << 7s in 64-bit integers and writes it field-lifted.
//
// Data path:  a split kernel writes the int8 limb planes of both operands ALREADY in the shared-memory image of the tiles
// (one 8 KB block per 128-row x 64-byte tile of A, one 4 KB block per 64 x 64 tile of B, each in the canonical no-swizzle
// K-major core-matrix layout: 8 rows x 16 bytes per core matrix; it also transposes where an operand is stored the other
// way round)  ->  one thread streams the blocks into a four-stage shared-memory ring with bulk asynchronous copies
// (cp.async.bulk, completion counted in bytes on the stage's "full" mbarrier)  ->  a second thread issues tcgen05.mma
// kind::i8, M = 128, N = 64, K = 32 per instruction, accumulators in tensor memory (5 x 64 columns), and hands the stage
// back with tcgen05.commit onto its "empty" mbarrier  ->  tcgen05.ld of the accumulators by the CTA's four warps (32
// lanes each) for the epilogue.
// Every wait on an mbarrier is bounded: when it runs out the kernel raises the device error flag, skips the remaining
// work, frees its tensor memory and returns (the caller then gets ZKH_ERR_DEVICE).
#include "common.cuh"

namespace zkh {

struct TcView { long long sb0, sb1, sr, sc; };

constexpr int TC_BM = 128, TC_BN = 64, TC_BK = 64;          // CTA tile; TC_BK bytes of inner dimension per stage
constexpr int TC_STAGES = 4;
constexpr int TC_A_BYTES = TC_BM * TC_BK, TC_B_BYTES = TC_BN * TC_BK;
constexpr int TC_STAGE_BYTES = 3 * TC_A_BYTES + 3 * TC_B_BYTES;          // 36 KB
constexpr uint32_t TC_TMEM_COLS = 512;                                    // 5 accumulators of 64 columns -> next power of two
constexpr uint32_t TC_SPIN_LIMIT = 1u << 22;
constexpr int TC_SMEM_BYTES = TC_STAGES * TC_STAGE_BYTES + 1024;     // 145 KB: one CTA (and one 512-column allocation) per SM

// ---- operand split: field-lifted integers -> three int8 limb planes in tile-image order ----
// src(b0, b1, row, k) at src + b0*sb0 + b1*sb1 + row*sr + k*sc.  Plane l of batch entry z holds, for row tile it (tile_rows
// rows) and k tile kt (64 bytes), one block of tile_rows * 64 bytes at ((z * RT + it) * KT + kt) * tile_rows * 64 whose bytes sit
// where the GEMM wants them in shared memory: row r, byte k of the tile at (r / 8) * 512 + (k / 16) * 128 + (r % 8) * 16 + k % 16.
// Source tiles of 64 x 64 go through shared memory so that the reads (along whichever source dimension has the smaller
// stride) and the writes (16-byte chunks, eight of them contiguous) are both coalesced.
__global__ void __launch_bounds__(256)
ig_limbs_kernel(const gl_t* __restrict__ src, TcView v, uint32_t nb1, uint32_t rows, uint32_t K, uint32_t tile_rows,
                int8_t* __restrict__ out, size_t plane, unsigned int* flags) {
    __shared__ __align__(16) int8_t sm[3][64][64 + 16];
    const uint32_t b0 = blockIdx.z / nb1, b1 = blockIdx.z % nb1;
    const uint32_t r0 = blockIdx.y * 64, k0 = blockIdx.x * 64;
    src += (long long)b0 * v.sb0 + (long long)b1 * v.sb1;
    const bool by_k = v.sc <= v.sr;
    bool big = false;
    for (uint32_t e = threadIdx.x; e < 64 * 64; e += blockDim.x) {
        const uint32_t r = by_k ? e / 64 : e % 64, k = by_k ? e % 64 : e / 64;
        const gl_t x = src[(long long)(r0 + r) * v.sr + (long long)(k0 + k) * v.sc];      // rows and K are multiples of 64
        const long long s = (long long)(x >> 63 ? x + 0xFFFFFFFFull : x);
        big |= (s <= -(1ll << 20)) | (s >= (1ll << 20));
        sm[0][r][k] = (int8_t)(s & 127);
        sm[1][r][k] = (int8_t)((s >> 7) & 127);
        sm[2][r][k] = (int8_t)(s >> 14);
    }
    __syncthreads();
    const uint32_t KT = K / 64, RT = rows / tile_rows;
    const uint32_t it = r0 / tile_rows, rbase = r0 % tile_rows, kt = k0 / 64;
    int8_t* blk = out + (((size_t)blockIdx.z * RT + it) * KT + kt) * ((size_t)tile_rows * 64);
    for (uint32_t e = threadIdx.x; e < 3 * 64 * 4; e += blockDim.x) {            // 16-byte chunks: 8 rows of one chunk column are contiguous
        const uint32_t l = e / 256, q = e % 256, rr = (q & 7) | ((q >> 5) << 3), kc = (q >> 3) & 3;
        const uint32_t r = rbase + rr;
        *reinterpret_cast<int4*>(blk + l * plane + (r >> 3) * 512 + kc * 128 + (r & 7) * 16) = *reinterpret_cast<const int4*>(&sm[l][rr][16 * kc]);
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
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// bulk asynchronous copy global -> shared (16-byte aligned, size a multiple of 16); completion is counted on the mbarrier
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
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

// One CTA (128 threads) = one 128 x 64 tile of C for one batch entry.  Al / Bl: limb planes in tile-image order.
// Thread 0 of warp 0 streams the tiles in; thread 0 of warp 1 issues the tensor-core instructions; all four warps run the epilogue.
__global__ void __launch_bounds__(128, 1)
ig_matmul_tc_kernel(const int8_t* __restrict__ Al, const int8_t* __restrict__ Bl, size_t planeA, size_t planeB, gl_t* __restrict__ C,
                    TcView vc, uint32_t nb1, uint32_t I, uint32_t K, uint32_t N, unsigned int* err) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ __align__(8) uint64_t bar_full[TC_STAGES];
    __shared__ __align__(8) uint64_t bar_empty[TC_STAGES];
    __shared__ __align__(8) uint64_t bar_done;
    __shared__ uint32_t tmem_base_sh;
    __shared__ uint32_t failed_sh;
    const uint32_t tid = threadIdx.x, warp = tid >> 5;
    const uint32_t b0 = blockIdx.z / nb1, b1 = blockIdx.z % nb1;
    const uint32_t i0 = blockIdx.y * TC_BM, n0 = blockIdx.x * TC_BN;
    const uint32_t KT = K / TC_BK;
    const int8_t* Ab = Al + (((size_t)blockIdx.z * (I / TC_BM) + blockIdx.y) * KT) * TC_A_BYTES;
    const int8_t* Bb = Bl + (((size_t)blockIdx.z * (N / TC_BN) + blockIdx.x) * KT) * TC_B_BYTES;
    C += (long long)b0 * vc.sb0 + (long long)b1 * vc.sb1;

    if (tid == 0) {
        for (int s = 0; s < TC_STAGES; s++) { mbar_init(&bar_full[s], 1); mbar_init(&bar_empty[s], 1); }
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

    if (tid == 0) {
        // producer: refill a stage as soon as the instructions that read it have retired (a fresh barrier counts as released)
        for (uint32_t kt = 0; kt < KT; kt++) {
            const uint32_t st = kt % TC_STAGES, use = kt / TC_STAGES;
            if (!mbar_wait(&bar_empty[st], (use & 1) ^ 1)) { failed_sh = 1; break; }
            uint8_t* sbuf = smem + (size_t)st * TC_STAGE_BYTES;
            mbar_expect_tx(&bar_full[st], TC_STAGE_BYTES);
#pragma unroll
            for (int l = 0; l < 3; l++) {
                bulk_g2s(sbuf + l * TC_A_BYTES, Ab + l * planeA + (size_t)kt * TC_A_BYTES, TC_A_BYTES, &bar_full[st]);
                bulk_g2s(sbuf + 3 * TC_A_BYTES + l * TC_B_BYTES, Bb + l * planeB + (size_t)kt * TC_B_BYTES, TC_B_BYTES, &bar_full[st]);
            }
        }
    } else if (tid == 32) {
        // tensor-core issuer
        bool ok = true;
        for (uint32_t kt = 0; kt < KT; kt++) {
            const uint32_t st = kt % TC_STAGES, use = kt / TC_STAGES;
            if (!mbar_wait(&bar_full[st], use & 1)) { failed_sh = 1; ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t sa = smem_u32(smem + (size_t)st * TC_STAGE_BYTES), sb = sa + 3 * TC_A_BYTES;
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
            mma_commit(&bar_empty[st]);
        }
        if (ok) mma_commit(&bar_done);
    }
    __syncwarp();
    // every thread waits for the last instruction to retire (bounded), then the CTA agrees on the outcome
    {
        const bool got = mbar_wait(&bar_done, 0);
        const bool all = __syncthreads_and(got);
        if (!all && tid == 0) failed_sh = 1;
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    __syncthreads();
    if (!failed_sh) {
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
    ig_limbs_kernel<<<dim3(J / 64, I / 64, (unsigned)nb), 256, 0, s>>>(A, va, nb1, I, J, TC_BM, Al, planeA, flags);
    ig_limbs_kernel<<<dim3(J / 64, K / 64, (unsigned)nb), 256, 0, s>>>(B, vb, nb1, K, J, TC_BN, Bl, planeB, flags);
    ZKH_CUDA(c, cudaGetLastError());
    ZKH_CUDA(c, cudaMemcpyAsync(&c->h_ctl->err, flags, 4, cudaMemcpyDeviceToHost, s));
    ZKH_CUDA(c, cudaStreamSynchronize(s));
    if (c->h_ctl->err & 1u) return 1;             // an operand outside (-2^20, 2^20): three 7-bit limbs do not hold it
    static ZkhOncePerDevice attr;
    zkh_once_on_device(attr, c->device, [] { cudaFuncSetAttribute(ig_matmul_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_BYTES); });
    static_assert(TC_STAGES * TC_STAGE_BYTES <= TC_SMEM_BYTES && 2 * TC_SMEM_BYTES > 227 * 1024, "one CTA per SM");
    ig_matmul_tc_kernel<<<dim3(K / TC_BN, I / TC_BM, (unsigned)nb), 128, TC_SMEM_BYTES, s>>>(
        Al, Bl, planeA, planeB, Cc, vc, nb1, I, J, K, flags);
    ZKH_CUDA(c, cudaGetLastError());
    ZKH_CUDA(c, cudaMemcpyAsync(&c->h_ctl->err, flags, 4, cudaMemcpyDeviceToHost, s));
    ZKH_CUDA(c, cudaStreamSynchronize(s));
    if (c->h_ctl->err & 64u) return zkh_fail(c, ZKH_ERR_DEVICE, "ig_matmul: a tensor-core stage did not complete within its wait bound");
    return ZKH_OK;
}

}  // namespace zkh
