// Multilinear evaluation for callers that must not allocate device memory.
//
// Who needs this: a host that has handed the whole GPU to its own arena (a proving
// service that reserves HBM up front and treats any later cudaMalloc as a bug), code
// running between cudaStreamBeginCapture/EndCapture where cudaMalloc is illegal, and
// latency-critical loops where an allocation's implicit device synchronisation would
// stall every stream.  The regular entry point, zkh_gl_mle_eval, grows a context
// workspace with cudaMalloc on demand; this one never does.
//
// How: the scratch the kernels need (two factor tables of the eq polynomial and the
// per-CTA partial sums) lives in ONE file-scope __device__ array of fixed size
// (ZKH_STATIC_SCRATCH_BYTES = 278,528 bytes).  Every GPU on which this library runs a
// kernel carries that array from module load until the process exits.  The fixed size
// caps the problem: at most ZKH_STATIC_MAX_V = 28 variables (2^28 coefficients).
//
// In host code the array's name is only a handle, not a device address.  The device
// address is looked up once per device with cudaGetSymbolAddress, with that device
// current, and kept in a per-device table; kernels receive that address as an argument.
// The lookup happens inside the first call made on each device, so make that first call
// outside of any stream capture.
//
// Sharing: all calls on a device use the same array.  It keeps whatever the previous
// call left in it; nothing in it has to start at zero, because every word a call reads
// (table entries up to the sizes of this call, partials up to this call's grid) is
// written earlier in the same call.  Two calls that overlap on the GPU (different
// streams, or different host threads without ordering) race on the array: serialise
// them on one stream or with events.
#include <mutex>
#include "common.cuh"

#define ZKH_STATIC_MAX_V 28
#define ZKH_STATIC_TBL_LOG 14
#define ZKH_STATIC_MAX_CTAS 2048
#define ZKH_STATIC_WORDS ((2u << ZKH_STATIC_TBL_LOG) + ZKH_STATIC_MAX_CTAS)
#define ZKH_STATIC_MAX_DEVICES 64

// words [0, 2^14): low-variable factor table; [2^14, 2^15): high-variable factor table;
// [2^15, 2^15 + 2048): per-CTA partial sums
static __device__ __align__(256) unsigned long long zkh_static_scratch[ZKH_STATIC_WORDS];

namespace {

struct StaticPoint { gl_t z[ZKH_STATIC_MAX_V]; };

// table[b] = prod_i (b_i ? z[v0+i] : 1 - z[v0+i]); the low table uses variables [0,vl),
// the high table [vl, vl+vh).  One launch fills both.
__global__ void static_tables_kernel(StaticPoint pt, uint32_t vl, uint32_t vh, gl_t* lo, gl_t* hi) {
    uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t nl = 1u << vl, nh = 1u << vh;
    if (t >= nl + nh) return;
    const bool high = t >= nl;
    const uint32_t b = high ? t - nl : t, v0 = high ? vl : 0, nv = high ? vh : vl;
    gl_t p = 1;
    for (uint32_t i = 0; i < nv; i++) {
        gl_t zi = pt.z[v0 + i];
        p = gl_mul(p, ((b >> i) & 1) ? zi : gl_sub(1, zi));
    }
    (high ? hi : lo)[b] = p;
}
// partials[cta] = sum over this CTA's elements of c[b] * lo[b & mask] * hi[b >> vl]
__global__ void __launch_bounds__(256)
static_dot_kernel(const gl_t* __restrict__ c, const gl_t* __restrict__ lo, const gl_t* __restrict__ hi,
                  uint32_t vl, size_t n, gl_t* partials) {
    __shared__ gl_t sh[32];
    Acc192 acc;
    acc.clear();
    const size_t stride = (size_t)gridDim.x * blockDim.x * 2;
    const size_t mask = ((size_t)1 << vl) - 1;
    for (size_t b = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 2; b < n; b += stride) {
        ulonglong2 cv = ld2(c + b);
        gl_t h = hi[b >> vl];
        acc.add_prod(cv.x, gl_mul(lo[b & mask], h));
        acc.add_prod(cv.y, gl_mul(lo[(b + 1) & mask], h));
    }
    gl_t s[1] = {acc.reduce()};
    block_sum<1>(s, sh);
    if (threadIdx.x == 0) partials[blockIdx.x] = s[0];
}
__global__ void static_sum_kernel(const gl_t* partials, uint32_t n, gl_t* out) {
    __shared__ gl_t sh[32];
    gl_t s[1] = {0};
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) s[0] = gl_add(s[0], partials[i]);
    block_sum<1>(s, sh);
    if (threadIdx.x == 0) *out = s[0];
}
__global__ void static_copy1_kernel(const gl_t* c, gl_t* out) { *out = c[0]; }

std::mutex g_mu;
gl_t* g_base[ZKH_STATIC_MAX_DEVICES] = {nullptr};

int fail(char* errbuf, size_t cap, int code, const char* msg, const char* detail = "") {
    if (errbuf && cap) snprintf(errbuf, cap, "%s%s", msg, detail);
    return code;
}

}  // namespace

extern "C" int zkh_gl_mle_eval_static(void* stream, const uint64_t* c_dev, const uint64_t* z, uint32_t v,
                                      uint64_t* y_dev, char* errbuf, size_t errbuf_len) {
    if (!c_dev || !y_dev || (v && !z)) return fail(errbuf, errbuf_len, ZKH_ERR_ARG, "mle_eval_static: null pointer");
    if (v > ZKH_STATIC_MAX_V)
        return fail(errbuf, errbuf_len, ZKH_ERR_LIMIT,
                    "mle_eval_static: at most 28 variables (2^28 coefficients) fit the fixed scratch array; "
                    "use zkh_gl_mle_eval for larger inputs");
    for (uint32_t i = 0; i < v; i++)
        if (z[i] >= GL_P) return fail(errbuf, errbuf_len, ZKH_ERR_ARG, "mle_eval_static: point not canonical");
    if (v && ((uintptr_t)c_dev & 15))
        return fail(errbuf, errbuf_len, ZKH_ERR_ARG, "mle_eval_static: the column must be 16-byte aligned (128-bit loads)");
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(errbuf, errbuf_len, ZKH_ERR_CUDA, "cudaGetDevice: ", cudaGetErrorString(e));
    if (dev < 0 || dev >= ZKH_STATIC_MAX_DEVICES)
        return fail(errbuf, errbuf_len, ZKH_ERR_LIMIT, "mle_eval_static: device ordinal beyond 63");
    gl_t* base;
    {
        // set-up, once per device, with that device current: resolve the array's device address
        std::lock_guard<std::mutex> lk(g_mu);
        if (!g_base[dev]) {
            void* p = nullptr;
            e = cudaGetSymbolAddress(&p, zkh_static_scratch);
            if (e != cudaSuccess || !p)
                return fail(errbuf, errbuf_len, ZKH_ERR_CUDA, "cudaGetSymbolAddress(zkh_static_scratch): ",
                            cudaGetErrorString(e));
            g_base[dev] = (gl_t*)p;
        }
        base = g_base[dev];
    }
    cudaStream_t s = (cudaStream_t)stream;
    if (v == 0) {
        static_copy1_kernel<<<1, 1, 0, s>>>(c_dev, y_dev);
    } else {
        gl_t* lo = base;
        gl_t* hi = base + (1u << ZKH_STATIC_TBL_LOG);
        gl_t* partials = base + (2u << ZKH_STATIC_TBL_LOG);
        const uint32_t vl = v <= 1 ? v : v / 2, vh = v - vl;  // both <= 14
        StaticPoint pt;
        for (uint32_t i = 0; i < ZKH_STATIC_MAX_V; i++) pt.z[i] = i < v ? z[i] : 0;
        const uint32_t nt = (1u << vl) + (1u << vh);
        static_tables_kernel<<<(nt + 255) / 256, 256, 0, s>>>(pt, vl, vh, lo, hi);
        const size_t n = (size_t)1 << v;
        size_t blocks = (n / 2 + 255) / 256;
        if (blocks > ZKH_STATIC_MAX_CTAS) blocks = ZKH_STATIC_MAX_CTAS;
        static_dot_kernel<<<(unsigned)blocks, 256, 0, s>>>(c_dev, lo, hi, vl, n, partials);
        static_sum_kernel<<<1, 256, 0, s>>>(partials, (uint32_t)blocks, y_dev);
    }
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail(errbuf, errbuf_len, ZKH_ERR_CUDA, "kernel launch: ", cudaGetErrorString(e));
    return ZKH_OK;
}
