// Context management, device memory, the host transcript entry points and the
// small multilinear vector kernels (eq table, MLE evaluation, bind).
#include "common.cuh"

using namespace zkh;

#define ZKH_PARTIALS_CAP (148 * 16 * 5)

int zkh_ws_reserve(zkh_ctx* c, size_t bytes) {
    if (bytes <= c->ws_bytes) return ZKH_OK;
    ZKH_CUDA(c, cudaStreamSynchronize(c->stream));
    if (c->ws) cudaFree(c->ws);
    c->ws = nullptr;
    c->ws_bytes = 0;
    size_t want = zkh_align(bytes, (size_t)1 << 21);
    cudaError_t e = cudaMalloc(&c->ws, want);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return zkh_fail(c, ZKH_ERR_NOMEM, "workspace allocation of " + std::to_string(want) + " bytes failed");
    }
    c->ws_bytes = want;
    return ZKH_OK;
}

extern "C" int zkh_ctx_release_workspace(zkh_ctx* c) {
    if (!c) return ZKH_ERR_ARG;
    ZKH_CUDA(c, cudaSetDevice(c->device));
    ZKH_CUDA(c, cudaStreamSynchronize(c->stream));
    if (c->ws) cudaFree(c->ws);
    c->ws = nullptr;
    c->ws_bytes = 0;
    cudaMemPool_t pool;                          // blocks that zkh_dev_free returned to the pool go back to the device
    if (cudaDeviceGetDefaultMemPool(&pool, c->device) == cudaSuccess) cudaMemPoolTrimTo(pool, 0);
    return ZKH_OK;
}

extern "C" const char* zkh_version(void) { return "zkh 0.1 (sm_100a)"; }

extern "C" int zkh_ctx_create(int device, void* stream, zkh_ctx** out) {
    if (!out) return ZKH_ERR_ARG;
    *out = nullptr;
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || device < 0 || device >= ndev) return ZKH_ERR_CUDA;
    if (cudaSetDevice(device) != cudaSuccess) return ZKH_ERR_CUDA;
    zkh_ctx* c = new zkh_ctx();
    c->device = device;
    cudaDeviceGetAttribute(&c->sm_count, cudaDevAttrMultiProcessorCount, device);
    if (c->sm_count <= 0) c->sm_count = ZKH_SM_COUNT_FALLBACK;
    if (stream) {
        c->stream = (cudaStream_t)stream;
    } else {
        if (cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess) { delete c; return ZKH_ERR_CUDA; }
        c->own_stream = true;
    }
    c->partials_cap = ZKH_PARTIALS_CAP;
    if (cudaMalloc(&c->d_ctl, sizeof(ZkhCtl)) != cudaSuccess ||
        cudaMalloc(&c->d_partials, c->partials_cap * sizeof(gl_t)) != cudaSuccess ||
        cudaMallocHost(&c->h_ctl, sizeof(ZkhCtl)) != cudaSuccess) {
        zkh_ctx_destroy(c);
        return ZKH_ERR_NOMEM;
    }
    cudaEventCreate(&c->prof_ev[0]);
    cudaEventCreate(&c->prof_ev[1]);
    cudaMemset(c->d_ctl, 0, sizeof(ZkhCtl));
    memset(c->h_ctl, 0, sizeof(ZkhCtl));
    *out = c;
    return ZKH_OK;
}
extern "C" void zkh_ctx_destroy(zkh_ctx* c) {
    if (!c) return;
    cudaSetDevice(c->device);
    if (c->stream) cudaStreamSynchronize(c->stream);
    zkh_p2p_disconnect(c);
    if (c->p2p.mine) cudaFree(c->p2p.mine);
    if (c->ws) cudaFree(c->ws);
    if (c->d_ctl) cudaFree(c->d_ctl);
    if (c->d_partials) cudaFree(c->d_partials);
    if (c->h_ctl) cudaFreeHost(c->h_ctl);
    for (auto& t : c->tw) {
        if (t.lo) cudaFree(t.lo);
        if (t.lo_inv) cudaFree(t.lo_inv);
    }
    if (c->prof_ev[0]) cudaEventDestroy(c->prof_ev[0]);
    if (c->prof_ev[1]) cudaEventDestroy(c->prof_ev[1]);
    if (c->own_stream && c->stream) cudaStreamDestroy(c->stream);
    delete c;
}
extern "C" int zkh_ctx_set_stream(zkh_ctx* c, void* stream) {
    if (!c) return ZKH_ERR_ARG;
    ZKH_CUDA(c, cudaStreamSynchronize(c->stream));
    if (c->own_stream) { cudaStreamDestroy(c->stream); c->own_stream = false; }
    if (stream) {
        c->stream = (cudaStream_t)stream;
    } else {
        ZKH_CUDA(c, cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
        c->own_stream = true;
    }
    return ZKH_OK;
}
extern "C" int zkh_ctx_sync(zkh_ctx* c) {
    if (!c) return ZKH_ERR_ARG;
    ZKH_CUDA(c, cudaStreamSynchronize(c->stream));
    return ZKH_OK;
}
extern "C" const char* zkh_last_error(const zkh_ctx* c) { return c ? c->err.c_str() : "null context"; }

extern "C" int zkh_profile_last(zkh_ctx* c, float* ms, uint64_t* bytes, const char** kernel) {
    if (!c || !ms || !bytes) return ZKH_ERR_ARG;
    if (!c->prof_valid) return zkh_fail(c, ZKH_ERR_ARG, "profile: the last call had no timed launch");
    ZKH_CUDA(c, cudaEventSynchronize(c->prof_ev[1]));
    ZKH_CUDA(c, cudaEventElapsedTime(ms, c->prof_ev[0], c->prof_ev[1]));
    *bytes = c->prof_bytes;
    if (kernel) *kernel = c->prof_kernel;
    return ZKH_OK;
}

// Device memory for host code that has no allocator of its own (the C++ host side): stream-ordered allocations from the
// device's default memory pool, whose release threshold is raised once per device so that freed blocks stay in the pool
// and a prover that allocates hundreds of short-lived columns per proof does not pay a cudaMalloc / cudaFree (each a
// device-wide synchronisation) for every one of them.  zkh_ctx_release_workspace trims the pool.
extern "C" int zkh_dev_alloc(zkh_ctx* c, size_t bytes, void** out) {
    if (!c || !out) return ZKH_ERR_ARG;
    ZKH_CUDA(c, cudaSetDevice(c->device));
    static ZkhOncePerDevice pool_set;
    zkh_once_on_device(pool_set, c->device, [c] {
        cudaMemPool_t pool;
        if (cudaDeviceGetDefaultMemPool(&pool, c->device) == cudaSuccess) {
            uint64_t keep = UINT64_MAX;
            cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
        }
    });
    cudaError_t e = cudaMallocAsync(out, bytes ? bytes : 1, c->stream);
    if (e != cudaSuccess) {
        cudaGetLastError();
        *out = nullptr;
        return zkh_fail(c, ZKH_ERR_NOMEM, "device allocation of " + std::to_string(bytes) + " bytes failed");
    }
    return ZKH_OK;
}
extern "C" int zkh_dev_free(zkh_ctx* c, void* p) {
    if (!c) return ZKH_ERR_ARG;
    if (!p) return ZKH_OK;
    ZKH_CUDA(c, cudaFreeAsync(p, c->stream));      // reusable once the stream has passed this point
    return ZKH_OK;
}
// page-locked host memory for inputs that are uploaded every proof (weights as a loader keeps them)
extern "C" int zkh_host_alloc(zkh_ctx* c, size_t bytes, void** out) {
    if (!c || !out) return ZKH_ERR_ARG;
    ZKH_CUDA(c, cudaSetDevice(c->device));
    if (cudaMallocHost(out, bytes ? bytes : 1) != cudaSuccess) {
        cudaGetLastError();
        *out = nullptr;
        return zkh_fail(c, ZKH_ERR_NOMEM, "page-locked host allocation of " + std::to_string(bytes) + " bytes failed");
    }
    return ZKH_OK;
}
extern "C" int zkh_host_free(zkh_ctx* c, void* p) {
    if (!c) return ZKH_ERR_ARG;
    if (p) ZKH_CUDA(c, cudaFreeHost(p));
    return ZKH_OK;
}
extern "C" int zkh_upload(zkh_ctx* c, void* dst, const void* src, size_t bytes) {
    if (!c || (bytes && (!dst || !src))) return ZKH_ERR_ARG;
    ZKH_CUDA(c, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, c->stream));
    ZKH_CUDA(c, cudaStreamSynchronize(c->stream));
    return ZKH_OK;
}
extern "C" int zkh_download(zkh_ctx* c, void* dst, const void* src, size_t bytes) {
    if (!c || (bytes && (!dst || !src))) return ZKH_ERR_ARG;
    ZKH_CUDA(c, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, c->stream));
    ZKH_CUDA(c, cudaStreamSynchronize(c->stream));
    return ZKH_OK;
}

// ---------------------------------------------------------------- host transcript
extern "C" void zkh_tr_init(uint8_t state[32], const void* seed, size_t n) {
    // SHA-256 of an arbitrary-length seed string
    uint32_t h[8];
    sha256_iv(h);
    const uint8_t* p = (const uint8_t*)seed;
    size_t off = 0;
    uint8_t blk[128];
    for (; off + 64 <= n; off += 64) {
        uint32_t w[16];
        for (int i = 0; i < 16; i++)
            w[i] = ((uint32_t)p[off + 4 * i] << 24) | ((uint32_t)p[off + 4 * i + 1] << 16) |
                   ((uint32_t)p[off + 4 * i + 2] << 8) | (uint32_t)p[off + 4 * i + 3];
        sha256_compress(h, w);
    }
    size_t rem = n - off;
    memset(blk, 0, sizeof blk);
    memcpy(blk, p + off, rem);
    blk[rem] = 0x80;
    size_t padded = rem < 56 ? 64 : 128;
    uint64_t bits = (uint64_t)n * 8;
    for (int i = 0; i < 8; i++) blk[padded - 1 - i] = (uint8_t)(bits >> (8 * i));
    for (size_t o = 0; o < padded; o += 64) {
        uint32_t w[16];
        for (int i = 0; i < 16; i++)
            w[i] = ((uint32_t)blk[o + 4 * i] << 24) | ((uint32_t)blk[o + 4 * i + 1] << 16) |
                   ((uint32_t)blk[o + 4 * i + 2] << 8) | (uint32_t)blk[o + 4 * i + 3];
        sha256_compress(h, w);
    }
    digest_to_bytes(h, state);
}
extern "C" void zkh_tr_absorb(uint8_t state[32], const char* label, const void* data, uint64_t len) {
    // streaming form: no length limit on the host
    size_t ll = strlen(label);
    std::string m;
    m.reserve(32 + 4 + ll + 8 + (size_t)len);
    m.append((const char*)state, 32);
    uint8_t b4[4] = {(uint8_t)ll, (uint8_t)(ll >> 8), (uint8_t)(ll >> 16), (uint8_t)(ll >> 24)};
    m.append((const char*)b4, 4);
    m.append(label, ll);
    uint8_t b8[8];
    for (int i = 0; i < 8; i++) b8[i] = (uint8_t)(len >> (8 * i));
    m.append((const char*)b8, 8);
    m.append((const char*)data, (size_t)len);
    zkh_tr_init(state, m.data(), m.size());
}
extern "C" void zkh_tr_challenge_bytes(uint8_t state[32], uint8_t out[32]) {
    uint32_t st[8], o[8];
    digest_from_bytes(state, st);
    tr_challenge(st, o);
    digest_to_bytes(st, state);
    digest_to_bytes(o, out);
}
extern "C" uint64_t zkh_tr_chal(uint8_t state[32]) {
    uint32_t st[8];
    digest_from_bytes(state, st);
    gl_t a = tr_chal_gl(st);
    digest_to_bytes(st, state);
    return a;
}
extern "C" uint64_t zkh_tr_idx(uint8_t state[32], uint64_t mod) {
    uint32_t st[8];
    digest_from_bytes(state, st);
    uint64_t a = tr_chal_idx(st, mod);
    digest_to_bytes(st, state);
    return a;
}

extern "C" void zkh_merkle_leaf_hash(uint64_t value, uint8_t out[32]) {
    uint32_t h[8];
    sha256_leaf(value, h);
    digest_to_bytes(h, out);
}
extern "C" void zkh_merkle_node_hash(const uint8_t left[32], const uint8_t right[32], uint8_t out[32]) {
    uint32_t l[8], r[8], h[8];
    digest_from_bytes(left, l);
    digest_from_bytes(right, r);
    sha256_node(l, r, h);
    digest_to_bytes(h, out);
}

// ---------------------------------------------------------------- eq table
// eq(b,z) = prod_i (b_i ? z_i : 1-z_i) factors over a split of the variables:
// eq(b) = lo[b & (2^vl-1)] * hi[b >> vl].  The two small tables cost O(sqrt N * v);
// the full table is then one multiply per element instead of the v multiplies
// per element of zkllm-src/p3_basefold.cuh:247-252.
__global__ void eq_small_kernel(const gl_t* z, uint32_t v0, uint32_t nv, gl_t* out) {
    uint32_t b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= (1u << nv)) return;
    gl_t p = 1;
    for (uint32_t i = 0; i < nv; i++) {
        gl_t zi = z[v0 + i];
        p = gl_mul(p, ((b >> i) & 1) ? zi : gl_sub(1, zi));
    }
    out[b] = p;
}
__global__ void __launch_bounds__(256)
eq_expand_kernel(const gl_t* __restrict__ lo, const gl_t* __restrict__ hi, uint32_t vl, gl_t* out, size_t n) {
    const size_t stride = (size_t)gridDim.x * blockDim.x * 2;
    const size_t mask = ((size_t)1 << vl) - 1;
    for (size_t b = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 2; b < n; b += stride) {
        gl_t h = hi[b >> vl];
        st2(out + b, gl_mul(lo[b & mask], h), gl_mul(lo[(b + 1) & mask], h));
    }
}
// y-partials of sum_b c[b]*lo[b&mask]*hi[b>>vl]
__global__ void __launch_bounds__(256)
dot_eq_kernel(const gl_t* __restrict__ c, const gl_t* __restrict__ lo, const gl_t* __restrict__ hi,
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
__global__ void sum_partials_kernel(const gl_t* partials, uint32_t n, gl_t* out) {
    __shared__ gl_t sh[32];
    gl_t s[1] = {0};
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) s[0] = gl_add(s[0], partials[i]);
    block_sum<1>(s, sh);
    if (threadIdx.x == 0) *out = s[0];
}

// Two factor tables of eq(.,z) in `scratch` (eq_scratch_bytes(v)); z is a host pointer.
size_t zkh::eq_scratch_bytes(uint32_t v) {
    uint32_t vl = v <= 1 ? v : v / 2;
    if (vl > 14) vl = 14;
    return zkh_align(((size_t)8) << vl) + zkh_align(((size_t)8) << (v - vl)) + zkh_align((size_t)64 * 8);
}
static int eq_tables(zkh_ctx* c, const uint64_t* z, uint32_t v, void* scratch, gl_t** lo, gl_t** hi, uint32_t* vl_out,
                     bool z_on_device = false) {
    uint32_t vl = v <= 1 ? v : v / 2;
    if (vl > 14) vl = 14;
    uint32_t vh = v - vl;
    if (v > 40) return zkh_fail(c, ZKH_ERR_LIMIT, "eq: more than 40 variables");
    size_t tl = zkh_align(((size_t)8) << vl), th = zkh_align(((size_t)8) << vh);
    *lo = (gl_t*)scratch;
    *hi = (gl_t*)((char*)scratch + tl);
    gl_t* dz = (gl_t*)((char*)scratch + tl + th);
    *vl_out = vl;
    // the point is staged in pageable memory by the runtime, so z may be reused by the caller at once
    if (z_on_device) dz = (gl_t*)z;
    else ZKH_CUDA(c, cudaMemcpyAsync(dz, z, (size_t)v * 8, cudaMemcpyHostToDevice, c->stream));
    eq_small_kernel<<<((1u << vl) + 255) / 256, 256, 0, c->stream>>>(dz, 0, vl, *lo);
    eq_small_kernel<<<((1u << vh) + 255) / 256, 256, 0, c->stream>>>(dz, vl, vh, *hi);
    ZKH_CUDA(c, cudaGetLastError());
    return ZKH_OK;
}
int zkh::eq_enqueue(zkh_ctx* c, const uint64_t* z, uint32_t v, gl_t* out_dev, void* scratch, bool z_on_device) {
    if (v == 0) {
        static const uint64_t one = 1;
        ZKH_CUDA(c, cudaMemcpyAsync(out_dev, &one, 8, cudaMemcpyHostToDevice, c->stream));
        return ZKH_OK;
    }
    gl_t *lo, *hi;
    uint32_t vl;
    ZKH_TRY(eq_tables(c, z, v, scratch, &lo, &hi, &vl, z_on_device));
    size_t n = (size_t)1 << v;
    size_t blocks = (n / 2 + 255) / 256, cap = (size_t)c->sm_count * 8;
    eq_expand_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, c->stream>>>(lo, hi, vl, out_dev, n);
    ZKH_CUDA(c, cudaGetLastError());
    return ZKH_OK;
}

extern "C" int zkh_gl_eq_build(zkh_ctx* c, const uint64_t* z, uint32_t v, uint64_t* out_dev) {
    if (!c || !out_dev || (v && !z)) return zkh_fail(c, ZKH_ERR_ARG, "eq_build: null pointer");
    if (v > 40) return zkh_fail(c, ZKH_ERR_LIMIT, "eq_build: more than 40 variables");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    ZKH_TRY(zkh_ws_reserve(c, eq_scratch_bytes(v)));
    ZKH_TRY(eq_enqueue(c, z, v, out_dev, c->ws));
    ZKH_CUDA(c, cudaStreamSynchronize(c->stream));
    return ZKH_OK;
}

extern "C" int zkh_gl_mle_eval(zkh_ctx* c, const uint64_t* c_dev, const uint64_t* z, uint32_t v, uint64_t* y) {
    if (!c || !c_dev || !z || !y) return zkh_fail(c, ZKH_ERR_ARG, "mle_eval: null pointer");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    if (v == 0) return zkh_download(c, y, c_dev, 8);
    if (v > 40) return zkh_fail(c, ZKH_ERR_LIMIT, "mle_eval: more than 40 variables");
    if ((uintptr_t)c_dev & 15) return zkh_fail(c, ZKH_ERR_ARG, "mle_eval: the column must be 16-byte aligned (it is read with 128-bit loads)");
    gl_t *lo, *hi;
    uint32_t vl;
    ZKH_TRY(zkh_ws_reserve(c, eq_scratch_bytes(v)));
    ZKH_TRY(eq_tables(c, z, v, c->ws, &lo, &hi, &vl));
    size_t n = (size_t)1 << v;
    size_t blocks = (n / 2 + 255) / 256, cap = (size_t)c->sm_count * 8;
    unsigned g = (unsigned)(blocks < cap ? blocks : cap);
    dot_eq_kernel<<<g, 256, 0, c->stream>>>(c_dev, lo, hi, vl, n, c->d_partials);
    sum_partials_kernel<<<1, 256, 0, c->stream>>>(c->d_partials, g, c->d_ctl->aux);
    ZKH_CUDA(c, cudaGetLastError());
    ZKH_CUDA(c, cudaMemcpyAsync(c->h_ctl->aux, c->d_ctl->aux, 8, cudaMemcpyDeviceToHost, c->stream));
    ZKH_CUDA(c, cudaStreamSynchronize(c->stream));
    *y = c->h_ctl->aux[0];
    return ZKH_OK;
}

// ---------------------------------------------------------------- bind (MLE fold)
// out[i] = in[2i] + a*(in[2i+1]-in[2i]); each thread folds two adjacent pairs:
// two 128-bit loads, one 128-bit store, 12 bytes of traffic per input element.
__global__ void __launch_bounds__(256)
bind_kernel(const gl_t* __restrict__ in, gl_t* __restrict__ out, size_t quads, gl_t a) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < quads; i += stride) {
        ulonglong2 x = ld2(in + 4 * i), y = ld2(in + 4 * i + 2);
        st2(out + 2 * i, gl_lerp(x.x, x.y, a), gl_lerp(y.x, y.y, a));
    }
}
__global__ void bind_small_kernel(const gl_t* in, gl_t* out, size_t half, gl_t a) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < half) out[i] = gl_lerp(in[2 * i], in[2 * i + 1], a);
}
extern "C" int zkh_gl_bind(zkh_ctx* c, const uint64_t* in_dev, uint64_t* out_dev, uint64_t n, uint64_t a) {
    if (!c || !in_dev || !out_dev) return zkh_fail(c, ZKH_ERR_ARG, "bind: null pointer");
    if (n < 2 || (n & (n - 1))) return zkh_fail(c, ZKH_ERR_ARG, "bind: n must be a power of two >= 2");
    if (a >= GL_P) return zkh_fail(c, ZKH_ERR_ARG, "bind: challenge not canonical");
    if (n >= 4 && (((uintptr_t)in_dev | (uintptr_t)out_dev) & 15))
        return zkh_fail(c, ZKH_ERR_ARG, "bind: columns must be 16-byte aligned (128-bit loads and stores)");
    ZKH_CUDA(c, cudaSetDevice(c->device));
    if (n < 4) {
        bind_small_kernel<<<1, 32, 0, c->stream>>>(in_dev, out_dev, n / 2, a);
    } else {
        size_t quads = n / 4, blocks = (quads + 255) / 256, cap = (size_t)c->sm_count * 8;
        bind_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, c->stream>>>(in_dev, out_dev, quads, a);
    }
    ZKH_CUDA(c, cudaGetLastError());
    return ZKH_OK;
}

// Public lookup tables of the integer layer whose entries come from double-precision functions
// (zkllm-src/p3_int_gadgets.cuh:99-118).  They are part of the proof statement (the table hash is absorbed),
// so they are computed here on the host with the same libm calls and roundings:
//   kind 0  EXPT  2^17 rows  (t, round(2^16 exp(-t/2^8)) for t < 2^16, else 0)
//   kind 1  SILU  2^20 rows  (x, round(2^16 silu(x/2^16))) for x = j - 2^19, both as field elements
//   kind 2  ISQ   2^16 rows  (m, round(2^32 sqrt(d/m)), 0 for m = 0)
#include <cmath>
extern "C" int zkh_ig_table(int kind, uint32_t d, uint64_t* col0, uint64_t* col1) {
    if (!col0 || !col1) return ZKH_ERR_ARG;
    auto lift = [](long long x) { return x >= 0 ? (uint64_t)x : GL_P - (uint64_t)(-x); };
    if (kind == 0) {
        for (size_t j = 0; j < ((size_t)1 << 17); j++) {
            col0[j] = j;
            col1[j] = j < 65536 ? (uint64_t)llround(65536.0 * exp(-(double)j / 256.0)) : 0;
        }
    } else if (kind == 1) {
        for (size_t j = 0; j < ((size_t)1 << 20); j++) {
            const long long xi = (long long)j - (1LL << 19);
            const double xr = (double)xi / 65536.0;
            col0[j] = lift(xi);
            col1[j] = lift(llround(65536.0 * xr / (1.0 + exp(-xr))));
        }
    } else if (kind == 2) {
        for (size_t j = 0; j < 65536; j++) {
            col0[j] = j;
            col1[j] = j ? (uint64_t)llround(4294967296.0 * sqrt((double)d / (double)j)) : 0;
        }
    } else {
        return ZKH_ERR_ARG;
    }
    return ZKH_OK;
}
