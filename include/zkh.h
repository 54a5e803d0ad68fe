/*
 * zkh -- C ABI of the B200 (sm_100a) prover kernels for the Goldilocks /
 * Basefold proving path.
 *
 * Plain pointers and sizes only.  Every function returns ZKH_OK (0) or a
 * negative ZKH_ERR_* code and never throws; zkh_last_error() gives the text.
 * One context per GPU; a context is thread-compatible, not thread-safe.
 * Pointers named *_dev are device addresses on the context's GPU, everything
 * else is host memory.  Field elements are canonical uint64 values in [0, p),
 * p = 2^64 - 2^32 + 1, exactly as the reference stores them.
 * Device columns of two or more elements must start on a 16-byte boundary
 * (the kernels read adjacent pairs with 128-bit loads): the sumcheck, fold,
 * evaluation and batched-opening entry points return ZKH_ERR_ARG for a column
 * that does not, before anything is launched.  Whole allocations and slices at
 * even element offsets qualify.  Function attributes and kernel set-up are kept
 * per device, so one process may hold contexts on several GPUs.
 *
 * Each entry point names the reference interface it stands in for
 * (file:line relative to the reference project root).  Results are
 * bit-identical to that interface on the same inputs.
 */
#ifndef ZKH_H
#define ZKH_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ZKH_OK 0
#define ZKH_ERR_ARG (-1)      /* bad argument (size, functor, null pointer) */
#define ZKH_ERR_CUDA (-2)     /* a CUDA runtime call failed */
#define ZKH_ERR_NOMEM (-3)    /* device allocation failed */
#define ZKH_ERR_DOMAIN (-4)   /* e.g. lookup index out of table, zero denominator */
#define ZKH_ERR_LIMIT (-5)    /* size beyond a documented maximum */
#define ZKH_ERR_DEVICE (-6)   /* a kernel reported an internal error flag */

/* Sumcheck summands.  cols = column values at one vertex, par = parameters. */
#define ZKH_F_PROD2 0 /* c0*c1                       nc=2        zkllm-src/p3_basefold.cuh:319-330 */
#define ZKH_F_PROD3 1 /* c0*c1*c2                    nc=3        zkllm-src/p3_int_gadgets.cuh:539-544 */
#define ZKH_F_GKR 2   /* c0*(c1*c4+c2*c3+p0*c3*c4)   nc=5 par=1  zkllm-src/p3_gkr.cuh:48-53 */
#define ZKH_F_LOGUP 3 /* p0*c0+c2*(c0*(c1+p1)-c3)    nc=4 par=2  zkllm-src/p3_logup.cuh:49-54 */

#define ZKH_F_IRS1 4  /* c0*(c1+p0-c2*p1-c3)           nc=4 par=2  zkllm-src/p3_int_gadgets.cuh:316-325 (one limb) */
#define ZKH_F_IRS2 5  /* c0*(c1+p0-c2*p1-c3-65536*c4)  nc=5 par=2  same, two limbs */
/* Quartic constraint summands of the fp8 matmul gadget (zkh_sumcheck_wide only; nt = 5).  Column and
 * constraint order as in zkllm-src/p3_hawkeye.cuh:87-101 and :850-1010; lam = the random coefficients. */
#define ZKH_F_HW_DP 6  /* per-product alignment      nc=12 nlam=6   F_dp  p3_hawkeye.cuh:850-864 */
#define ZKH_F_HW_DG 7  /* per-group accumulate       nc=30 nlam=18  F_dg  p3_hawkeye.cuh:866-895 */
#define ZKH_F_HW_CH 8  /* group state chain          nc=11 nlam=6   F_ch  p3_hawkeye.cuh:897-905 */
#define ZKH_F_HW_GS 9  /* group sum + attainment     nc=3  nlam=2   F_gs  p3_hawkeye.cuh:907-909 */
#define ZKH_F_HW_DS 10 /* per-row scale decomposition nc=8 nlam=6   F_ds  p3_hawkeye.cuh:915-927 */
#define ZKH_F_HW_DO 11 /* per-output float pipeline  nc=57 nlam=49  F_do  p3_hawkeye.cuh:929-1010 */
/* (the reference's F_y, p3_hawkeye.cuh:911-913, is ZKH_F_PROD3) */

#if defined(__GNUC__)
#define ZKH_API __attribute__((visibility("default")))
#else
#define ZKH_API
#endif

typedef struct zkh_ctx zkh_ctx;

/* ---- context ---- */
/* Creates a context on `device`.  stream == NULL: the context makes its own
 * non-blocking stream; otherwise work is queued on the given cudaStream_t. */
ZKH_API int zkh_ctx_create(int device, void* stream, zkh_ctx** out);
ZKH_API void zkh_ctx_destroy(zkh_ctx* ctx);
ZKH_API int zkh_ctx_set_stream(zkh_ctx* ctx, void* stream);
ZKH_API int zkh_ctx_sync(zkh_ctx* ctx);
/* Frees the context's scratch workspace (it grows to the largest call made so far and is otherwise kept until the
 * context is destroyed); the next call that needs scratch allocates again.  Synchronises the stream first. */
ZKH_API int zkh_ctx_release_workspace(zkh_ctx* ctx);
ZKH_API const char* zkh_last_error(const zkh_ctx* ctx);
ZKH_API const char* zkh_version(void);

/* Device time of the largest launch of the dominant kernel inside the most recent
 * proving call on this context (CUDA events on the context's stream), with the
 * algorithmic bytes that launch moved.  Measurement aid; no reference counterpart
 * (the reference times phases on the host, zkllm-src/p3_basefold.cuh:348-349). */
ZKH_API int zkh_profile_last(zkh_ctx* ctx, float* ms, uint64_t* bytes, const char** kernel);

/* ---- device memory (stands in for p3bf::dmalloc / cudaMallocAsync use,
 *      zkllm-src/p3_basefold.cuh:50-72) ---- */
/* Stream-ordered on the context's stream, from the device's default memory pool (freed blocks stay in the pool until
 * zkh_ctx_release_workspace trims it): a block is usable by work queued on that stream after the call, and after zkh_dev_free
 * it is reused only by work queued later on that stream. */
ZKH_API int zkh_dev_alloc(zkh_ctx* ctx, size_t bytes, void** out_dev);
ZKH_API int zkh_dev_free(zkh_ctx* ctx, void* ptr_dev);
/* Page-locked host memory (uploads from it need no staging copy). */
ZKH_API int zkh_host_alloc(zkh_ctx* ctx, size_t bytes, void** out);
ZKH_API int zkh_host_free(zkh_ctx* ctx, void* ptr);
ZKH_API int zkh_upload(zkh_ctx* ctx, void* dst_dev, const void* src, size_t bytes);
ZKH_API int zkh_download(zkh_ctx* ctx, void* dst, const void* src_dev, size_t bytes);

/* ---- Fiat-Shamir transcript on the host (zkllm-src/fs_transcript.hpp:115-166;
 *      challenge mapping zkllm-src/p3_scgpu.cuh:31-35, p3_fri.cuh:422-426).
 *      The state is the 32-byte running digest. ---- */
ZKH_API void zkh_tr_init(uint8_t state[32], const void* seed, size_t seed_len);
ZKH_API void zkh_tr_absorb(uint8_t state[32], const char* label, const void* data, uint64_t len);
ZKH_API void zkh_tr_challenge_bytes(uint8_t state[32], uint8_t out[32]);
ZKH_API uint64_t zkh_tr_chal(uint8_t state[32]);
ZKH_API uint64_t zkh_tr_idx(uint8_t state[32], uint64_t mod);
/* Merkle hashes of the commitment trees, on the host (p3fri::leaf_hash / node_hash, zkllm-src/p3_fri.cuh:33-39): a leaf is
 * SHA-256 of the 8-byte little-endian value; a node is ONE compression of left | right from the standard initial state,
 * without a padding block (p3_sha256_compress64, zkllm-src/p3_merkle.cuh:69-109).  What a verifier needs to check paths. */
ZKH_API void zkh_merkle_leaf_hash(uint64_t value, uint8_t out[32]);
ZKH_API void zkh_merkle_node_hash(const uint8_t left[32], const uint8_t right[32], uint8_t out[32]);

/* ---- multilinear vector kernels ---- */
/* out_dev[b] = eq(b, z), b < 2^v.          zkllm-src/p3_basefold.cuh:247-252 (p3bf_eq_kernel) */
ZKH_API int zkh_gl_eq_build(zkh_ctx* ctx, const uint64_t* z, uint32_t v, uint64_t* out_dev);
/* *y = sum_b c[b]*eq(b,z).                 zkllm-src/p3_basefold.cuh:262-273 (eval_h_gpu) */
ZKH_API int zkh_gl_mle_eval(zkh_ctx* ctx, const uint64_t* c_dev, const uint64_t* z, uint32_t v, uint64_t* y);
/* out[i] = in[2i] + a*(in[2i+1]-in[2i]), i < n/2 (the MLE fold).
 *                                          zkllm-src/p3_basefold.cuh:336-339 (p3bf_bind_kernel) */
ZKH_API int zkh_gl_bind(zkh_ctx* ctx, const uint64_t* in_dev, uint64_t* out_dev, uint64_t n, uint64_t a);

/* The same evaluation for callers that cannot allocate device memory: hosts that gave the
 * whole GPU to their own arena, code inside a stream capture (cudaMalloc is illegal there),
 * loops that cannot afford an allocation's device-wide synchronisation.  It calls no
 * cudaMalloc/cudaFree or any allocating routine: its scratch (two eq factor tables and the
 * per-CTA partial sums, 278,528 bytes) is a fixed __device__ array inside the library, which
 * every GPU that runs it holds until the process exits.  Limits and rules:
 *   - v <= 28 variables (2^28 coefficients); larger v returns ZKH_ERR_LIMIT with a message;
 *   - works on the CURRENT device; queues three kernels on `stream` and returns without
 *     synchronising; *y_dev (device memory of the caller) is valid once the stream reaches it;
 *   - the first call on each device resolves the array's device address
 *     (cudaGetSymbolAddress), so make that first call outside of any stream capture;
 *   - all calls on a device share the array; it keeps the previous call's contents and
 *     needs no clearing (each call writes every word it later reads); calls that overlap on
 *     the GPU race on it, so order them on one stream or with events.
 * errbuf (optional, errbuf_len bytes) receives the error text.
 * This entry point has no counterpart in the reference, whose eval_h_gpu allocates four
 * buffers per call (zkllm-src/p3_basefold.cuh:262-273). */
ZKH_API int zkh_gl_mle_eval_static(void* stream, const uint64_t* c_dev, const uint64_t* z, uint32_t v,
                                   uint64_t* y_dev, char* errbuf, size_t errbuf_len);

/* ---- sumcheck prover (zkllm-src/p3_scgpu.cuh:91-160, p3sg::sc_prove_gpu) ----
 * Proves sum_b F(cols(b)) over 2^logn vertices, LSB-first binding.
 * Per round: nt evaluations at t=0..nt-1 are absorbed under `tag` (nt*8 bytes),
 * one challenge is drawn, all columns are bound.  Unlike the reference the input
 * columns are left untouched (rounds run in the context's workspace).
 *   cols_dev[k]  nc device columns of 2^logn elements
 *   par          npar summand parameters (may be NULL when npar == 0)
 *   state        in: transcript state before the first round; out: after the last
 *   msgs         logn*nt values out;  chals: logn values out
 *   finals       nc values out: each column bound at all challenges (may be NULL)
 * nt: 3..5 and at least degree(F)+1. */
ZKH_API int zkh_sumcheck(zkh_ctx* ctx, int functor, int nt, const uint64_t* const* cols_dev, int nc,
                 uint32_t logn, const uint64_t* par, int npar, const char* tag, uint8_t state[32],
                 uint64_t* msgs, uint64_t* chals, uint64_t* finals);
/* Same with HOST columns: uploads, proves, returns (the path sc5_run takes for
 * host-resident witness columns, zkllm-src/p3_hawkeye.cuh:1016-1033). */
ZKH_API int zkh_sumcheck_host(zkh_ctx* ctx, int functor, int nt, const uint64_t* const* cols, int nc,
                      uint32_t logn, const uint64_t* par, int npar, const char* tag,
                      uint8_t state[32], uint64_t* msgs, uint64_t* chals, uint64_t* finals);
/* Bytes of workspace zkh_sumcheck needs for (nc, logn). */
ZKH_API size_t zkh_sumcheck_workspace(int nc, uint32_t logn);

/* Quartic zero-check sumcheck over many device columns: replaces p3hwl::sc5_run<FF> /
 * sc5_prove (zkllm-src/p3_hawkeye.cuh:1016-1033, :641-700; non-zk) for the ZKH_F_HW_* summands.
 * Five evaluations per round (Msg5), messages absorbed under `tag`, columns bound LSB-first; the
 * caller's columns are left untouched.  lam: nlam canonical coefficients (host).  msgs: logn*5 out,
 * chals: logn out, finals: nc out (may be NULL).  nc and nlam must equal the summand's shape. */
ZKH_API int zkh_sumcheck_wide(zkh_ctx* ctx, int functor, const uint64_t* const* cols_dev, int nc, uint32_t logn,
                      const uint64_t* lam, int nlam, const char* tag, uint8_t state[32], uint64_t* msgs,
                      uint64_t* chals, uint64_t* finals);
/* Programmable eq-weighted zero-check: the summand is
 *   col0 * (konst + sum_j coef_j * prod_{k < deg_j} col[idx_jk]),   deg_j in 1..3,
 * the shape of the integer-layer gadgets' constraint polynomials (zkllm-src/p3_int_gadgets.cuh:326, :726,
 * :977-1035, :1307, :1563-1640, :1818), which the reference proves with its host loop p3hwl::sc5_prove
 * (non-zk path of sc5z).  Five evaluations per round (Msg5), absorbed under `tag`.
 * prog: word 0 = number of terms (<= 2048), word 1 = konst, then per term two words: coefficient,
 * degree | idx0 << 8 | idx1 << 16 | idx2 << 24.  nwords = 2 + 2*terms.  1 <= nc <= 224.
 * A term whose degree byte has bit 7 set (degree | 0x80) is added OUTSIDE the col0 factor: with it the summand of a
 * blinded chain, F + rho*(B1 + E*B2 + E^2*B3 + E^3*B4) with E = col0 (zkllm-src/p3_hawkeye.cuh:1035-1053, :1333-1341),
 * is one program.
 * Programs of more than 32 columns or 120 terms (the bf16 gadgets of the fp8 transformer layer, zkllm-src/p3_bfadd.cuh:
 * 214-330, p3_swiglu.cuh:172-207 and siblings) run on a variant that keeps the column values in shared memory. */
ZKH_API int zkh_sumcheck_zerocheck(zkh_ctx* ctx, const uint64_t* const* cols_dev, int nc, uint32_t logn,
                           const uint64_t* prog, int nwords, const char* tag, uint8_t state[32], uint64_t* msgs,
                           uint64_t* chals, uint64_t* finals);
/* The same chain under a structured Libra blind g(x) = sum_j g_j(x_j), g_j of degree 4 (zkllm-src/p3_hawkeye.cuh:1065-1110 sb_fix,
 * :1329-1331): the message of round rd gains A_rd * (pref + g_rd(t)) + B_rd, pref = sum_{i < rd} g_i(a_i), applied on the device
 * before the message is absorbed.  fix: 7 words per round (host): the five coefficients of g_rd, A_rd = rho * 2^(v-1-rd),
 * B_rd = rho * 2^(v-2-rd) * suf[rd+1].  pref_out: g(r) after the last round. */
ZKH_API int zkh_sumcheck_zerocheck_blind(zkh_ctx* ctx, const uint64_t* const* cols_dev, int nc, uint32_t logn,
                                 const uint64_t* prog, int nwords, const uint64_t* fix, const char* tag, uint8_t state[32],
                                 uint64_t* msgs, uint64_t* chals, uint64_t* finals, uint64_t* pref_out);
/* The first `rounds` rounds of such a chain when its later variables belong to other columns (the factored matmul chain of
 * p3imm, whose summand eq * X * W splits over the index groups): messages, challenges and the transcript advance as in the
 * full chain; left receives, column after column, the 2^(logn - rounds) values that remain after the last bind.  fix: NULL or
 * the structured blind's rows of THESE rounds; pref_in / pref_out carry its running prefix from one partial chain to the next.
 * Programs of the small engine only (<= 32 columns, <= 120 terms). */
ZKH_API int zkh_sumcheck_zerocheck_partial(zkh_ctx* ctx, const uint64_t* const* cols_dev, int nc, uint32_t logn, uint32_t rounds,
                                   const uint64_t* prog, int nwords, const uint64_t* fix, uint64_t pref_in, const char* tag,
                                   uint8_t state[32], uint64_t* msgs, uint64_t* chals, uint64_t* left, uint64_t* pref_out);
/* Column and coefficient counts of a ZKH_F_HW_* summand (ZKH_ERR_ARG for any other id). */
ZKH_API int zkh_sumcheck_wide_shape(int functor, int* nc, int* nlam);

/* ---- sumcheck sharded over several GPUs of one node ----
 * The reference has no multi-GPU code; this is the sharded form of p3sg::sc_prove_gpu
 * (zkllm-src/p3_scgpu.cuh:91-160) with an identical transcript.  The hypercube is split on
 * its top log2(G) variables: GPU g (one context, one process) holds elements
 * [g*2^logn_local, (g+1)*2^logn_local) of every column.  Per local round r = 0..logn_local-1:
 *   zkh_shard_round_local(r, sums_dev)     this GPU's nt round sums -> sums_dev (device)
 *   <caller all-gathers the G*nt values, rank-major, into gathered_dev on every GPU>
 *   zkh_shard_round_combine(r, gathered_dev, G)   mod-p sum, absorb, challenge (same on every GPU)
 * then zkh_shard_finals(finals_dev) gives this GPU's nc bound values; the caller all-gathers
 * them (rank-major [G][nc]) and zkh_shard_residual runs the last log2(G) rounds on every GPU.
 * zkh_shard_end returns the transcript state, (logn_local+log2 G)*nt message values, the
 * challenges and the nc final values -- the same on every GPU and equal to an unsharded proof.
 * Everything between begin and end is stream-ordered; nothing waits on another GPU inside a
 * kernel. */
ZKH_API int zkh_shard_begin(zkh_ctx* ctx, int functor, int nt, const uint64_t* const* cols_dev, int nc,
                            uint32_t logn_local, const uint64_t* par, int npar, const char* tag,
                            const uint8_t state[32]);
/* Peer-to-peer exchange of the round sums (one process per GPU, NVLink peer stores, no NCCL call per round).
 * zkh_p2p_create: allocate this GPU's mailbox, return its 64-byte CUDA IPC handle.  The caller exchanges the
 * handles between ranks and passes all G of them, in rank order, to zkh_p2p_connect on every rank (collective:
 * all ranks must connect before any of them runs a fused round).  zkh_shard_round_fused(r) then runs round r of
 * the running sharded sumcheck as ONE kernel (bind, local sums, peer stores, bounded wait of about a second per
 * round for the other ranks, sum in rank order, absorb, challenge).  A rank that never arrives makes the others
 * return ZKH_ERR_DEVICE from zkh_shard_end; a rank that arrives after another rank's wait ran out is told so by that
 * rank's next flag (a poison bit) and returns ZKH_ERR_DEVICE as well.  After such an error disconnect and connect
 * again on all ranks. */
ZKH_API int zkh_p2p_create(zkh_ctx* ctx, uint8_t handle_out[64]);
ZKH_API int zkh_p2p_connect(zkh_ctx* ctx, uint32_t rank, uint32_t G, const uint8_t* handles);
ZKH_API int zkh_p2p_disconnect(zkh_ctx* ctx);
ZKH_API int zkh_shard_round_fused(zkh_ctx* ctx, uint32_t r);
/* All local rounds after zkh_shard_begin with the peer exchange; the rounds on columns of at most 2^12 elements
 * run inside one single-CTA kernel per GPU.  finals_dev receives this rank's nc bound column values (what
 * zkh_shard_finals would return); continue with the all-gather of those and zkh_shard_residual. */
ZKH_API int zkh_shard_local_fused(zkh_ctx* ctx, uint64_t* finals_dev);
/* The whole sharded proof after zkh_shard_begin with the peer exchange: the local rounds as above, then -- inside the
 * same single-CTA kernel -- one more mailbox exchange that all-gathers every GPU's nc bound values, and the log2(G)
 * residual rounds, which every GPU runs identically.  No collective library call and no host round trip between
 * zkh_shard_begin and zkh_shard_end.  The device waits are bounded (about a second each), so the caller must see that
 * the ranks start within that time of one another (a host rendezvous before the first proof of a series; proofs that
 * follow back to back only have kernel skew between them).  A GPU whose wait ran out marks every later exchange, so
 * the proof ends with ZKH_ERR_DEVICE from zkh_shard_end on every GPU that took part after that point. */
ZKH_API int zkh_shard_prove_fused(zkh_ctx* ctx);
ZKH_API int zkh_shard_round_local(zkh_ctx* ctx, uint32_t r, uint64_t* sums_dev);
ZKH_API int zkh_shard_round_combine(zkh_ctx* ctx, uint32_t r, const uint64_t* gathered_dev, uint32_t G);
ZKH_API int zkh_shard_finals(zkh_ctx* ctx, uint64_t* finals_dev);
ZKH_API int zkh_shard_residual(zkh_ctx* ctx, const uint64_t* gathered_finals_dev, uint32_t G);
ZKH_API int zkh_shard_end(zkh_ctx* ctx, uint8_t state[32], uint64_t* msgs, uint64_t* chals, uint64_t* finals);

/* ---- Reed-Solomon encode / NTT (zkllm-src/p3_ntt.cuh:170-230 P3Ntt::run,
 *      p3_basefold.cuh:188-197 rs_encode_gpu_dev) ----
 * out[k] = sum_j in[j]*w^(jk) over the 2^logn subgroup, natural order in and out; inverse
 * divides by n.  in_dev and out_dev must differ.  Stream-ordered (no host sync). */
ZKH_API int zkh_ntt(zkh_ctx* ctx, const uint64_t* in_dev, uint64_t* out_dev, uint32_t logn, int inverse);
/* Codeword of the 2^v coefficients at rate 2^-R: forward NTT of the zero-padded vector.
 * cw_dev: 2^(v+R) elements.  Stream-ordered. */
ZKH_API int zkh_rs_encode(zkh_ctx* ctx, const uint64_t* c_dev, uint32_t v, uint32_t R, uint64_t* cw_dev);

/* ---- SHA-256 Merkle tree (zkllm-src/p3_fri.cuh:97-178 DeviceMerkle, p3_merkle.cuh:161-207) ----
 * Leaf = SHA-256(8-byte LE element), node = one compression of left|right from the IV.
 * tree_dev (optional, zkh_merkle_tree_bytes(M) bytes) receives all levels: M leaf digests,
 * M/2, ..., root.  root (optional, host) receives the 32-byte root; when given the call
 * synchronises.  With tree_dev == NULL only the root is computed. */
ZKH_API size_t zkh_merkle_tree_bytes(uint64_t M);
ZKH_API int zkh_merkle_build(zkh_ctx* ctx, const uint64_t* cw_dev, uint64_t M, uint8_t* tree_dev, uint8_t root[32]);
/* Authentication paths (zkllm-src/p3_fri.cuh:164-178 paths_batch): for each of the n leaf
 * indices, log2(M) sibling digests from the leaf level up; out: n*log2(M)*32 bytes (host). */
ZKH_API int zkh_merkle_paths(zkh_ctx* ctx, const uint8_t* tree_dev, uint64_t M, const uint32_t* idx, uint32_t n,
                             uint8_t* out);

/* ---- Basefold ---- */
/* MLE fold of a codeword of length M with challenge beta:
 * out[c] = (1-beta)*(f[c]+f[c+M/2])/2 + beta*(f[c]-f[c+M/2])/(2*w^c), w the primitive M-th root.
 * (zkllm-src/p3_basefold.cuh:239-245 p3bf_fold_kernel, p3_fri.cuh:396-415.)  Stream-ordered. */
ZKH_API int zkh_gl_fold_codeword(zkh_ctx* ctx, const uint64_t* f_dev, uint64_t* out_dev, uint64_t M, uint64_t beta);
/* Commitment root of the 2^v device coefficients at rate 2^-R (zkllm-src/p3_basefold.cuh:210-227
 * commit_gpu_rootonly).  cw_dev (optional, 2^(v+R) elements) keeps the codeword. */
ZKH_API int zkh_basefold_commit(zkh_ctx* ctx, const uint64_t* c_dev, uint32_t v, uint32_t R, uint64_t* cw_dev,
                                uint8_t root[32]);
/* Same from HOST coefficients (upload inside), as the reference's entry point takes them. */
ZKH_API int zkh_basefold_commit_host(zkh_ctx* ctx, const uint64_t* coeffs, uint32_t v, uint32_t R, uint8_t root[32]);
/* Evaluation opening (zkllm-src/p3_basefold.cuh:355-420 prove_eval_dev): proves y = c~(z).
 * cw0_dev: the committed codeword (2^(v+R) elements) or NULL to re-encode here.
 * The proof is serialised little-endian as
 *   u32 logN, R, Q | roots v*32 | messages v*24 | final word 2^R*8 |
 *   per query, per round r: a(8) b(8) path_a((v+R-r)*32) path_b((v+R-r)*32) | z v*8 | y 8
 * (the fields of p3bf::EvalProof in declaration order); *written = zkh_basefold_proof_size. */
ZKH_API size_t zkh_basefold_proof_size(uint32_t v, uint32_t R, uint32_t Q);
ZKH_API int zkh_basefold_open(zkh_ctx* ctx, const uint64_t* c_dev, const uint64_t* z, uint32_t v, uint64_t y,
                              uint32_t R, uint32_t Q, const uint64_t* cw0_dev, const char* seed, uint8_t* out,
                              size_t cap, size_t* written);

/* Batched opening of one size class, non-zk (zkllm-src/p3_batchopen.cuh:307-1147 p3bo::prove_class).
 * Ledger of k claims over columns of 2^v rows: entry j = (cols_dev[j], roots + 32*j, zid[j]) claims the
 * column committed under that root at point pts[zid[j]] (T points of v coordinates, host).  Entries
 * with equal roots are one column (deduplicated by first appearance, like the reference).
 * state: the MAIN transcript, in/out (mu, "bo-rm" rounds, "bo-ys", rho are drawn/absorbed on it); the
 * opening itself runs on a fresh transcript seeded with `label`, as in the reference.
 * The proof is the fields of p3bo::BatchProof in declaration order (zk fields omitted):
 *   u32 v, R, Q, nc | ystar nc*8 | rmsgs v*24 | roots (v-1)*32 | omsgs v*24 | final 2^R*8 |
 *   per query, per round r = 1..v-1: a(8) b(8) path_a((v+R-r)*32) path_b((v+R-r)*32) |
 *   per distinct column: u32 nvals, vals nvals*8, u32 nnodes, nodes nnodes*32
 * cap must be at least zkh_batchopen_proof_bound(v, R, Q, number of distinct columns <= k). */
ZKH_API size_t zkh_batchopen_proof_bound(uint32_t v, uint32_t R, uint32_t Q, uint32_t ncols);
ZKH_API int zkh_batchopen_prove_class(zkh_ctx* ctx, uint32_t v, const uint64_t* pts, uint32_t T,
                                      const uint64_t* const* cols_dev, const uint8_t* roots, const uint32_t* zid,
                                      uint32_t k, uint32_t R, uint32_t Q, const char* label, uint8_t state[32],
                                      uint8_t* out, size_t cap, size_t* written);
/* Commitment that keeps its codeword (2^(v+R) elements) and its CAPPED Merkle tree (zkh_basefold_kept_tree_bytes(v+R)
 * bytes) in caller-owned device buffers, and the batched opening that reads them: with 180 GB of HBM a prover can keep
 * the trees of a whole layer resident, so prove_class no longer re-encodes and re-hashes every opened column as the
 * reference does (zkllm-src/p3_batchopen.cuh:393-445 resolves and rebuilds them).  Proof bytes are unchanged.
 * A capped tree holds the levels from 64 leaves per node upwards in the layout of zkh_merkle_build (for fewer than 256
 * leaves: the whole tree): 9 bytes per codeword element together with the codeword instead of 72; the lowest six
 * siblings of an opened path are recomputed from 64 codeword elements (191 compressions per opened leaf).
 * kept_cw[j] / kept_tree[j]: buffers of entry j's column, or NULL to recompute that column. */
ZKH_API size_t zkh_basefold_kept_tree_bytes(uint32_t logM);
ZKH_API int zkh_basefold_commit_keep(zkh_ctx* ctx, const uint64_t* c_dev, uint32_t v, uint32_t R, uint64_t* cw_dev,
                             uint8_t* tree_dev, uint8_t root[32]);
ZKH_API int zkh_batchopen_prove_class_kept(zkh_ctx* ctx, uint32_t v, const uint64_t* pts, uint32_t T,
                                   const uint64_t* const* cols_dev, const uint8_t* roots, const uint32_t* zid,
                                   uint32_t k, uint32_t R, uint32_t Q, const char* label, uint8_t state[32],
                                   uint8_t* out, size_t cap, size_t* written, const uint64_t* const* kept_cw,
                                   const uint8_t* const* kept_tree);

/* Batched opening of the hiding mode (zkllm-src/p3_batchopen.cuh:969-1131, the zk_salted branches of p3bo::prove_class):
 * every column of the class was committed with zkh_basefold_commit_salted under sseeds[j] (equal roots carry equal seeds).
 * The protocol is the one above; each distinct column's round-0 section becomes
 *   u32 nvals, vals nvals*8, salts nvals*32, u32 nnodes, nodes nnodes*32
 * (BQ0C vals / salts / nodes).  The class blinder (one fresh uniform salted column claimed at a fresh point, its root and
 * claim absorbed under "bo-blr" / "bo-bly", :315-384) is an ordinary ledger entry the caller appends before the call.
 * cap: zkh_batchopen_proof_bound(...) + distinct columns * 2*Q*32.  kept_cw / kept_tree as above (arrays or NULL). */
ZKH_API int zkh_batchopen_prove_class_salted(zkh_ctx* ctx, uint32_t v, const uint64_t* pts, uint32_t T,
                                     const uint64_t* const* cols_dev, const uint8_t* roots, const uint32_t* zid,
                                     const uint64_t* sseeds, uint32_t k, uint32_t R, uint32_t Q, const char* label,
                                     uint8_t state[32], uint8_t* out, size_t cap, size_t* written,
                                     const uint64_t* const* kept_cw, const uint8_t* const* kept_tree);

/* Roots of k independent columns (2^vs[j] elements each) with one host synchronisation; roots: k*32 bytes (host).  The bytes
 * equal k calls of zkh_basefold_commit (zkllm-src/p3_basefold.cuh:210-227 commit_gpu_rootonly). */
ZKH_API int zkh_basefold_commit_many(zkh_ctx* ctx, const uint64_t* const* cols_dev, const uint32_t* vs, uint32_t k, uint32_t R,
                             uint8_t* roots);
/* Hiding commitment: salted Merkle leaves (zkllm-src/p3_zkc.cuh:230-292 salt_of / salted_leaf / p3zkc_salted_leaf_kernel,
 * :320-397 salted_commit_root, salted_commit_root_dev).  Leaf i = SHA-256(value_le8 | SHA-256(sseed_le8 | i_le8)); internal
 * nodes as in the plain tree, so authentication paths verify unchanged.  cw_dev (2^(v+R) elements) and tree_dev
 * (capped: zkh_basefold_kept_tree_bytes(v+R) bytes) are optional; a kept tree needs the kept codeword. */
ZKH_API int zkh_basefold_commit_salted(zkh_ctx* ctx, const uint64_t* c_dev, uint32_t v, uint32_t R, uint64_t sseed,
                               uint64_t* cw_dev, uint8_t* tree_dev, uint8_t root[32]);

/* Randomness of the hiding mode (zkllm-src/p3_zkc.cuh:100-123 zprng / zprng_at, :471-534 zprng_fill / zprng_fill_at /
 * blind_col_aug_dev, :158-185 fresh_mask_into / augment).  Stream-ordered.
 *   zkh_zk_fill_at     out[i] = zprng_at(seed, i0 + i): the random-access stream of blind columns
 *   zkh_zk_fill_chain  out[i] = element k0 + i of the zprng chain started at state s0 (element 0 = first output)
 *   zkh_zk_augment     out = [col (2^v) | mask slices ((2^e - 1) * 2^v chain elements from mask_seed)]; mask_seed 0
 *                      gives zero slices (the reference's masks-off control) */
ZKH_API int zkh_zk_fill_at(zkh_ctx* ctx, uint64_t seed, uint64_t i0, uint64_t n, uint64_t* out_dev);
ZKH_API int zkh_zk_fill_chain(zkh_ctx* ctx, uint64_t s0, uint64_t k0, uint64_t n, uint64_t* out_dev);
ZKH_API int zkh_zk_augment(zkh_ctx* ctx, const uint64_t* col_dev, uint32_t v, uint32_t e, uint64_t mask_seed, uint64_t* out_dev);

/* ---- logUp ---- */
/* Multiplicities: cnt_dev[j] = #{i : idx_dev[i] == j}, j < M (zkllm-src/p3_logup.cuh:149-172,
 * host loop :1412-1475).  An index >= M returns ZKH_ERR_DOMAIN (the reference throws). */
ZKH_API int zkh_histogram(zkh_ctx* ctx, const uint32_t* idx_dev, uint64_t n, uint32_t M, uint64_t* cnt_dev);
/* out[i] = 1/(A[i]+beta) by batched inversion (zkllm-src/p3_logup.cuh:636-660 inv_all_add).
 * A zero denominator returns ZKH_ERR_DOMAIN ("resample beta" in the reference). */
ZKH_API int zkh_gl_inv_all_add(zkh_ctx* ctx, const uint64_t* A_dev, uint64_t n, uint64_t beta, uint64_t* out_dev);
/* out[i] = sum_k g^k * cols[k][i] (zkllm-src/p3_logup.cuh:663-672 combine).  Stream-ordered. */
ZKH_API int zkh_gl_combine(zkh_ctx* ctx, const uint64_t* const* cols_dev, int ncols, uint64_t n, uint64_t g,
                           uint64_t* out_dev);
/* out[i] = addend + sum_k g^k * cols[k][i]: the gamma-combination with the logUp shift folded in
 * (leaf denominators A_i + beta of zkllm-src/p3_logup.cuh:1645-1647, :1788-1789).  ncols = 0 fills out with the
 * constant addend (padding members of a merged lookup, all-ones numerators).  Stream-ordered. */
ZKH_API int zkh_gl_affine(zkh_ctx* ctx, const uint64_t* const* cols_dev, int ncols, uint64_t n, uint64_t g,
                          uint64_t addend, uint64_t* out_dev);
/* Dense field helpers for binding one index group of a committed matrix M (rows x cols, row-major):
 * along_rows != 0: out[r] = sum_c M[r][c]*w[c] (rows values); else out[c] = sum_r w[r]*M[r][c] (cols values).
 * They replace the 2^(lj+lk+li) broadcast columns that p3imm::prove materialises on the host
 * (zkllm-src/p3_int_gadgets.cuh:574-593): the matmul summand EQ*X*W factors over the index groups,
 * so its round messages come from these partial evaluations (see p3.imm_prove).  Stream-ordered. */
ZKH_API int zkh_gl_matvec(zkh_ctx* ctx, const uint64_t* M_dev, uint64_t rows, uint64_t cols, const uint64_t* w_dev,
                          int along_rows, uint64_t* out_dev);
/* C = A * B over the field, row-major, A: I x J, B: J x K (device): the product of the operands' first mask slices that links the
 * mask of a matmul accumulator in hiding mode (zkllm-src/p3_int_gadgets.cuh:510-527 accum_mask1, a host triple loop there).
 * Stream-ordered. */
ZKH_API int zkh_gl_matmul(zkh_ctx* ctx, const uint64_t* A_dev, const uint64_t* B_dev, uint64_t I, uint64_t J, uint64_t K,
                          uint64_t* C_dev);
/* Exact integer matrix products of the integer decoder layer's witness chain: p3itf::build_witness computes the seven
 * weight matmuls and the per-head score / attention-output products on the host (zkllm-src/p3_int_layer.cuh:182-318 over
 * p3imm::matmul_i64, p3_int_gadgets.cuh:493-508).  For every batch entry (b0, b1), b0 < nb0, b1 < nb1:
 *     C[b0][b1][i][k] = sum_j A[b0][b1][i][j] * B[b0][b1][j][k],   i < I, j < J, k < K,
 * where X[b0][b1][r][c] is the element at X_dev + b0*s[0] + b1*s[1] + r*s[2] + c*s[3] (element strides), so the per-head
 * slices of the (batch, position, head, lane) activations are addressed in place.  Operands and results are field
 * elements standing for signed integers (v, or p - |v|); operands must lie in (-2^24, 2^24) (ZKH_ERR_DOMAIN otherwise)
 * and J <= 2^15, so every sum is exact in 64 bits.  Synchronises the stream (it reports the range check). */
ZKH_API int zkh_ig_matmul(zkh_ctx* ctx, const uint64_t* A_dev, const int64_t a_strides[4], const uint64_t* B_dev,
                          const int64_t b_strides[4], uint64_t* C_dev, const int64_t c_strides[4], uint32_t nb0,
                          uint32_t nb1, uint32_t I, uint32_t J, uint32_t K);
/* Witness replays of the integer layer's gadgets on the device (the host loops of p3iadd / p3iswg / p3irope / p3irms /
 * p3ismx ::gen_witness, zkllm-src/p3_int_gadgets.cuh:690-710, :1738-1788, :1228-1273, :830-916, :1416-1512, and the RS20 row
 * index of p3itf::build_witness).  Columns are field-lifted signed integers; index arrays are uint32 lookup rows.  A value
 * outside a gadget's window returns ZKH_ERR_DOMAIN (the reference throws).  Each call synchronises the stream.
 *   add:      out = a + b, idx = out + 2^19
 *   rs20:     idx = v + 2^19
 *   swiglu:   sil = SILU[g + 2^19] (silu_col: the table's value column, 2^20 rows), m = sil * u, mo = round(m / 2^16),
 *             rem = m + 2^15 - mo * 2^16; idxG = g + 2^19, idxRem = rem, idxMo = mo + 2^19
 *   rope:     q over (2^lT positions x 2^ld lanes), heads of 2^ldh lanes, cos / sin: int32 tables [2^lseq][2^(ldh-1)] at scale
 *             2^14; y = round((q C + q' S2) / 2^14), q' = the partner lane of the rotate-half, C / S2 the signed public columns
 *   rms:      per row M = 2^14 + sum x^2 ... the 18 per-row columns db (order p3irms::B_*), W / remW / remY per element, y, and
 *             the lookup rows: irow = e, m, m - 2^14, m, L40 L41 L42 D40 D41 D42 L20 D20 LR0, LR1; iel = remW, W + 2^19, remY, Y + 2^19
 *   softmax:  rows of 2^lseq keys, 2^(la+lseq) rows, causal; xe = first, dm, E, r1 lo, r1 hi, r2 lo, r2 hi; xb = mx, S per row;
 *             p; idxDM, idxL[4] per element, idxMX = mx + 2^15 per row (expt_col: the EXPT table's value column, 2^17 rows) */
/* Signed integers (|v| < 2^63 for the 64-bit form) -> field elements v or p - |v| (p3ig::gsig, zkllm-src/p3_int_gadgets.cuh:57):
 * weights and activations as a loader keeps them, and the int64 public columns the RoPE replay returns.  in == out is allowed for
 * the 64-bit form.  Stream-ordered. */
ZKH_API int zkh_gl_lift_i32(zkh_ctx* ctx, const int32_t* in_dev, uint64_t n, uint64_t* out_dev);
ZKH_API int zkh_gl_lift_i64(zkh_ctx* ctx, const int64_t* in_dev, uint64_t n, uint64_t* out_dev);
ZKH_API int zkh_ig_add_witness(zkh_ctx* ctx, const uint64_t* a_dev, const uint64_t* b_dev, uint64_t n, uint64_t* out_dev,
                               uint32_t* idx_dev);
ZKH_API int zkh_ig_rs20_index(zkh_ctx* ctx, const uint64_t* v_dev, uint64_t n, uint32_t* idx_dev);
ZKH_API int zkh_ig_swiglu_witness(zkh_ctx* ctx, const uint64_t* g_dev, const uint64_t* u_dev, const uint64_t* silu_col_dev, uint64_t n,
                                  uint64_t* sil_dev, uint64_t* rem_dev, uint64_t* mo_dev, uint32_t* idxG_dev, uint32_t* idxRem_dev,
                                  uint32_t* idxMo_dev);
ZKH_API int zkh_ig_rope_witness(zkh_ctx* ctx, const uint64_t* q_dev, const int32_t* cos_dev, const int32_t* sin_dev, uint32_t lseq,
                                uint32_t ldh, uint32_t lT, uint32_t ld, uint64_t* y_dev, uint64_t* rem_dev, uint32_t* idxRem_dev,
                                uint32_t* idxY_dev, int64_t* c_dev, int64_t* s2_dev);
ZKH_API int zkh_ig_rms_witness(zkh_ctx* ctx, const uint64_t* x_dev, const uint64_t* g_dev, const uint64_t* isq_col_dev, uint32_t lT,
                               uint32_t ld, uint64_t* const db_dev[18], uint64_t* const de_dev[3], uint64_t* y_dev,
                               uint32_t* const irow_dev[14], uint32_t* const iel_dev[4]);
ZKH_API int zkh_ig_softmax_witness(zkh_ctx* ctx, const uint64_t* z_dev, const uint64_t* expt_col_dev, uint32_t la, uint32_t lseq,
                                   uint64_t* const xe_dev[7], uint64_t* const xb_dev[2], uint64_t* p_dev, uint32_t* idxDM_dev,
                                   uint32_t* const idxL_dev[4], uint32_t* idxMX_dev);
/* out[i] = a[i]*b[i]: the helper column hT = cnt * 1/(Tc+beta) of the standalone lookup
 * (zkllm-src/p3_logup.cuh:984).  Stream-ordered. */
ZKH_API int zkh_gl_mul(zkh_ctx* ctx, const uint64_t* a_dev, const uint64_t* b_dev, uint64_t n, uint64_t* out_dev);
/* out[i] = s*in[i].  Stream-ordered. */
ZKH_API int zkh_gl_scale(zkh_ctx* ctx, const uint64_t* in_dev, uint64_t n, uint64_t s, uint64_t* out_dev);
/* Operand views as maps on index bits (p3imm::op_off / y_off, zkllm-src/p3_int_gadgets.cuh:448-470, and the broadcast
 * columns of the hiding mode): idx(u) = konst | OR over the set bits b < nbits of u of masks[b]  (nbits <= 32, n <= 2^nbits).
 * gather: out[u] = col[idx(u)] for u < n (every idx must lie below col_len, else ZKH_ERR_DOMAIN and nothing runs);
 * scatter: out[idx(u)] = vals[u] (idx below out_len; the map must be injective, other entries of out keep their value).
 * Stream-ordered. */
ZKH_API int zkh_gl_gather_bits(zkh_ctx* ctx, const uint64_t* col_dev, uint64_t col_len, uint64_t n, uint64_t konst,
                               const uint64_t* masks, uint32_t nbits, uint64_t* out_dev);
ZKH_API int zkh_gl_scatter_bits(zkh_ctx* ctx, const uint64_t* vals_dev, uint64_t n, uint64_t konst, const uint64_t* masks,
                                uint32_t nbits, uint64_t* out_dev, uint64_t out_len);
/* out[u] = col[u ^ xor_mask] for u < n (n a power of two, xor_mask < n): the rotate-half partner column of the RoPE gadget
 * (zkllm-src/p3_int_gadgets.cuh:1297-1298).  Stream-ordered. */
ZKH_API int zkh_gl_gather_xor(zkh_ctx* ctx, const uint64_t* col_dev, uint64_t n, uint64_t xor_mask, uint64_t* out_dev);
/* p3ismx::mask_col (zkllm-src/p3_int_gadgets.cuh:1490-1498): out[u] = 1 where key index j <= query index i over
 * u = j | i << lseq | a << 2*lseq, 2^(la + 2*lseq) elements.  Stream-ordered. */
ZKH_API int zkh_ig_causal_mask(zkh_ctx* ctx, uint32_t la, uint32_t lseq, uint64_t* out_dev);
/* Rescale witness (zkllm-src/p3_int_gadgets.cuh:230-275 p3irs::gen_witness): for each signed acc value
 * y = floor((acc + 2^(sf-1)) / 2^sf), remainder limbs L0 (16 bits), L1 (sf > 16 only), and the lookup row
 * indices of the limbs and of y in its window (rng 1: [-2^19,2^19), rng 2: [-2^15,2^15), rng 0: none).
 * y outside the window returns ZKH_ERR_DOMAIN ("y out of range" in the reference). */
ZKH_API int zkh_irs_witness(zkh_ctx* ctx, const uint64_t* acc_dev, uint64_t n, uint32_t sf, int rng, uint64_t* y_dev,
                            uint64_t* L0_dev, uint64_t* L1_dev, uint32_t* idxL0_dev, uint32_t* idxL1_dev,
                            uint32_t* idxY_dev);
/* GKR fractional-sum tree prover (zkllm-src/p3_gkr.cuh:200-364 p3gkr::prove / prove_dev).
 * p_dev, q_dev: 2^L leaf numerators / denominators (left untouched, unlike prove_dev which
 * takes ownership).  state: transcript in/out.  rfin: L values (combine_last) or L-1.
 * cpq: (p~(rfin), q~(rfin)) when combine_last.  Proof serialised as
 *   P(8) Q(8) | per layer h = L..1: u32 rounds, rounds*32 message bytes, p0 p1 q0 q1 (32)
 * (p3gkr::Proof / Lay in declaration order).  A zero root denominator returns ZKH_ERR_DOMAIN. */
ZKH_API size_t zkh_gkr_proof_size(uint32_t L);
ZKH_API int zkh_gkr_prove(zkh_ctx* ctx, const uint64_t* p_dev, const uint64_t* q_dev, uint32_t L, int combine_last,
                          const char* tag, uint8_t state[32], uint64_t* rfin, uint64_t cpq[2], uint8_t* out,
                          size_t cap, size_t* written);

/* Witness of the fp8 (Hawkeye) matmul gadget: the exact replay of the fp8 forward pass that p3hwl::gen_witness runs as a host
 * loop (zkllm-src/p3_hawkeye.cuh:342-637), as one kernel with a warp per output.  Padded grids: 2^lb rows of X, 2^ln rows of
 * W, 2^lg groups of 32 products (lg covers one phantom group after the last real one), K padded to 32*2^lg.
 *   xcodes_dev  2^lb * 32*2^lg fp8-e4m3 codes of X as field elements, row-major (zero beyond the real grid)
 *   wcodes_dev  2^ln * 32*2^lg codes of W;  xsb_dev / wsb_dev: 2^lb / 2^ln fp32 bit patterns of the per-row scales
 *   cols_dev    99 output columns in the order dp[10] (2^(lb+ln+lg+5) elements each, index ((g*2^(lb+ln) + b*2^ln + n)*32 + kk),
 *               dg[29] (2^(lb+ln+lg)), dob[46] (2^(lb+ln)), db[6] (2^lb), dn[6] (2^ln), va, vb (product domain): the columns of
 *               LayerWit in the reference's enum order (p3_hawkeye.cuh:86-101)
 *   lidx_dev    38 uint32 lookup-index columns in the order of the reference's LU_* enum (p3_hawkeye.cuh:104-112)
 * A layer outside the gadget's supported domain returns ZKH_ERR_DOMAIN with the message the reference throws. */
ZKH_API int zkh_hwl_witness(zkh_ctx* ctx, uint32_t lb, uint32_t ln, uint32_t lg, const uint64_t* xcodes_dev,
                            const uint64_t* wcodes_dev, const uint64_t* xsb_dev, const uint64_t* wsb_dev,
                            uint64_t* const* cols_dev, uint32_t* const* lidx_dev);

/* Host-side construction of the integer layer's function tables (p3ig::build_tables,
 * zkllm-src/p3_int_gadgets.cuh:99-118): kind 0 EXPT (2^17 rows), 1 SILU (2^20 rows), 2 ISQ (2^16 rows, uses d).
 * col0 / col1: host arrays of that many field elements.  No GPU involved. */
ZKH_API int zkh_ig_table(int kind, uint32_t d, uint64_t* col0, uint64_t* col1);

/* ======================================================================================
 * BLS12-381 scalar field (Fr) back-end: the reference's first proof stack.
 * An element is the reference's Fr_t (zkllm-src/bls12-381.cuh:116-120): eight 32-bit limbs, little
 * endian, 32 bytes, holding a PLAIN canonical integer below
 *   p = 0x73eda753299d7d483339d80809a1d80553bda402fffe5bfeffffffff00000001
 * (the reference keeps tensors plain and converts around each Montgomery product).  Device arrays
 * must be 16-byte aligned.  Points and challenges are host arrays of 32-byte elements.
 * ====================================================================================== */

/* E[b] = prod_i (bit_i(b) ? u[i] : 1 - u[i]), 2^v entries: build_eq_tensor / k_eq_expand
 * (zkllm-src/zkob_lookup.cuh:202-212, :247-268). */
ZKH_API int zkh_fr_eq_build(zkh_ctx* ctx, const void* u, uint32_t v, void* out_dev);
/* out[i] = in[i] + w*(in[i+h] - in[i]), i < h: k_fr_fold (zkllm-src/zkob_lookup.cuh:285-293 call sites).  out_dev may equal
 * in_dev (every element is read by the thread that overwrites it, before it does). */
ZKH_API int zkh_fr_fold(zkh_ctx* ctx, const void* in_dev, uint64_t h, const void* w, void* out_dev);
/* FrTensor::partial_me (zkllm-src/fr-tensor.cu:542-561, :601-632) for a power-of-two dimension:
 * t viewed as [other][2^logd][window]; out[o][w] = sum_d eq(u, d) * t[o][d][w], u[0] bound first.
 * One pass over t instead of logd passes with intermediates. */
ZKH_API int zkh_fr_partial_me(zkh_ctx* ctx, const void* t_dev, uint64_t other, uint32_t logd, uint64_t window,
                      const void* u, void* out_dev);
/* FrTensor::operator()(u) / Fr_me (zkllm-src/fr-tensor.cu:578-600): the multilinear extension of the
 * 2^v-element t at u (u[0] pairs adjacent elements).  out32: 32 bytes, host. */
ZKH_API int zkh_fr_mle_eval(zkh_ctx* ctx, const void* t_dev, const void* u, uint32_t v, void* out32);
/* Product sumcheck over nc (2..4) device columns of 2^logn elements, binding the TOP variable first
 * (pairs (i, i+h)), nt = nc+1 evaluations per round at t = 0..nc:
 *   nc=2  the inner-product rounds of zkob_fc   (zkllm-src/zkob_fc.cu:290-332; labels "p0","p1","p2")
 *   nc=3  fs_hadamard                            (zkllm-src/zkob_lookup.cuh:297-318; "hp0".."hp3")
 *   nc=4  the bracket sumcheck fs_quartic        (zkllm-src/zkob_lookup.cuh:321-425)
 * Per round: each evaluation is absorbed as 32 bytes under labels[t], then the challenge is drawn as
 * fs_challenge_fr does (zkllm-src/vrf_common.cuh:233-244).  The columns are left untouched.
 *   state   transcript in/out;  evals: logn*nt*32 bytes out;  chals: logn*32 bytes out (round order);
 *   finals  nc*32 bytes out: every column bound at all challenges (may be NULL). */
/* out[i] += c * in[i] over n elements: k_bo_axpy of the batch opening (zkllm-src/zkob_claims.cuh:386-391).  c32: one scalar, host.
 * Stream-ordered. */
ZKH_API int zkh_fr_axpy(zkh_ctx* ctx, void* out_dev, const void* in_dev, const void* c32, uint64_t n);
/* out[i] = a[i] * b[i] over n elements, out may alias an input: FrTensor::operator* (zkllm-src/fr-tensor.cu:141-147, :343-350).
 * Stream-ordered. */
ZKH_API int zkh_fr_mul(zkh_ctx* ctx, void* out_dev, const void* a_dev, const void* b_dev, uint64_t n);
/* The three round evaluations (t = 0, 1, 2) of sum_x a(x) b(x) with the top variable free: sum over i < h of
 * (a[i] + t (a[i+h] - a[i])) (b[i] + t (b[i+h] - b[i])): k_bo_hp2 plus its three sums (zkllm-src/zkob_claims.cuh:365-384, :930-937).
 * out96: three scalars, host; the call synchronises the stream. */
ZKH_API int zkh_fr_round_sums(zkh_ctx* ctx, const void* a_dev, const void* b_dev, uint64_t h, void* out96);
/* sum_i a[i]*b[i]: (B * m).sum() of the lookup set-up (zkllm-src/zkob_rescale.cu:137).  out32: 32 bytes, host. */
ZKH_API int zkh_fr_dot(zkh_ctx* ctx, const void* a_dev, const void* b_dev, uint64_t n, void* out32);
/* out[i] = 1/(in[i] + beta), 0 where in[i] + beta = 0: tlookup_inv_kernel (zkllm-src/tlookup.cu:50-62), with one
 * Fermat inversion per eight elements instead of one per element. */
ZKH_API int zkh_fr_inv_add(zkh_ctx* ctx, const void* in_dev, uint64_t n, const void* beta, void* out_dev);
/* The logUp sumcheck of the reference's first stack: fs_phase1 + fs_phase2 (zkllm-src/zkob_lookup.cuh:143-198) over
 * tLookup_phase1/2_step_poly (zkllm-src/tlookup.cu:184-296).  A, S: 2^logD entries (A = 1/(S+beta)); B, T, m: 2^logN
 * entries (B = 1/(T+beta), table, multiplicities); logN <= logD.  alpha, beta, Cc (= alpha^2 - sum B*m) and the
 * point u (logD entries) are host values.  Per round the four evaluations p(0..3) are absorbed under "p0".."p3"
 * and the challenge is drawn as fs_challenge_fr does.  Out (host): evals logD*4*32 bytes, ws logD*32 bytes (round
 * order), terminals 5*32 bytes (A_f, S_f, B_f, T_f, m_f).  The columns are left untouched. */
ZKH_API int zkh_fr_lookup_sumcheck(zkh_ctx* ctx, const void* A_dev, const void* S_dev, const void* B_dev, const void* T_dev,
                           const void* m_dev, uint32_t logD, uint32_t logN, const void* alpha, const void* beta,
                           const void* Cc, const void* u, uint8_t state[32], void* evals, void* ws, void* terminals);
/* Measured rate of Montgomery products on this GPU in 10^9 per second (four independent chains per
 * thread, grid = 8 CTAs per SM): the integer-pipe ceiling the Fr kernels are read against, as
 * zkllm-src/p3_field_bench.cu does for its two fields. */
ZKH_API int zkh_fr_mul_throughput(zkh_ctx* ctx, uint32_t iters, double* gmul_per_s);
ZKH_API int zkh_fr_sumcheck(zkh_ctx* ctx, const void* const* cols_dev, int nc, uint32_t logn,
                    const char* const* labels, uint8_t state[32], void* evals, void* chals, void* finals);

/* ---- BLS12-381 G1: Pedersen row commitments of the first proof stack (zkllm-src/commitment.cu:41-103,
 *      Commitment::commit -> commit_pippenger) ----
 * out[r] = sum_i scalars[r][i] * gens[i] for m rows of n scalars.  gens, out: the reference's G1Jacobian_t (144 bytes: X, Y, Z,
 * each twelve 32-bit limbs in Montgomery form); scalars: the reference's Fr_t (32 bytes), whose RAW limbs are the multiplier,
 * as in the reference.  The sums are formed in the reference's order (4-bit windows, buckets filled in generator order,
 * running sum from bucket 15, Horner from the top window), so the Jacobian triples equal the reference's byte for byte.
 * All buffers on the device, 16-byte aligned.  Stream-ordered. */
ZKH_API int zkh_g1_pedersen_commit(zkh_ctx* ctx, const void* gens_dev, const void* scalars_dev, uint32_t m, uint32_t n, void* out_dev);

/* ---- BLS12-381 G1: openings of the first proof stack (zkllm-src/vrf_common.cuh) ----
 * Points are the reference's G1Jacobian_t (144 bytes), scalars its Fr_t (32 bytes, plain integers below the modulus).  The
 * proof files hold Jacobian triples, so every point below is produced by the reference's own sequence of additions and
 * doublings (G1Jacobian_mul from the lowest bit up, zkllm-src/g1-tensor.cu:445-453; dev_msm's halving sums) and equals the
 * reference's byte for byte.  Device buffers 16-byte aligned; results are returned to host memory and the calls synchronise
 * the stream before they return.
 *
 * zkh_g1_msm: <g, a> over n points, n a power of two: dev_msm (vrf_common.cuh:165-184).
 * zkh_g1_fold_chain: fold_chain (vrf_common.cuh:144-163): nu pair folds of `size` points with the challenges us (host, nu
 *   scalars); orientation 0 = c[2i] + u (c[2i+1] - c[2i]) (k_com_me, :52-58), 1 = c[2i+1] + u (c[2i] - c[2i+1]) (k_gen_fold,
 *   :59-65); odd levels are padded with a record of zero bytes as the reference pads them.  out144 = element 0 after the folds.
 * zkh_g1_ipa_prove: ipa_prove (vrf_common.cuh:302-336), the Fiat-Shamir inner-product argument for P = <g, a> + <a, b> Q:
 *   log2(n) rounds of L, R under the labels "L", "R", challenge by the reference's limb mapping, folds of a, b, g.  a_dev,
 *   b_dev: n scalars; g_dev: n points; Q144: host.  state: the caller's transcript state, advanced in place.  L_out, R_out: host,
 *   log2(n) points each; a_final32: host.  The whole argument runs on the device (transcript included): no host round trip per
 *   round.
 * zkh_g1_ipa_verify: ipa_verify (vrf_common.cuh:340-371): replays the transcript, folds P0 with x^2 L + P + x^-2 R, the public
 *   weights me_weights(u_b) (log2(n) scalars, host) and the generators (through the s-vector product), and sets *accept to 1 iff
 *   P == a_f g_f + (a_f b_f) Q as group elements.  A rejected proof is ZKH_OK with *accept = 0. */
/* *n_bad = the number of rows j < rows with lhs[j] != s a[j] + b[j] as group elements: the homomorphic affine link of the
 * rescaling obligation (zkllm-src/zkob_rescale.cu:226-241, com_X[j] == sf com_Xr[j] + com_rem[j]).  s32: one scalar, host. */
ZKH_API int zkh_g1_rows_check(zkh_ctx* ctx, const void* lhs_dev, const void* a_dev, const void* s32, const void* b_dev, uint32_t rows,
                              uint32_t* n_bad);
/* out[j] = a[j] + b[j] for j < rows: the homomorphic sum of two commitment vectors (hom_add, zkllm-src/zkob_skip.cu:39-48), each
 * sum the reference's Jacobian triple.  Stream-ordered; out_dev may not overlap the inputs. */
ZKH_API int zkh_g1_rows_add(zkh_ctx* ctx, const void* a_dev, const void* b_dev, uint32_t rows, void* out_dev);
/* out[j] = s a[j] + b[j] for j < rows, each the reference's Jacobian triple: hb_addmul (zkllm-src/zkob_fastg1.cuh:56-92), the
 * combined commitment com_G + r com_S of the mapping-lookup drivers; mul_first selects the operand order of the addition
 * (1: (s a) + b, 0: b + (s a)).  s32: one scalar, host.  Stream-ordered; out_dev may not overlap the inputs. */
ZKH_API int zkh_g1_rows_lincomb(zkh_ctx* ctx, const void* a_dev, const void* s32, const void* b_dev, uint32_t rows, int mul_first, void* out_dev);
ZKH_API int zkh_g1_msm(zkh_ctx* ctx, const void* g_dev, const void* a_dev, uint32_t n, void* out144);
ZKH_API int zkh_g1_fold_chain(zkh_ctx* ctx, const void* src_dev, uint32_t size, const void* us, uint32_t nu, int orientation,
                              void* out144);
ZKH_API int zkh_g1_ipa_prove(zkh_ctx* ctx, const void* a_dev, const void* b_dev, const void* g_dev, const void* Q144, uint32_t n,
                             uint8_t state[32], void* L_out, void* R_out, void* a_final32);
ZKH_API int zkh_g1_ipa_verify(zkh_ctx* ctx, const void* g_dev, uint32_t n, const void* Q144, const void* P0_144, const void* u_b,
                              const void* L, const void* R, const void* a_final32, uint8_t state[32], int* accept);

#ifdef __cplusplus
}
#endif
#endif
