/*
 * CPU oracle for the Goldilocks proving hot path (TEST INFRASTRUCTURE ONLY).
 *
 * This is a plain-C restatement of the algorithms of the reference's "p3"
 * prover stack.  It exists so that the CUDA library can be checked bit for
 * bit on a machine that has no copy of the reference.  It is never linked
 * into, imported by, or called from the product library; only the test
 * suite, the smoke check and the benchmark's CPU-baseline leg may use it.
 *
 * Parity pin: every function below is checked here against the reference's
 * own host code (compiled unchanged into oracle/_ref/libp3ref.so by
 * oracle/Makefile) and against committed golden vectors that were generated
 * from that reference build (tests/golden/make_golden.py).
 *
 * Each function cites the reference file:line (paths relative to the
 * reference project root) whose behaviour it restates.
 */
#ifndef ZKH_ORACLE_H
#define ZKH_ORACLE_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ORC_GL_P 0xFFFFFFFF00000001ULL

/* sumcheck summand ids (same numbering as include/zkh.h) */
enum {
    ORC_F_PROD2 = 0, /* c0*c1                        nc=2 */
    ORC_F_PROD3 = 1, /* c0*c1*c2                     nc=3 */
    ORC_F_GKR   = 2, /* c0*(c1*c4+c2*c3+p0*c3*c4)    nc=5 par=1 */
    ORC_F_LOGUP = 3, /* p0*c0+c2*(c0*(c1+p1)-c3)     nc=4 par=2 */
    ORC_F_IRS1  = 4, /* c0*(c1+p0-c2*p1-c3)          nc=4 par=2 */
    ORC_F_IRS2  = 5  /* c0*(c1+p0-c2*p1-c3-65536*c4) nc=5 par=2 */
};

/* ---- field: zkllm-src/p3_goldilocks.cuh:16-73 ---- */
uint64_t orc_gl_add(uint64_t a, uint64_t b);
uint64_t orc_gl_sub(uint64_t a, uint64_t b);
uint64_t orc_gl_mul(uint64_t a, uint64_t b);
uint64_t orc_gl_pow(uint64_t a, uint64_t e);
uint64_t orc_gl_inv(uint64_t a);
uint64_t orc_gl_root_of_unity(uint32_t logn);

/* ---- hashing: zkllm-src/fs_transcript.hpp:24-99, p3_merkle.cuh:69-104 ---- */
void orc_sha256(const void* data, size_t n, uint8_t out[32]);
void orc_sha256_compress64(const uint8_t in[64], uint8_t out[32]);

/* ---- Fiat-Shamir transcript: zkllm-src/fs_transcript.hpp:115-166 ---- */
void orc_tr_init(uint8_t st[32], const void* seed, size_t n);
void orc_tr_absorb(uint8_t st[32], const char* label, const void* data, uint64_t len);
void orc_tr_challenge_bytes(uint8_t st[32], uint8_t out[32]);
uint64_t orc_tr_chal(uint8_t st[32]);              /* p3_scgpu.cuh:31-35 */
uint64_t orc_tr_idx(uint8_t st[32], uint64_t mod); /* p3_fri.cuh:422-426 */

/* ---- multilinear helpers: zkllm-src/p3_basefold.cuh:125-155, 300-316 ---- */
void orc_build_eq(const uint64_t* z, uint32_t v, uint64_t* out);
uint64_t orc_eval_h(const uint64_t* c, const uint64_t* eq, size_t n);
uint64_t orc_mle_eval(const uint64_t* c, const uint64_t* z, uint32_t v);
uint64_t orc_quad_eval(uint64_t s0, uint64_t s1, uint64_t s2, uint64_t t);
uint64_t orc_cubic_eval(uint64_t s0, uint64_t s1, uint64_t s2, uint64_t s3, uint64_t t);
uint64_t orc_quartic_eval(const uint64_t s[5], uint64_t t);
uint64_t orc_eq_point(const uint64_t* a, const uint64_t* z, uint32_t v);
void orc_bind_lsb(uint64_t* f, size_t n, uint64_t a); /* in place, result in f[0..n/2) */

/* ---- generic sumcheck prover: zkllm-src/p3_scgpu.cuh:91-160,
 *      p3_hawkeye.cuh:659-695, p3_logup.cuh:679-729 ----
 * cols[k] has 2^logn entries and is bound in place (destroyed).
 * msgs: logn*nt values; chals: logn values; finals: nc values (may be NULL).
 * nthreads <= 1 runs serially.  Returns 0 on success. */
int orc_sumcheck(uint8_t st[32], const char* tag, int functor, int nt,
                 uint64_t** cols, int nc, uint32_t logn, const uint64_t* par,
                 uint64_t* msgs, uint64_t* chals, uint64_t* finals, int nthreads);

/* ---- Reed-Solomon encode: zkllm-src/p3_basefold.cuh:162-172 (Horner form),
 *      p3_ntt.cuh:210-230 (same codeword, natural order) ---- */
void orc_rs_encode_horner(const uint64_t* c, uint32_t v, uint32_t R, uint64_t* cw);
void orc_rs_encode(const uint64_t* c, uint32_t v, uint32_t R, uint64_t* cw);
void orc_ntt(uint64_t* a, uint32_t logn, int inverse); /* in place, natural order */

/* ---- Merkle tree: zkllm-src/p3_fri.cuh:33-91 ----
 * tree holds all levels back to back: level 0 (M leaf hashes), level 1 (M/2) ...
 * total (2M-1)*32 bytes. */
void orc_leaf_hash(uint64_t v, uint8_t out[32]);
void orc_zprng_fill(uint64_t s, uint64_t* out, size_t n);
uint64_t orc_zprng_at(uint64_t seed, uint64_t i);
void orc_salted_leaf_hash(uint64_t v, uint64_t sseed, uint64_t idx, uint8_t out[32]);
void orc_merkle_build_salted(const uint64_t* cw, size_t M, uint64_t sseed, uint8_t* tree);
void orc_node_hash(const uint8_t l[32], const uint8_t r[32], uint8_t out[32]);
void orc_merkle_build(const uint64_t* cw, size_t M, uint8_t* tree);
void orc_merkle_root(const uint64_t* cw, size_t M, uint8_t root[32]);
void orc_merkle_path(const uint8_t* tree, size_t M, size_t idx, uint8_t* path /* logM*32 */);
int  orc_merkle_verify_path(const uint8_t leaf[32], size_t idx, const uint8_t* path,
                            uint32_t plen, const uint8_t root[32]);

/* ---- codeword fold: zkllm-src/p3_fri.cuh:396-415 ---- */
uint64_t orc_fold_pair(uint64_t a, uint64_t b, uint64_t invx, uint64_t beta, int mle);
void orc_fold(const uint64_t* f, size_t M, uint64_t wM, uint64_t beta, int mle, uint64_t* out);

/* ---- Basefold evaluation opening: zkllm-src/p3_basefold.cuh:355-496 ----
 * Serialized proof layout (little-endian):
 *   u32 logN, R, Q | roots v*32 | msgs v*24 | final 2^R*8 |
 *   per query q, per round r: a(8) b(8) pa((logM0-r)*32) pb((logM0-r)*32) |
 *   z v*8 | y 8
 * Returns bytes written (0 if cap too small; call with out=NULL to size). */
size_t orc_bf_proof_size(uint32_t v, uint32_t R, uint32_t Q);
size_t orc_bf_prove_eval(const uint64_t* c, const uint64_t* z, uint32_t v, uint64_t y,
                         uint32_t R, uint32_t Q, const uint64_t* cw0,
                         const char* seed, uint8_t* out, size_t cap);
/* verifier: zkllm-src/p3_basefold.cuh:499-535, p3_fri.cuh:466-502.  1 = accept */
int orc_bf_verify_eval(const uint8_t* proof, size_t len, const char* seed);

/* ---- GKR fractional-sum tree: zkllm-src/p3_gkr.cuh:200-364 ----
 * Serialized proof: P(8) Q(8) | per layer h=L..1: nmsg(u32) msgs nmsg*32 p0 p1 q0 q1 (32)
 * rfin gets L values if combine_last else L-1; cpq gets (cp,cq) if combine_last. */
size_t orc_gkr_proof_size(uint32_t L);
size_t orc_gkr_prove(uint8_t st[32], const char* tag, const uint64_t* p, const uint64_t* q,
                     uint32_t L, int combine_last, uint64_t* rfin, uint64_t cpq[2],
                     uint8_t* out, size_t cap);
/* zkllm-src/p3_gkr.cuh:370-421; out4 as in the reference.  1 = accept */
int orc_gkr_verify(uint8_t st[32], const char* tag, uint32_t L, const uint8_t* proof,
                   size_t len, int combine_last, uint64_t* rfin, uint64_t out4[4]);

/* ---- batched opening of one size class, non-zk: zkllm-src/p3_batchopen.cuh:307-1302 ----
 * Ledger: k entries (column values, commitment root, point index zid, claimed value y), T points
 * of v coordinates.  Entries with equal roots are the same column.  st = main transcript.
 * Serialized BatchProof: see zkh_oracle.c. */
size_t orc_bo_proof_bound(uint32_t v, uint32_t R, uint32_t Q, uint32_t nc);
size_t orc_bo_prove_class(uint8_t st[32], uint32_t v, const uint64_t* pts, uint32_t T,
                          const uint64_t* const* cols, const uint8_t* roots, const uint32_t* zid, uint32_t k,
                          uint32_t R, uint32_t Q, const char* label, uint8_t* out, size_t cap);
/* hiding mode: columns committed with salted leaves under sseeds[j]; round-0 sections carry the salts after the values
 * (zkllm-src/p3_batchopen.cuh:1028-1131); cap: orc_bo_proof_bound + nc*2*Q*32 */
size_t orc_bo_prove_class_salted(uint8_t st[32], uint32_t v, const uint64_t* pts, uint32_t T,
                                 const uint64_t* const* cols, const uint8_t* roots, const uint32_t* zid,
                                 const uint64_t* sseeds, uint32_t k, uint32_t R, uint32_t Q, const char* label,
                                 uint8_t* out, size_t cap);
void orc_salt_of(uint64_t sseed, uint64_t idx, uint8_t out[32]);
int orc_bo_verify_class(uint8_t st[32], uint32_t v, const uint64_t* pts, uint32_t T, const uint8_t* roots,
                        const uint32_t* zid, const uint64_t* y, uint32_t k, uint32_t R, uint32_t Q,
                        const char* label, const uint8_t* proof, size_t len);

/* ---- logUp primitives: zkllm-src/p3_logup.cuh:149-172, 636-672 ---- */
int  orc_histogram(const uint32_t* idx, size_t n, uint32_t M, uint64_t* cnt); /* -1 on oob */
int  orc_inv_all_add(const uint64_t* A, size_t n, uint64_t beta, uint64_t* out); /* -1 on zero */
void orc_combine(const uint64_t* const* cols, int c, size_t n, uint64_t g, uint64_t* out);

/* test LCG used by the reference's selftests: p3_basefold_selftest.cu:12-13 */
void orc_lcg_fill(uint64_t* out, size_t n, uint64_t* state);

#ifdef __cplusplus
}
#endif
#endif
