"""ctypes binding of the C ABI declared in include/zkh.h.

There is no fallback: if libzkh.so has not been built, loading raises.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
u64p = C.POINTER(C.c_uint64)
_lib = None

ERRORS = {-1: "ZKH_ERR_ARG", -2: "ZKH_ERR_CUDA", -3: "ZKH_ERR_NOMEM", -4: "ZKH_ERR_DOMAIN",
          -5: "ZKH_ERR_LIMIT", -6: "ZKH_ERR_DEVICE"}


class ZkhError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__("%s (%d): %s" % (ERRORS.get(code, "ZKH_ERR"), code, msg))
        self.code = code


def lib_path():
    return os.path.join(HERE, "libzkh.so")


def load_library():
    """Returns the loaded CDLL with argument types declared."""
    global _lib
    if _lib is not None:
        return _lib
    path = lib_path()
    if not os.path.exists(path):
        raise FileNotFoundError(
            "%s is missing: build it with `python zk-hillclimb_b200/build.py` "
            "(there is no CPU fallback)" % path)
    L = C.CDLL(path)
    vp, sz, u32, u64, i = C.c_void_p, C.c_size_t, C.c_uint32, C.c_uint64, C.c_int
    sig = {
        "zkh_ctx_create": (i, [i, vp, C.POINTER(vp)]),
        "zkh_ctx_destroy": (None, [vp]),
        "zkh_ctx_set_stream": (i, [vp, vp]),
        "zkh_ctx_sync": (i, [vp]),
        "zkh_last_error": (C.c_char_p, [vp]),
        "zkh_version": (C.c_char_p, []),
        "zkh_profile_last": (i, [vp, C.POINTER(C.c_float), C.POINTER(u64), C.POINTER(C.c_char_p)]),
        "zkh_dev_alloc": (i, [vp, sz, C.POINTER(vp)]),
        "zkh_host_alloc": (i, [vp, sz, C.POINTER(vp)]),
        "zkh_host_free": (i, [vp, vp]),
        "zkh_dev_free": (i, [vp, vp]),
        "zkh_upload": (i, [vp, vp, vp, sz]),
        "zkh_download": (i, [vp, vp, vp, sz]),
        "zkh_tr_init": (None, [vp, vp, sz]),
        "zkh_tr_absorb": (None, [vp, C.c_char_p, vp, u64]),
        "zkh_tr_challenge_bytes": (None, [vp, vp]),
        "zkh_tr_chal": (u64, [vp]),
        "zkh_tr_idx": (u64, [vp, u64]),
        "zkh_gl_eq_build": (i, [vp, vp, u32, vp]),
        "zkh_gl_mle_eval": (i, [vp, vp, vp, u32, vp]),
        "zkh_gl_mle_eval_static": (i, [vp, vp, vp, u32, vp, C.c_char_p, sz]),
        "zkh_gl_bind": (i, [vp, vp, vp, u64, u64]),
        "zkh_sumcheck": (i, [vp, i, i, vp, i, u32, vp, i, C.c_char_p, vp, vp, vp, vp]),
        "zkh_sumcheck_host": (i, [vp, i, i, vp, i, u32, vp, i, C.c_char_p, vp, vp, vp, vp]),
        "zkh_sumcheck_workspace": (sz, [i, u32]),
        "zkh_sumcheck_wide": (i, [vp, i, vp, i, u32, vp, i, C.c_char_p, vp, vp, vp, vp]),
        "zkh_sumcheck_wide_shape": (i, [i, vp, vp]),
        "zkh_sumcheck_zerocheck": (i, [vp, vp, i, u32, vp, i, C.c_char_p, vp, vp, vp, vp]),
        "zkh_sumcheck_zerocheck_blind": (i, [vp, vp, i, u32, vp, i, vp, C.c_char_p, vp, vp, vp, vp, vp]),
        "zkh_sumcheck_zerocheck_partial": (i, [vp, vp, i, u32, u32, vp, i, vp, u64, C.c_char_p, vp, vp, vp, vp, vp]),
        "zkh_ig_table": (i, [i, u32, vp, vp]),
        "zkh_fr_eq_build": (i, [vp, vp, u32, vp]),
        "zkh_fr_fold": (i, [vp, vp, u64, vp, vp]),
        "zkh_fr_partial_me": (i, [vp, vp, u64, u32, u64, vp, vp]),
        "zkh_fr_mle_eval": (i, [vp, vp, vp, u32, vp]),
        "zkh_fr_mul_throughput": (i, [vp, u32, vp]),
        "zkh_fr_inv_add": (i, [vp, vp, u64, vp, vp]),
        "zkh_fr_dot": (i, [vp, vp, vp, u64, vp]),
        "zkh_fr_lookup_sumcheck": (i, [vp, vp, vp, vp, vp, vp, u32, u32, vp, vp, vp, vp, vp, vp, vp, vp]),
        "zkh_fr_sumcheck": (i, [vp, vp, i, u32, vp, vp, vp, vp, vp]),
        "zkh_ctx_release_workspace": (i, [vp]),
        "zkh_ig_add_witness": (i, [vp, vp, vp, u64, vp, vp]),
        "zkh_ig_rs20_index": (i, [vp, vp, u64, vp]),
        "zkh_ig_swiglu_witness": (i, [vp, vp, vp, vp, u64, vp, vp, vp, vp, vp, vp]),
        "zkh_ig_rope_witness": (i, [vp, vp, vp, vp, u32, u32, u32, u32, vp, vp, vp, vp, vp, vp]),
        "zkh_ig_rms_witness": (i, [vp, vp, vp, vp, u32, u32, vp, vp, vp, vp, vp]),
        "zkh_ig_softmax_witness": (i, [vp, vp, vp, u32, u32, vp, vp, vp, vp, vp, vp]),
        "zkh_ig_matmul": (i, [vp, vp, vp, vp, vp, vp, vp, u32, u32, u32, u32, u32]),
        "zkh_shard_begin": (i, [vp, i, i, vp, i, u32, vp, i, C.c_char_p, vp]),
        "zkh_shard_round_local": (i, [vp, u32, vp]),
        "zkh_p2p_create": (i, [vp, vp]),
        "zkh_p2p_connect": (i, [vp, u32, u32, vp]),
        "zkh_p2p_disconnect": (i, [vp]),
        "zkh_shard_round_fused": (i, [vp, u32]),
        "zkh_shard_local_fused": (i, [vp, vp]),
        "zkh_shard_prove_fused": (i, [vp]),
        "zkh_shard_round_combine": (i, [vp, u32, vp, u32]),
        "zkh_shard_finals": (i, [vp, vp]),
        "zkh_shard_residual": (i, [vp, vp, u32]),
        "zkh_shard_end": (i, [vp, vp, vp, vp, vp]),
        "zkh_batchopen_proof_bound": (sz, [u32, u32, u32, u32]),
        "zkh_batchopen_prove_class": (i, [vp, u32, vp, u32, vp, vp, vp, u32, u32, u32, C.c_char_p, vp, vp, sz,
                                          C.POINTER(sz)]),
        "zkh_batchopen_prove_class_kept": (i, [vp, u32, vp, u32, vp, vp, vp, u32, u32, u32, C.c_char_p, vp, vp, sz,
                                               C.POINTER(sz), vp, vp]),
        "zkh_batchopen_prove_class_salted": (i, [vp, u32, vp, u32, vp, vp, vp, vp, u32, u32, u32, C.c_char_p, vp, vp, sz,
                                                 C.POINTER(sz), vp, vp]),
        "zkh_basefold_commit_keep": (i, [vp, vp, u32, u32, vp, vp, vp]),
        "zkh_histogram": (i, [vp, vp, u64, u32, vp]),
        "zkh_gl_inv_all_add": (i, [vp, vp, u64, u64, vp]),
        "zkh_gl_combine": (i, [vp, vp, i, u64, u64, vp]),
        "zkh_gl_affine": (i, [vp, vp, i, u64, u64, u64, vp]),
        "zkh_gl_matvec": (i, [vp, vp, u64, u64, vp, i, vp]),
        "zkh_gl_matmul": (i, [vp, vp, vp, u64, u64, u64, vp]),
        "zkh_gl_scale": (i, [vp, vp, u64, u64, vp]),
        "zkh_gl_gather_bits": (i, [vp, vp, u64, u64, u64, vp, u32, vp]),
        "zkh_gl_scatter_bits": (i, [vp, vp, u64, u64, vp, u32, vp, u64]),
        "zkh_gl_gather_xor": (i, [vp, vp, u64, u64, vp]),
        "zkh_g1_pedersen_commit": (i, [vp, vp, vp, u32, u32, vp]),
        "zkh_g1_msm": (i, [vp, vp, vp, u32, vp]),
        "zkh_g1_rows_lincomb": (i, [vp, vp, vp, vp, u32, i, vp]),
        "zkh_g1_rows_add": (i, [vp, vp, vp, u32, vp]),
        "zkh_fr_axpy": (i, [vp, vp, vp, vp, u64]),
        "zkh_fr_round_sums": (i, [vp, vp, vp, u64, vp]),
        "zkh_fr_mul": (i, [vp, vp, vp, vp, u64]),
        "zkh_g1_rows_check": (i, [vp, vp, vp, vp, vp, u32, vp]),
        "zkh_g1_fold_chain": (i, [vp, vp, u32, vp, u32, i, vp]),
        "zkh_g1_ipa_prove": (i, [vp, vp, vp, vp, vp, u32, vp, vp, vp, vp]),
        "zkh_g1_ipa_verify": (i, [vp, vp, u32, vp, vp, vp, vp, vp, vp, vp, vp]),
        "zkh_gl_lift_i32": (i, [vp, vp, u64, vp]),
        "zkh_gl_lift_i64": (i, [vp, vp, u64, vp]),
        "zkh_ig_causal_mask": (i, [vp, u32, u32, vp]),
        "zkh_gl_mul": (i, [vp, vp, vp, u64, vp]),
        "zkh_irs_witness": (i, [vp, vp, u64, u32, i, vp, vp, vp, vp, vp, vp]),
        "zkh_basefold_commit_many": (i, [vp, vp, vp, u32, u32, vp]),
        "zkh_basefold_commit_salted": (i, [vp, vp, u32, u32, u64, vp, vp, vp]),
        "zkh_zk_fill_at": (i, [vp, u64, u64, u64, vp]),
        "zkh_zk_fill_chain": (i, [vp, u64, u64, u64, vp]),
        "zkh_zk_augment": (i, [vp, vp, u32, u32, u64, vp]),
        "zkh_hwl_witness": (i, [vp, u32, u32, u32, vp, vp, vp, vp, vp, vp]),
        "zkh_gkr_proof_size": (sz, [u32]),
        "zkh_gkr_prove": (i, [vp, vp, vp, u32, i, C.c_char_p, vp, vp, vp, vp, sz, C.POINTER(sz)]),
        "zkh_ntt": (i, [vp, vp, vp, u32, i]),
        "zkh_rs_encode": (i, [vp, vp, u32, u32, vp]),
        "zkh_merkle_tree_bytes": (sz, [u64]),
        "zkh_basefold_kept_tree_bytes": (sz, [u32]),
        "zkh_merkle_build": (i, [vp, vp, u64, vp, vp]),
        "zkh_merkle_paths": (i, [vp, vp, u64, vp, u32, vp]),
        "zkh_gl_fold_codeword": (i, [vp, vp, vp, u64, u64]),
        "zkh_basefold_commit": (i, [vp, vp, u32, u32, vp, vp]),
        "zkh_basefold_commit_host": (i, [vp, vp, u32, u32, vp]),
        "zkh_basefold_proof_size": (sz, [u32, u32, u32]),
        "zkh_basefold_open": (i, [vp, vp, vp, u32, u64, u32, u32, vp, C.c_char_p, vp, sz, C.POINTER(sz)]),
    }
    for name, (res, args) in sig.items():
        f = getattr(L, name)
        f.restype = res
        f.argtypes = args
    _lib = L
    return L
