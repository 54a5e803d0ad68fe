"""ctypes bindings for the test oracle (TEST INFRASTRUCTURE ONLY).

Two libraries share one calling convention:

* ``Oracle()``  -> oracle/libzkh_oracle.so, the plain-C restatement (prefix ``orc_``)
* ``Reference()`` -> oracle/_ref/libp3ref.so, the unmodified reference headers
  behind a C shim (prefix ``ref_``); present only where it was built.

Only tests, the smoke check and the benchmark's CPU-baseline leg import this.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
GL_P = 0xFFFFFFFF00000001
u64p = C.POINTER(C.c_uint64)
u8p = C.POINTER(C.c_uint8)

F_PROD2, F_PROD3, F_GKR, F_LOGUP, F_IRS1, F_IRS2 = 0, 1, 2, 3, 4, 5
FUNCTOR_NC = {F_PROD2: 2, F_PROD3: 3, F_GKR: 5, F_LOGUP: 4, F_IRS1: 4, F_IRS2: 5}
F_HW_DP, F_HW_DG, F_HW_CH, F_HW_GS, F_HW_DS, F_HW_DO = 6, 7, 8, 9, 10, 11
HW_SHAPE = {6: (12, 6), 7: (30, 18), 8: (11, 6), 9: (3, 2), 10: (8, 6), 11: (57, 49)}   # functor -> (columns, coefficients)


def build(ref=True):
    """Compile the oracle (and the reference shim when its tree is present)."""
    subprocess.check_call(["make", "-s", "-C", HERE, "oracle"])
    if ref:
        subprocess.check_call(["make", "-s", "-C", HERE, "ref"])


def _u64(a):
    a = np.ascontiguousarray(a, dtype=np.uint64)
    return a, a.ctypes.data_as(u64p)


def _bytes32(b=None):
    buf = (C.c_uint8 * 32)()
    if b is not None:
        buf[:] = bytes(b)
    return buf


class _Lib:
    prefix = ""
    path = ""

    def __init__(self):
        if not os.path.exists(self.path):
            raise FileNotFoundError(self.path)
        self.lib = C.CDLL(self.path)
        L, p = self.lib, self.prefix
        for name in ("gl_add", "gl_sub", "gl_mul", "gl_pow"):
            f = getattr(L, p + name); f.restype = C.c_uint64; f.argtypes = [C.c_uint64, C.c_uint64]
        for name in ("gl_inv",):
            f = getattr(L, p + name); f.restype = C.c_uint64; f.argtypes = [C.c_uint64]
        f = getattr(L, p + "gl_root_of_unity"); f.restype = C.c_uint64; f.argtypes = [C.c_uint32]
        getattr(L, p + "tr_chal").restype = C.c_uint64
        getattr(L, p + "tr_idx").restype = C.c_uint64
        getattr(L, p + "tr_idx").argtypes = [C.c_void_p, C.c_uint64]
        getattr(L, p + "eval_h").restype = C.c_uint64
        getattr(L, p + "eval_h").argtypes = [u64p, u64p, C.c_size_t]
        getattr(L, p + "quad_eval").restype = C.c_uint64
        getattr(L, p + "quad_eval").argtypes = [C.c_uint64] * 4
        getattr(L, p + "cubic_eval").restype = C.c_uint64
        getattr(L, p + "cubic_eval").argtypes = [C.c_uint64] * 5
        getattr(L, p + "quartic_eval").restype = C.c_uint64
        getattr(L, p + "quartic_eval").argtypes = [u64p, C.c_uint64]
        getattr(L, p + "eq_point").restype = C.c_uint64
        getattr(L, p + "eq_point").argtypes = [u64p, u64p, C.c_uint32]
        getattr(L, p + "bf_prove_eval").restype = C.c_size_t
        getattr(L, p + "bf_prove_eval").argtypes = [u64p, u64p, C.c_uint32, C.c_uint64, C.c_uint32,
                                                    C.c_uint32, u64p, C.c_char_p, C.c_void_p, C.c_size_t]
        getattr(L, p + "bf_verify_eval").argtypes = [C.c_void_p, C.c_size_t, C.c_char_p]
        getattr(L, p + "gkr_prove").restype = C.c_size_t
        getattr(L, p + "fold").argtypes = [u64p, C.c_size_t, C.c_uint64, C.c_uint64, C.c_int, u64p]
        getattr(L, p + "merkle_root").argtypes = [u64p, C.c_size_t, C.c_void_p]
        getattr(L, p + "merkle_build").argtypes = [u64p, C.c_size_t, C.c_void_p]
        getattr(L, p + "rs_encode_horner").argtypes = [u64p, C.c_uint32, C.c_uint32, u64p]
        getattr(L, p + "build_eq").argtypes = [u64p, C.c_uint32, u64p]
        getattr(L, p + "inv_all_add").argtypes = [u64p, C.c_size_t, C.c_uint64, u64p]
        getattr(L, p + "combine").argtypes = [C.POINTER(u64p), C.c_int, C.c_size_t, C.c_uint64, u64p]
        getattr(L, p + "sha256").argtypes = [C.c_void_p, C.c_size_t, C.c_void_p]

    def _f(self, name):
        return getattr(self.lib, self.prefix + name)

    # ---- field ----
    def gl_add(self, a, b): return self._f("gl_add")(a, b)
    def gl_sub(self, a, b): return self._f("gl_sub")(a, b)
    def gl_mul(self, a, b): return self._f("gl_mul")(a, b)
    def gl_pow(self, a, e): return self._f("gl_pow")(a, e)
    def gl_inv(self, a): return self._f("gl_inv")(a)
    def gl_root_of_unity(self, logn): return self._f("gl_root_of_unity")(logn)

    # ---- hashing / transcript (state is a 32-byte ``bytes``) ----
    def sha256(self, data):
        out = _bytes32(); self._f("sha256")(bytes(data), len(data), out); return bytes(out)

    def compress64(self, data):
        assert len(data) == 64
        out = _bytes32(); self._f("sha256_compress64")(bytes(data), out); return bytes(out)

    def tr_init(self, seed):
        seed = seed.encode() if isinstance(seed, str) else bytes(seed)
        st = _bytes32(); self._f("tr_init")(st, seed, C.c_size_t(len(seed))); return bytes(st)

    def tr_absorb(self, st, label, data):
        s = _bytes32(st); data = bytes(data)
        self._f("tr_absorb")(s, label.encode(), data, C.c_uint64(len(data))); return bytes(s)

    def tr_challenge_bytes(self, st):
        s = _bytes32(st); out = _bytes32(); self._f("tr_challenge_bytes")(s, out)
        return bytes(s), bytes(out)

    def tr_chal(self, st):
        s = _bytes32(st); a = self._f("tr_chal")(s); return bytes(s), a

    def tr_idx(self, st, mod):
        s = _bytes32(st); a = self._f("tr_idx")(s, mod); return bytes(s), a

    # ---- multilinear helpers ----
    def build_eq(self, z):
        z, zp = _u64(z); out = np.empty(1 << len(z), dtype=np.uint64)
        self._f("build_eq")(zp, len(z), out.ctypes.data_as(u64p)); return out

    def eval_h(self, c, eq):
        c, cp = _u64(c); eq, ep = _u64(eq); return self._f("eval_h")(cp, ep, len(c))

    def quad_eval(self, s0, s1, s2, t): return self._f("quad_eval")(s0, s1, s2, t)
    def cubic_eval(self, s0, s1, s2, s3, t): return self._f("cubic_eval")(s0, s1, s2, s3, t)

    def quartic_eval(self, s, t):
        s, sp = _u64(s); return self._f("quartic_eval")(sp, t)

    def eq_point(self, a, z):
        a, ap = _u64(a); z, zp = _u64(z); return self._f("eq_point")(ap, zp, len(a))

    # ---- encode / merkle / fold ----
    def rs_encode_horner(self, c, R):
        c, cp = _u64(c); v = int(len(c)).bit_length() - 1
        out = np.empty(len(c) << R, dtype=np.uint64)
        self._f("rs_encode_horner")(cp, v, R, out.ctypes.data_as(u64p)); return out

    def merkle_root(self, cw):
        cw, p = _u64(cw); out = _bytes32(); self._f("merkle_root")(p, len(cw), out); return bytes(out)

    def merkle_build(self, cw):
        cw, p = _u64(cw); out = np.empty((2 * len(cw) - 1) * 32, dtype=np.uint8)
        self._f("merkle_build")(p, len(cw), out.ctypes.data_as(C.c_void_p)); return out

    def zprng_fill(self, s, n):
        """n elements of the hiding mode's mask chain from state s (reference: p3zkc::zprng_fill)"""
        out = np.empty(n, dtype=np.uint64)
        f = self.lib.ref_zprng_fill if self.prefix == "ref_" else self.lib.orc_zprng_fill
        f(C.c_uint64(s), out.ctypes.data_as(u64p), C.c_size_t(n))
        return out

    def zprng_at(self, seed, i):
        f = self.lib.ref_zprng_at if self.prefix == "ref_" else self.lib.orc_zprng_at
        f.restype = C.c_uint64
        return int(f(C.c_uint64(seed), C.c_uint64(i)))

    def salted_leaf(self, v, sseed, idx):
        """hiding-commitment leaf SHA-256(value | SHA-256(seed | index)) (reference: p3zkc::salted_leaf o salt_of)"""
        out = _bytes32()
        if self.prefix == "ref_":
            self.lib.ref_salted_leaf(C.c_uint64(v), C.c_uint64(sseed), C.c_uint64(idx), out)
        else:
            self.lib.orc_salted_leaf_hash(C.c_uint64(v), C.c_uint64(sseed), C.c_uint64(idx), out)
        return bytes(out)

    def fold(self, f, wM, beta, mle=True):
        f, p = _u64(f); out = np.empty(len(f) // 2, dtype=np.uint64)
        self._f("fold")(p, len(f), wM, beta, int(mle), out.ctypes.data_as(u64p)); return out

    # ---- Basefold opening ----
    @staticmethod
    def bf_proof_size(v, R, Q):
        s = 12 + v * 32 + v * 24 + (8 << R)
        for r in range(v):
            s += Q * (16 + 2 * (v + R - r) * 32)
        return s + v * 8 + 8

    def bf_prove_eval(self, c, z, y, R, Q, cw0, seed="p3-bf"):
        c, cp = _u64(c); z, zp = _u64(z); cw0, wp = _u64(cw0)
        v = len(z); cap = self.bf_proof_size(v, R, Q)
        out = (C.c_uint8 * cap)()
        n = self._f("bf_prove_eval")(cp, zp, v, y, R, Q, wp, seed.encode(), out, cap)
        assert n == cap, (n, cap)
        return bytes(out)

    def bf_verify_eval(self, proof, seed="p3-bf"):
        return bool(self._f("bf_verify_eval")(bytes(proof), len(proof), seed.encode()))

    # ---- GKR ----
    @staticmethod
    def gkr_proof_size(L):
        return 16 + sum(4 + (L - h) * 32 + 32 for h in range(1, L + 1))

    def gkr_prove(self, st, tag, p, q, combine_last=True, gpu=False):
        p, pp = _u64(p); q, qp = _u64(q); L = int(len(p)).bit_length() - 1
        s = _bytes32(st); cap = self.gkr_proof_size(L); out = (C.c_uint8 * cap)()
        rfin = np.zeros(L + 1, dtype=np.uint64); cpq = np.zeros(2, dtype=np.uint64)
        args = [s, tag.encode(), pp, qp, C.c_uint32(L), C.c_int(int(combine_last)),
                rfin.ctypes.data_as(u64p), cpq.ctypes.data_as(u64p), out, C.c_size_t(cap)]
        if self.prefix == "ref_":
            args.append(C.c_int(int(gpu)))   # the reference's own CUDA path (GPU machine only)
        n = self._f("gkr_prove")(*args)
        if n == 0:
            raise ValueError("gkr_prove failed (zero denominator?)")
        nr = L if combine_last else L - 1
        return bytes(s), bytes(out)[:n], rfin[:nr].copy(), (int(cpq[0]), int(cpq[1]))

    def gkr_verify(self, st, tag, L, proof, combine_last=True):
        s = _bytes32(st); rfin = np.zeros(L + 1, dtype=np.uint64); out4 = np.zeros(4, dtype=np.uint64)
        ok = self._f("gkr_verify")(s, tag.encode(), C.c_uint32(L), bytes(proof), C.c_size_t(len(proof)),
                                   C.c_int(int(combine_last)), rfin.ctypes.data_as(u64p),
                                   out4.ctypes.data_as(u64p))
        nr = L if combine_last else L - 1
        return bool(ok), bytes(s), rfin[:nr].copy(), out4

    # ---- batched opening of one size class ----
    @staticmethod
    def _bo_args(pts, roots, zid):
        pts = np.ascontiguousarray(pts, dtype=np.uint64)
        T, v = pts.shape
        rb = b"".join(bytes(r) for r in roots)
        zid = np.ascontiguousarray(zid, dtype=np.uint32)
        return pts, T, v, rb, zid

    def bo_verify_class(self, st, pts, roots, zid, y, R, Q, label, proof):
        """p3bo::verify_class on the serialised BatchProof.  Returns (ok, new transcript state)."""
        pts, T, v, rb, zid = self._bo_args(pts, roots, zid)
        y = np.ascontiguousarray(y, dtype=np.uint64)
        s = _bytes32(st)
        ok = self._f("bo_verify_class")(s, C.c_uint32(v), pts.ctypes.data_as(u64p), C.c_uint32(T), rb,
                                        zid.ctypes.data_as(C.c_void_p), y.ctypes.data_as(u64p),
                                        C.c_uint32(len(zid)), C.c_uint32(R), C.c_uint32(Q), label.encode(),
                                        bytes(proof), C.c_size_t(len(proof)))
        return bool(ok), bytes(s)

    def bo_prove_class(self, st, pts, cols, roots, zid, R, Q, label):
        """p3bo::prove_class; cols[j] = values of entry j.  Returns (proof bytes, new state[, ms])."""
        pts, T, v, rb, zid = self._bo_args(pts, roots, zid)
        arrs = [np.ascontiguousarray(c, dtype=np.uint64) for c in cols]
        ptrs = (u64p * len(arrs))(*[a.ctypes.data_as(u64p) for a in arrs])
        nc = len(set(bytes(r) for r in roots))
        cap = 16 + nc * 8 + v * 48 + max(v - 1, 0) * 32 + (8 << R) + \
            sum(Q * (16 + 2 * (v + R - r) * 32) for r in range(1, v)) + nc * (8 + 2 * Q * 8 + 2 * Q * (v + R) * 32)
        out = (C.c_uint8 * cap)()
        s = _bytes32(st)
        f = self._f("bo_prove_class")
        f.restype = C.c_size_t
        args = [s, C.c_uint32(v), pts.ctypes.data_as(u64p), C.c_uint32(T), ptrs, rb,
                zid.ctypes.data_as(C.c_void_p), C.c_uint32(len(zid)), C.c_uint32(R), C.c_uint32(Q),
                label.encode(), out, C.c_size_t(cap)]
        ms = C.c_double(0)
        if self.prefix == "ref_":
            args.append(C.byref(ms))
        n = f(*args)
        if n == 0:
            raise RuntimeError("bo_prove_class failed")
        return (bytes(out)[:n], bytes(s)) + ((ms.value,) if self.prefix == "ref_" else ())

    def bo_prove_class_salted(self, st, pts, cols, roots, zid, sseeds, R, Q, label):
        """The hiding mode's prove_class after the blinder was appended (oracle restatement only): salted round-0 openings."""
        pts, T, v, rb, zid = self._bo_args(pts, roots, zid)
        arrs = [np.ascontiguousarray(c, dtype=np.uint64) for c in cols]
        ptrs = (u64p * len(arrs))(*[a.ctypes.data_as(u64p) for a in arrs])
        ss = np.ascontiguousarray(sseeds, dtype=np.uint64)
        nc = len(set(bytes(r) for r in roots))
        cap = 16 + nc * 8 + v * 48 + max(v - 1, 0) * 32 + (8 << R) + \
            sum(Q * (16 + 2 * (v + R - r) * 32) for r in range(1, v)) + nc * (8 + 2 * Q * 40 + 2 * Q * (v + R) * 32)
        out = (C.c_uint8 * cap)()
        s = _bytes32(st)
        f = self.lib.orc_bo_prove_class_salted
        f.restype = C.c_size_t
        n = f(s, C.c_uint32(v), pts.ctypes.data_as(u64p), C.c_uint32(T), ptrs, rb, zid.ctypes.data_as(C.c_void_p),
              ss.ctypes.data_as(u64p), C.c_uint32(len(zid)), C.c_uint32(R), C.c_uint32(Q), label.encode(), out, C.c_size_t(cap))
        if n == 0:
            raise RuntimeError("bo_prove_class_salted failed")
        return bytes(out)[:n], bytes(s)

    # ---- logUp primitives ----
    def inv_all_add(self, A, beta):
        A, ap = _u64(A); out = np.empty(len(A), dtype=np.uint64)
        rc = self._f("inv_all_add")(ap, len(A), beta, out.ctypes.data_as(u64p))
        if rc != 0:
            raise ZeroDivisionError("zero denominator")
        return out

    def combine(self, cols, g):
        arrs = [np.ascontiguousarray(c, dtype=np.uint64) for c in cols]
        ptrs = (u64p * len(arrs))(*[a.ctypes.data_as(u64p) for a in arrs])
        out = np.empty(len(arrs[0]), dtype=np.uint64)
        self._f("combine")(ptrs, len(arrs), len(arrs[0]), g, out.ctypes.data_as(u64p)); return out


class Oracle(_Lib):
    prefix = "orc_"
    path = os.path.join(HERE, "libzkh_oracle.so")

    def __init__(self):
        if not os.path.exists(self.path):
            build(ref=False)
        super().__init__()
        L = self.lib
        L.orc_mle_eval.restype = C.c_uint64
        L.orc_mle_eval.argtypes = [u64p, u64p, C.c_uint32]
        L.orc_rs_encode.argtypes = [u64p, C.c_uint32, C.c_uint32, u64p]
        L.orc_ntt.argtypes = [u64p, C.c_uint32, C.c_int]
        L.orc_histogram.argtypes = [C.c_void_p, C.c_size_t, C.c_uint32, u64p]
        L.orc_lcg_fill.argtypes = [u64p, C.c_size_t, u64p]
        L.orc_bind_lsb.argtypes = [u64p, C.c_size_t, C.c_uint64]

    def sumcheck(self, st, tag, functor, nt, cols, par=(), nthreads=1, inplace=False):
        """Returns (state, msgs[v,nt], chals[v], finals[nc]); cols are copied unless inplace
        (then they are consumed: bound in place)."""
        arrs = [np.ascontiguousarray(c, dtype=np.uint64) if inplace else np.array(c, dtype=np.uint64, copy=True)
                for c in cols]
        nc = len(arrs); logn = int(len(arrs[0])).bit_length() - 1
        ptrs = (u64p * nc)(*[a.ctypes.data_as(u64p) for a in arrs])
        par, pp = _u64(list(par) if len(par) else [0])
        msgs = np.zeros((logn, nt), dtype=np.uint64); chals = np.zeros(logn, dtype=np.uint64)
        fin = np.zeros(nc, dtype=np.uint64); s = _bytes32(st)
        rc = self.lib.orc_sumcheck(s, tag.encode(), functor, nt, ptrs, nc, C.c_uint32(logn), pp,
                                   msgs.ctypes.data_as(u64p), chals.ctypes.data_as(u64p),
                                   fin.ctypes.data_as(u64p), nthreads)
        assert rc == 0
        return bytes(s), msgs, chals, fin

    def merkle_build_salted(self, cw, sseed):
        cw, p = _u64(cw); out = np.empty((2 * len(cw) - 1) * 32, dtype=np.uint8)
        self.lib.orc_merkle_build_salted(p, C.c_size_t(len(cw)), C.c_uint64(sseed), out.ctypes.data_as(C.c_void_p)); return out

    def mle_eval(self, c, z):
        c, cp = _u64(c); z, zp = _u64(z); return self.lib.orc_mle_eval(cp, zp, len(z))

    def rs_encode(self, c, R):
        c, cp = _u64(c); v = int(len(c)).bit_length() - 1
        out = np.empty(len(c) << R, dtype=np.uint64)
        self.lib.orc_rs_encode(cp, v, R, out.ctypes.data_as(u64p)); return out

    def ntt(self, a, inverse=False):
        a = np.array(a, dtype=np.uint64, copy=True)
        self.lib.orc_ntt(a.ctypes.data_as(u64p), int(len(a)).bit_length() - 1, int(inverse)); return a

    def histogram(self, idx, M):
        idx = np.ascontiguousarray(idx, dtype=np.uint32); cnt = np.zeros(M, dtype=np.uint64)
        rc = self.lib.orc_histogram(idx.ctypes.data_as(C.c_void_p), len(idx), M, cnt.ctypes.data_as(u64p))
        if rc != 0:
            raise IndexError("lookup index out of table")
        return cnt

    def lcg(self, n, state):
        out = np.empty(n, dtype=np.uint64); s = C.c_uint64(state)
        self.lib.orc_lcg_fill(out.ctypes.data_as(u64p), n, C.byref(s)); return out, s.value

    def bind_lsb(self, f, a):
        f = np.array(f, dtype=np.uint64, copy=True)
        self.lib.orc_bind_lsb(f.ctypes.data_as(u64p), len(f), a); return f[: len(f) // 2].copy()


class Reference(_Lib):
    prefix = "ref_"
    path = os.path.join(HERE, "_ref", "libp3ref.so")

    def __init__(self):
        super().__init__()
        L = self.lib
        L.ref_bf_prove_eval_dev.restype = C.c_size_t

    @staticmethod
    def available():
        return os.path.exists(Reference.path)

    def gpu_available(self):
        return bool(self.lib.ref_gpu_available())

    def lu_sc_prove(self, st, tag, H, V, E, D, lam, beta):
        H, hp = _u64(H); V, vp = _u64(V); E, ep = _u64(E); D, dp = _u64(D)
        logn = int(len(H)).bit_length() - 1
        msgs = np.zeros((logn, 4), dtype=np.uint64); chals = np.zeros(logn, dtype=np.uint64)
        s = _bytes32(st)
        self.lib.ref_lu_sc_prove(s, tag.encode(), hp, vp, ep, dp, C.c_uint32(logn), C.c_uint64(lam),
                                 C.c_uint64(beta), msgs.ctypes.data_as(u64p), chals.ctypes.data_as(u64p))
        return bytes(s), msgs, chals

    def sc5_prove(self, st, tag, functor, cols):
        arrs = [np.ascontiguousarray(c, dtype=np.uint64) for c in cols]
        nc = len(arrs); logn = int(len(arrs[0])).bit_length() - 1
        ptrs = (u64p * nc)(*[a.ctypes.data_as(u64p) for a in arrs])
        msgs = np.zeros((logn, 5), dtype=np.uint64); chals = np.zeros(logn, dtype=np.uint64)
        s = _bytes32(st)
        rc = self.lib.ref_sc5_prove(s, tag.encode(), functor, ptrs, nc, C.c_uint32(logn),
                                    msgs.ctypes.data_as(u64p), chals.ctypes.data_as(u64p))
        assert rc == 0
        return bytes(s), msgs, chals

    def sc5_prove_lam(self, st, tag, functor, cols, lam):
        """p3hwl::sc5_prove with the reference's fp8-gadget constraint function `functor` (6..11)."""
        arrs = [np.ascontiguousarray(c, dtype=np.uint64) for c in cols]
        nc = len(arrs); logn = int(len(arrs[0])).bit_length() - 1
        ptrs = (u64p * nc)(*[a.ctypes.data_as(u64p) for a in arrs])
        la, lp = _u64(lam)
        msgs = np.zeros((logn, 5), dtype=np.uint64); chals = np.zeros(logn, dtype=np.uint64)
        s = _bytes32(st)
        rc = self.lib.ref_sc5_prove_lam(s, tag.encode(), functor, ptrs, nc, C.c_uint32(logn), lp, len(la),
                                        msgs.ctypes.data_as(u64p), chals.ctypes.data_as(u64p))
        assert rc == 0
        return bytes(s), msgs, chals

    # ---- the reference's CUDA paths (GPU machine only) ----
    def sc_prove_gpu(self, st, tag, functor, nt, cols, par=()):
        arrs = [np.ascontiguousarray(c, dtype=np.uint64) for c in cols]
        nc = len(arrs); logn = int(len(arrs[0])).bit_length() - 1
        ptrs = (u64p * nc)(*[a.ctypes.data_as(u64p) for a in arrs])
        par_a, pp = _u64(list(par) if len(par) else [0])
        msgs = np.zeros((logn, nt), dtype=np.uint64); chals = np.zeros(logn, dtype=np.uint64)
        s = _bytes32(st); ms = C.c_double(0)
        rc = self.lib.ref_sc_prove_gpu(s, tag.encode(), functor, nt, ptrs, nc, C.c_uint32(logn), pp,
                                       C.c_uint32(len(par)), msgs.ctypes.data_as(u64p),
                                       chals.ctypes.data_as(u64p), C.byref(ms))
        if rc != 0:
            raise RuntimeError("ref_sc_prove_gpu rc=%d" % rc)
        return bytes(s), msgs, chals, ms.value

    def commit_gpu_rootonly(self, c, R):
        c, cp = _u64(c); v = int(len(c)).bit_length() - 1
        out = _bytes32(); ms = C.c_double(0)
        rc = self.lib.ref_commit_gpu_rootonly(cp, C.c_uint32(v), C.c_uint32(R), out, C.byref(ms))
        if rc != 0:
            raise RuntimeError("ref_commit_gpu_rootonly failed")
        return bytes(out), ms.value

    def salted_commit_root(self, c, R, sseed):
        """p3zkc::salted_commit_root_dev on the GPU (salting on)"""
        c, cp = _u64(c); v = int(len(c)).bit_length() - 1
        out = _bytes32()
        rc = self.lib.ref_salted_commit_root(cp, C.c_uint32(v), C.c_uint32(R), C.c_uint64(sseed), out)
        if rc != 0:
            raise RuntimeError("ref_salted_commit_root rc=%d" % rc)
        return bytes(out)

    def rs_encode_gpu(self, c, R):
        c, cp = _u64(c); v = int(len(c)).bit_length() - 1
        out = np.empty(len(c) << R, dtype=np.uint64)
        rc = self.lib.ref_rs_encode_gpu(cp, C.c_uint32(v), C.c_uint32(R), out.ctypes.data_as(u64p))
        if rc != 0:
            raise RuntimeError("ref_rs_encode_gpu failed")
        return out

    def bf_prove_eval_dev(self, c, z, y, R, Q, cw0, seed="p3-bf"):
        c, cp = _u64(c); z, zp = _u64(z); cw0, wp = _u64(cw0)
        v = len(z); cap = self.bf_proof_size(v, R, Q); out = (C.c_uint8 * cap)(); ms = C.c_double(0)
        n = self.lib.ref_bf_prove_eval_dev(cp, zp, C.c_uint32(v), C.c_uint64(y), C.c_uint32(R),
                                           C.c_uint32(Q), wp, seed.encode(), out, C.c_size_t(cap),
                                           C.byref(ms))
        assert n == cap
        return bytes(out), ms.value
