"""Host-side mirror of the reference's in-process prover interface ("p3" stack).

Names, argument meaning and error behaviour follow the reference so that the
parity tests read like the reference's own selftests:

  Transcript              fs::Transcript            zkllm-src/fs_transcript.hpp:115-166
  chal / idx_from         p3sg::chal, p3fri::idx_from   p3_scgpu.cuh:31-35, p3_fri.cuh:422-426
  Prover.sc_prove_gpu     p3sg::sc_prove_gpu        zkllm-src/p3_scgpu.cuh:91-160
  Prover.build_eq_gpu     p3bf::build_eq_gpu        zkllm-src/p3_basefold.cuh:275-283
  Prover.eval_h_gpu       p3bf::eval_h_gpu          zkllm-src/p3_basefold.cuh:262-273
  Prover.bind             p3bf_bind_kernel          zkllm-src/p3_basefold.cuh:336-339

All computation happens in libzkh.so (CUDA, sm_100a).  Device buffers are torch
int64 CUDA tensors holding the uint64 bit patterns; torch is only the allocator.
Errors from the library raise ZkhError (the reference throws std::runtime_error).
"""
import ctypes as C

import numpy as np

from ._lib import ZkhError, load_library, u64p

GL_P = 0xFFFFFFFF00000001
F_PROD2, F_PROD3, F_GKR, F_LOGUP, F_IRS1, F_IRS2 = 0, 1, 2, 3, 4, 5
FUNCTOR_NC = {F_PROD2: 2, F_PROD3: 3, F_GKR: 5, F_LOGUP: 4, F_IRS1: 4, F_IRS2: 5}
F_HW_DP, F_HW_DG, F_HW_CH, F_HW_GS, F_HW_DS, F_HW_DO = 6, 7, 8, 9, 10, 11   # wide quartic summands (sc5_run)


def _buf32(b=None):
    buf = (C.c_uint8 * 32)()
    if b is not None:
        buf[:] = bytes(b)
    return buf


class Transcript:
    """fs::Transcript: SHA-256 Fiat-Shamir state (32 bytes)."""

    def __init__(self, seed=None, state=None):
        self._L = load_library()
        self._st = _buf32(state)
        if state is None:
            seed = seed.encode() if isinstance(seed, str) else bytes(seed or b"")
            self._L.zkh_tr_init(self._st, seed, len(seed))

    @property
    def state(self):
        return bytes(self._st)

    @state.setter
    def state(self, b):
        self._st[:] = bytes(b)

    def absorb(self, label, data):
        if isinstance(data, np.ndarray):
            data = np.ascontiguousarray(data).tobytes()
        data = bytes(data)
        self._L.zkh_tr_absorb(self._st, label.encode(), data, len(data))

    def challenge_bytes(self):
        out = _buf32()
        self._L.zkh_tr_challenge_bytes(self._st, out)
        return bytes(out)

    def chal(self):
        """Field challenge (first 8 digest bytes, little endian, mod p)."""
        return int(self._L.zkh_tr_chal(self._st))

    def idx_from(self, mod):
        return int(self._L.zkh_tr_idx(self._st, mod))


def zc_program(terms, konst=0):
    """Pack [(coef, (idx, ...)), ...] and the constant into the word list zkh_sumcheck_zerocheck reads.  A term with a
    third element that is true stands outside the col0 factor (the blind of a hiding chain)."""
    words = [len(terms), int(konst) % GL_P]
    for term in terms:
        coef, idx = term[0], term[1]
        if not 1 <= len(idx) <= 3:
            raise ValueError("zero-check term: one to three columns")
        pk = len(idx) | (0x80 if len(term) > 2 and term[2] else 0)
        for k, i in enumerate(idx):
            pk |= int(i) << (8 + 8 * k)
        words += [int(coef) % GL_P, pk]
    return np.array(words, dtype=np.uint64)


def to_device(arr, device="cuda:0"):
    """numpy uint64 array -> torch int64 CUDA tensor with the same bits."""
    import torch
    a = np.ascontiguousarray(arr, dtype=np.uint64)
    return torch.from_numpy(a.view(np.int64)).to(device)


def to_host(t):
    """torch int64 tensor -> numpy uint64 array."""
    return t.detach().cpu().numpy().view(np.uint64)


def _ptr(t):
    return t if isinstance(t, int) else t.data_ptr()


def eval_h_static(c_dev, z, y_dev, stream=None):
    """MLE evaluation without any device allocation (zkh_gl_mle_eval_static): for hosts that
    own all of HBM through their own arena, for code inside a stream capture, and for loops
    that must not trigger an allocation's device synchronisation.  Works on the current CUDA
    device; c_dev and y_dev are the caller's device tensors (y_dev: one element); at most 28
    variables.  Asynchronous on ``stream``; calls sharing a device must not overlap."""
    L = load_library()
    z = np.ascontiguousarray(z, dtype=np.uint64)
    err = C.create_string_buffer(256)
    rc = L.zkh_gl_mle_eval_static(C.c_void_p(stream or 0), _ptr(c_dev), z.ctypes.data, len(z), _ptr(y_dev),
                                  err, len(err))
    if rc != 0:
        raise ZkhError(rc, err.value.decode())


class Prover:
    """One per GPU: owns a library context (workspace, control block, stream)."""

    def __init__(self, device=0, stream=None):
        """stream: None -> the context creates its own non-blocking stream; an integer
        cudaStream_t handle -> work is queued there (0, torch's default stream, is passed as
        cudaStreamLegacy so that it orders with torch's own kernels)."""
        self._L = load_library()
        h = C.c_void_p()
        if stream is not None and int(stream) == 0:
            stream = 1  # cudaStreamLegacy
        rc = self._L.zkh_ctx_create(int(device), C.c_void_p(stream or 0), C.byref(h))
        if rc != 0:
            raise ZkhError(rc, "zkh_ctx_create(device=%d) failed" % device)
        self._h = h
        self.device = int(device)

    def close(self):
        if getattr(self, "_h", None):
            self._L.zkh_ctx_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _ck(self, rc):
        if rc != 0:
            raise ZkhError(rc, (self._L.zkh_last_error(self._h) or b"").decode())

    def set_stream(self, stream):
        if stream is not None and int(stream) == 0:
            stream = 1  # cudaStreamLegacy
        self._ck(self._L.zkh_ctx_set_stream(self._h, C.c_void_p(stream or 0)))

    def sync(self):
        self._ck(self._L.zkh_ctx_sync(self._h))

    def release_workspace(self):
        """Give the context's scratch workspace back to the device (it is re-allocated on demand)."""
        self._ck(self._L.zkh_ctx_release_workspace(self._h))

    def profile_last(self):
        """(kernel name, milliseconds, algorithmic bytes) of the dominant launch of the last call."""
        ms, nb, nm = C.c_float(0), C.c_uint64(0), C.c_char_p()
        self._ck(self._L.zkh_profile_last(self._h, C.byref(ms), C.byref(nb), C.byref(nm)))
        return (nm.value or b"").decode(), float(ms.value), int(nb.value)

    # ---- multilinear vector kernels ----
    def build_eq_gpu(self, z, out=None):
        """eq(b,z) for all b, on device.  Returns a torch tensor of 2^len(z) elements."""
        import torch
        z = np.ascontiguousarray(z, dtype=np.uint64)
        if out is None:
            out = torch.empty(1 << len(z), dtype=torch.int64, device="cuda:%d" % self.device)
        self._ck(self._L.zkh_gl_eq_build(self._h, z.ctypes.data, len(z), _ptr(out)))
        return out

    def eval_h_gpu(self, c_dev, z):
        z = np.ascontiguousarray(z, dtype=np.uint64)
        y = C.c_uint64(0)
        self._ck(self._L.zkh_gl_mle_eval(self._h, _ptr(c_dev), z.ctypes.data, len(z), C.byref(y)))
        return int(y.value)

    def element(self, col_dev, i):
        return int(to_host(col_dev[i:i + 1])[0])

    def bind(self, in_dev, a, out=None, n=None):
        import torch
        n = n if n is not None else in_dev.numel()
        if out is None:
            out = torch.empty(n // 2, dtype=torch.int64, device=in_dev.device)
        self._ck(self._L.zkh_gl_bind(self._h, _ptr(in_dev), _ptr(out), n, a))
        return out

    # ---- Reed-Solomon / Merkle / Basefold ----
    def ntt(self, in_dev, inverse=False, out=None):
        """P3Ntt::run (zkllm-src/p3_ntt.cuh:210-230): natural order in and out."""
        import torch
        n = in_dev.numel()
        if out is None:
            out = torch.empty(n, dtype=torch.int64, device=in_dev.device)
        self._ck(self._L.zkh_ntt(self._h, _ptr(in_dev), _ptr(out), n.bit_length() - 1, int(inverse)))
        return out

    def rs_encode_gpu_dev(self, c_dev, R, out=None):
        """p3bf::rs_encode_gpu_dev (zkllm-src/p3_basefold.cuh:188-197): device codeword of device coefficients."""
        import torch
        n = c_dev.numel()
        if out is None:
            out = torch.empty(n << R, dtype=torch.int64, device=c_dev.device)
        self._ck(self._L.zkh_rs_encode(self._h, _ptr(c_dev), n.bit_length() - 1, R, _ptr(out)))
        return out

    def merkle_build_dev(self, cw_dev, keep_tree=True):
        """p3fri::DeviceMerkle::build_dev (zkllm-src/p3_fri.cuh:109-139).  Returns (root bytes, tree tensor or None)."""
        import torch
        M = cw_dev.numel()
        tree = None
        if keep_tree:
            tree = torch.empty(self._L.zkh_merkle_tree_bytes(M), dtype=torch.uint8, device=cw_dev.device)
        root = _buf32()
        self._ck(self._L.zkh_merkle_build(self._h, _ptr(cw_dev), M, _ptr(tree) if keep_tree else 0, root))
        return bytes(root), tree

    def paths_batch(self, tree_dev, M, idxs):
        """DeviceMerkle::paths_batch (zkllm-src/p3_fri.cuh:164-178): list of paths, each a list of 32-byte digests."""
        idx = np.ascontiguousarray(idxs, dtype=np.uint32)
        logM = int(M).bit_length() - 1
        out = np.zeros(len(idx) * logM * 32, dtype=np.uint8)
        self._ck(self._L.zkh_merkle_paths(self._h, _ptr(tree_dev), M, idx.ctypes.data, len(idx), out.ctypes.data))
        raw = out.tobytes()
        return [[raw[(i * logM + l) * 32:(i * logM + l + 1) * 32] for l in range(logM)] for i in range(len(idx))]

    def fold_gpu(self, f_dev, beta, out=None):
        """p3bf_fold_kernel / fold_gpu (zkllm-src/p3_basefold.cuh:239-245, :285-292), MLE form."""
        import torch
        M = f_dev.numel()
        if out is None:
            out = torch.empty(M // 2, dtype=torch.int64, device=f_dev.device)
        self._ck(self._L.zkh_gl_fold_codeword(self._h, _ptr(f_dev), _ptr(out), M, beta))
        return out

    def commit_gpu_rootonly(self, c, R):
        """p3bf::commit_gpu_rootonly (zkllm-src/p3_basefold.cuh:210-227).  c: host numpy array
        (uploaded inside, like the reference) or a device tensor."""
        root = _buf32()
        if isinstance(c, np.ndarray):
            c = np.ascontiguousarray(c, dtype=np.uint64)
            self._ck(self._L.zkh_basefold_commit_host(self._h, c.ctypes.data, len(c).bit_length() - 1, R, root))
        elif getattr(self, "keep_trees", False) and c.numel() >= 2:
            # keep the codeword and the tree resident for the batched openings (released by release_kept())
            import torch
            v = c.numel().bit_length() - 1
            M = 1 << (v + R)
            cw = torch.empty(M, dtype=torch.int64, device=c.device)
            tree = torch.empty(self._L.zkh_basefold_kept_tree_bytes(v + R), dtype=torch.uint8, device=c.device)
            self._ck(self._L.zkh_basefold_commit_keep(self._h, _ptr(c), v, R, _ptr(cw), _ptr(tree), root))
            self.__dict__.setdefault("_kept", {})[(c.data_ptr(), R)] = (c, cw, tree)
        else:
            self._ck(self._L.zkh_basefold_commit(self._h, _ptr(c), c.numel().bit_length() - 1, R, 0, root))
        return bytes(root)

    def commit_many(self, cols, R):
        """Commitment roots of several device columns with one host synchronisation (same roots as commit_gpu_rootonly on
        each).  With kept trees enabled the columns are committed one by one so that their codewords and trees stay."""
        if getattr(self, "keep_trees", False) or not cols:
            return [self.commit_gpu_rootonly(c, R) for c in cols]
        k = len(cols)
        ptrs = (C.c_uint64 * k)(*[_ptr(c) for c in cols])
        vs = (C.c_uint32 * k)(*[int(c.numel()).bit_length() - 1 for c in cols])
        roots = (C.c_uint8 * (32 * k))()
        self._ck(self._L.zkh_basefold_commit_many(self._h, ptrs, vs, k, R, roots))
        rb = bytes(roots)
        return [rb[32 * j:32 * j + 32] for j in range(k)]

    def commit_salted(self, c, R, sseed, keep=False):
        """p3zkc::salted_commit_root_dev (zkllm-src/p3_zkc.cuh:362-397): hiding commitment root of a device column, leaves
        salted with SHA-256(seed | index).  keep: also return the codeword and the tree (device tensors)."""
        import torch
        v = int(c.numel()).bit_length() - 1
        root = _buf32()
        cw = tree = None
        if keep:
            M = 1 << (v + R)
            cw = torch.empty(M, dtype=torch.int64, device=c.device)
            tree = torch.empty(self._L.zkh_basefold_kept_tree_bytes(v + R), dtype=torch.uint8, device=c.device)
        self._ck(self._L.zkh_basefold_commit_salted(self._h, _ptr(c), v, R, sseed, _ptr(cw) if keep else 0, _ptr(tree) if keep else 0, root))
        return (bytes(root), cw, tree) if keep else bytes(root)

    def zk_fill_at(self, seed, n, i0=0):
        """p3zkc::zprng_at stream (zkllm-src/p3_zkc.cuh:108-118): out[i] = zprng_at(seed, i0 + i)."""
        import torch
        out = torch.empty(n, dtype=torch.int64, device="cuda:%d" % self.device)
        self._ck(self._L.zkh_zk_fill_at(self._h, seed, i0, n, _ptr(out)))
        return out

    def zk_fill_chain(self, s0, n, k0=0):
        """p3zkc::zprng_fill / zprng_fill_at (zkllm-src/p3_zkc.cuh:498-534): n elements of the chain from state s0, offset k0."""
        import torch
        out = torch.empty(n, dtype=torch.int64, device="cuda:%d" % self.device)
        self._ck(self._L.zkh_zk_fill_chain(self._h, s0, k0, n, _ptr(out)))
        return out

    def zk_augment(self, col, e, mask_seed):
        """p3zkc::augment(vals, fresh mask from mask_seed) (zkllm-src/p3_zkc.cuh:158-185): [real | mask slices]."""
        import torch
        v = int(col.numel()).bit_length() - 1
        out = torch.empty(1 << (v + e), dtype=torch.int64, device=col.device)
        self._ck(self._L.zkh_zk_augment(self._h, _ptr(col), v, e, mask_seed, _ptr(out)))
        return out

    def release_kept(self):
        """Drop the codewords and trees kept by commit_gpu_rootonly under ``keep_trees``."""
        self.__dict__.pop("_kept", None)

    def prove_eval_dev(self, c_dev, z, y, R, Q, cw0_dev=None, seed="p3-bf"):
        """p3bf::prove_eval_dev (zkllm-src/p3_basefold.cuh:355-420).  Returns the serialised EvalProof."""
        z = np.ascontiguousarray(z, dtype=np.uint64)
        v = len(z)
        cap = self._L.zkh_basefold_proof_size(v, R, Q)
        out = np.zeros(cap, dtype=np.uint8)
        wr = C.c_size_t(0)
        self._ck(self._L.zkh_basefold_open(self._h, _ptr(c_dev), z.ctypes.data, v, y, R, Q,
                                           _ptr(cw0_dev) if cw0_dev is not None else 0, seed.encode(),
                                           out.ctypes.data, cap, C.byref(wr)))
        return out.tobytes()[:wr.value]

    def prove_class(self, tr, pts, ents, R, Q, label):
        """p3bo::prove_class (zkllm-src/p3_batchopen.cuh:307-1147), non-zk.  pts: T x v points;
        ents: ledger entries (device column, 32-byte root, point index) in insertion order.
        ``tr`` (the main transcript) advances as in the reference.  Returns the serialised BatchProof."""
        pts = np.ascontiguousarray(pts, dtype=np.uint64)
        T, v = pts.shape
        k = len(ents)
        ptrs = (C.c_uint64 * k)(*[_ptr(e[0]) for e in ents])
        roots = b"".join(bytes(e[1]) for e in ents)
        zid = np.ascontiguousarray([e[2] for e in ents], dtype=np.uint32)
        cap = self._L.zkh_batchopen_proof_bound(v, R, Q, k)
        out = np.zeros(cap, dtype=np.uint8)
        wr = C.c_size_t(0)
        st = _buf32(tr.state)
        kept = self.__dict__.get("_kept")
        if kept:
            hit = [kept.get((_ptr(e[0]), R)) for e in ents]
            hit = [h if (h is not None and h[0] is e[0]) else None for h, e in zip(hit, ents)]
            kcw = (C.c_uint64 * k)(*[(_ptr(h[1]) if h else 0) for h in hit])
            ktr = (C.c_uint64 * k)(*[(_ptr(h[2]) if h else 0) for h in hit])
            self._ck(self._L.zkh_batchopen_prove_class_kept(self._h, v, pts.ctypes.data, T, ptrs, roots, zid.ctypes.data, k,
                                                            R, Q, label.encode(), st, out.ctypes.data, cap, C.byref(wr), kcw, ktr))
        else:
            self._ck(self._L.zkh_batchopen_prove_class(self._h, v, pts.ctypes.data, T, ptrs, roots, zid.ctypes.data, k,
                                                       R, Q, label.encode(), st, out.ctypes.data, cap, C.byref(wr)))
        tr.state = bytes(st)
        return out.tobytes()[:wr.value]

    def prove_class_salted(self, tr, pts, ents, R, Q, label):
        """The hiding mode's p3bo::prove_class after its blinder was appended (zkllm-src/p3_batchopen.cuh:385-1147 with
        zk_salted): ents = (device column, root, point index, salt seed, kept codeword or None, kept tree or None)."""
        pts = np.ascontiguousarray(pts, dtype=np.uint64)
        T, v = pts.shape
        k = len(ents)
        ptrs = (C.c_uint64 * k)(*[_ptr(e[0]) for e in ents])
        roots = b"".join(bytes(e[1]) for e in ents)
        zid = np.ascontiguousarray([e[2] for e in ents], dtype=np.uint32)
        ss = np.ascontiguousarray([e[3] for e in ents], dtype=np.uint64)
        kcw = (C.c_uint64 * k)(*[(_ptr(e[4]) if len(e) > 5 and e[4] is not None and e[5] is not None else 0) for e in ents])
        ktr = (C.c_uint64 * k)(*[(_ptr(e[5]) if len(e) > 5 and e[4] is not None and e[5] is not None else 0) for e in ents])
        cap = self._L.zkh_batchopen_proof_bound(v, R, Q, k) + k * 2 * Q * 32
        out = np.zeros(cap, dtype=np.uint8)
        wr = C.c_size_t(0)
        st = _buf32(tr.state)
        self._ck(self._L.zkh_batchopen_prove_class_salted(self._h, v, pts.ctypes.data, T, ptrs, roots, zid.ctypes.data,
                                                          ss.ctypes.data, k, R, Q, label.encode(), st, out.ctypes.data, cap,
                                                          C.byref(wr), kcw, ktr))
        tr.state = bytes(st)
        return out.tobytes()[:wr.value]

    def matvec(self, M_dev, rows, cols, w_dev, along_rows):
        """Row-major rows x cols field matrix times vector: along_rows -> out[r] = sum_c M[r][c] w[c],
        else out[c] = sum_r w[r] M[r][c]."""
        import torch
        out = torch.empty(rows if along_rows else cols, dtype=torch.int64, device=M_dev.device)
        self._ck(self._L.zkh_gl_matvec(self._h, _ptr(M_dev), rows, cols, _ptr(w_dev), int(along_rows), _ptr(out)))
        return out

    def matmul(self, A_dev, B_dev, I, J, K):
        """C = A * B over the field, row-major (A: I x J, B: J x K): zkh_gl_matmul."""
        import torch
        out = torch.empty(I * K, dtype=torch.int64, device=A_dev.device)
        self._ck(self._L.zkh_gl_matmul(self._h, _ptr(A_dev), _ptr(B_dev), I, J, K, _ptr(out)))
        return out

    def ig_matmul(self, A, a_str, B, b_str, Cc, c_str, nb0, nb1, I, J, K):
        """Exact integer matrix products of the layer's witness chain (zkh_ig_matmul): C[b0][b1] = A[b0][b1] . B[b0][b1] with
        A: I x J, B: J x K, all three read / written through element strides (outer batch, inner batch, row, column) over
        columns of field-lifted signed integers."""
        sa, sb, sc = ((C.c_int64 * 4)(*[int(x) for x in st]) for st in (a_str, b_str, c_str))
        self._ck(self._L.zkh_ig_matmul(self._h, _ptr(A), sa, _ptr(B), sb, _ptr(Cc), sc, nb0, nb1, I, J, K))

    # ---- witness replays of the integer layer's gadgets (one kernel each; see zkh.h) ----
    def _new(self, n, like, i32=False):
        import torch
        return torch.empty(n, dtype=torch.int32 if i32 else torch.int64, device=like.device)

    def ig_add_witness(self, a, b):
        n = a.numel()
        out, idx = self._new(n, a), self._new(n, a, True)
        self._ck(self._L.zkh_ig_add_witness(self._h, _ptr(a), _ptr(b), n, _ptr(out), _ptr(idx)))
        return out, idx

    def ig_rs20_index(self, v):
        idx = self._new(v.numel(), v, True)
        self._ck(self._L.zkh_ig_rs20_index(self._h, _ptr(v), v.numel(), _ptr(idx)))
        return idx

    def ig_swiglu_witness(self, g, u, silu_col):
        n = g.numel()
        sil, rem, mo = (self._new(n, g) for _ in range(3))
        iG, iR, iM = (self._new(n, g, True) for _ in range(3))
        self._ck(self._L.zkh_ig_swiglu_witness(self._h, _ptr(g), _ptr(u), _ptr(silu_col), n, _ptr(sil), _ptr(rem), _ptr(mo),
                                               _ptr(iG), _ptr(iR), _ptr(iM)))
        return sil, rem, mo, iG, iR, iM

    def ig_rope_witness(self, q, ct, st, lseq, ldh, lT, ld):
        n = q.numel()
        y, rem, Cc, S2 = (self._new(n, q) for _ in range(4))
        iR, iY = self._new(n, q, True), self._new(n, q, True)
        self._ck(self._L.zkh_ig_rope_witness(self._h, _ptr(q), _ptr(ct), _ptr(st), lseq, ldh, lT, ld, _ptr(y), _ptr(rem), _ptr(iR),
                                             _ptr(iY), _ptr(Cc), _ptr(S2)))
        return y, rem, iR, iY, Cc, S2

    def ig_rms_witness(self, x, g, isq_col, lT, ld):
        B, n = 1 << lT, 1 << (lT + ld)
        db = [self._new(B, x) for _ in range(18)]
        de = [self._new(n, x) for _ in range(3)]
        y = self._new(n, x)
        irow = [self._new(B, x, True) for _ in range(14)]
        iel = [self._new(n, x, True) for _ in range(4)]
        arr = lambda ts: (C.c_uint64 * len(ts))(*[_ptr(t) for t in ts])
        self._ck(self._L.zkh_ig_rms_witness(self._h, _ptr(x), _ptr(g), _ptr(isq_col), lT, ld, arr(db), arr(de), _ptr(y), arr(irow), arr(iel)))
        return db, de, y, irow, iel

    def ig_softmax_witness(self, z, expt_col, la, lseq):
        NR, n = 1 << (la + lseq), 1 << (la + 2 * lseq)
        xe = [self._new(n, z) for _ in range(7)]
        xb = [self._new(NR, z) for _ in range(2)]
        p = self._new(n, z)
        idm = self._new(n, z, True)
        il = [self._new(n, z, True) for _ in range(4)]
        imx = self._new(NR, z, True)
        arr = lambda ts: (C.c_uint64 * len(ts))(*[_ptr(t) for t in ts])
        self._ck(self._L.zkh_ig_softmax_witness(self._h, _ptr(z), _ptr(expt_col), la, lseq, arr(xe), arr(xb), _ptr(p), _ptr(idm), arr(il),
                                                _ptr(imx)))
        return xe, xb, p, idm, il, imx

    def scale(self, col_dev, s):
        import torch
        out = torch.empty_like(col_dev)
        self._ck(self._L.zkh_gl_scale(self._h, _ptr(col_dev), col_dev.numel(), s, _ptr(out)))
        return out

    def mul(self, a_dev, b_dev):
        import torch
        out = torch.empty_like(a_dev)
        self._ck(self._L.zkh_gl_mul(self._h, _ptr(a_dev), _ptr(b_dev), a_dev.numel(), _ptr(out)))
        return out

    def irs_witness(self, acc_dev, sf, rng):
        """p3irs::gen_witness on the device: returns (y, [L0(, L1)], [idxL0(, idxL1)], idxY or None)."""
        import torch
        n, dev = acc_dev.numel(), acc_dev.device
        nl = 1 if sf <= 16 else 2
        y = torch.empty(n, dtype=torch.int64, device=dev)
        L = [torch.empty(n, dtype=torch.int64, device=dev) for _ in range(nl)]
        iL = [torch.empty(n, dtype=torch.int32, device=dev) for _ in range(nl)]
        iY = torch.empty(n, dtype=torch.int32, device=dev) if rng else None
        self._ck(self._L.zkh_irs_witness(self._h, _ptr(acc_dev), n, sf, rng, _ptr(y), _ptr(L[0]),
                                         _ptr(L[1]) if nl == 2 else 0, _ptr(iL[0]), _ptr(iL[1]) if nl == 2 else 0,
                                         _ptr(iY) if rng else 0))
        return y, L, iL, iY

    def hwl_witness(self, lb, ln, lg, xcodes, wcodes, xsb, wsb, cols, lidx):
        """p3hwl::gen_witness (zkllm-src/p3_hawkeye.cuh:342-637) as one kernel: fills the 99 field columns and the 38
        lookup-index columns (preallocated tensors, reference enum order) from the padded operand columns."""
        pc = (C.c_uint64 * len(cols))(*[_ptr(t) for t in cols])
        pl = (C.c_uint64 * len(lidx))(*[_ptr(t) for t in lidx])
        self._ck(self._L.zkh_hwl_witness(self._h, lb, ln, lg, _ptr(xcodes), _ptr(wcodes), _ptr(xsb), _ptr(wsb), pc, pl))

    def upload(self, arr):
        return to_device(arr, "cuda:%d" % self.device)

    def bcast_rows(self, col, ld):
        """out[e] = col[e >> ld]: a per-row value repeated along the row (p3ig::eqb_col / bc_aug)."""
        return col.repeat_interleave(1 << ld).contiguous()

    def bcast_cols(self, col, lT):
        """out[e] = col[e mod len(col)]: a per-column value repeated over 2^lT rows."""
        return col.repeat(1 << lT).contiguous()

    def causal_mask(self, la, lseq):
        """p3ismx::mask_col: 1 where key index j <= query index i over u = j | (i << lseq) | (a << 2 lseq)."""
        import torch
        u = torch.arange(1 << (la + 2 * lseq), dtype=torch.int64, device="cuda:%d" % self.device)
        seq = 1 << lseq
        return ((u & (seq - 1)) <= ((u >> lseq) & (seq - 1))).to(torch.int64)

    def gather(self, col, idx):
        """out[t] = col[idx[t]] (idx: host int64 array): the dense operand behind a p3imm operand view."""
        import torch
        return col[torch.from_numpy(np.ascontiguousarray(idx, dtype=np.int64)).to(col.device)].contiguous()

    @staticmethod
    def _bit_map(fn, n):
        """(konst, masks) when the index map fn is a map on index bits -- fn(u) = konst | OR over the set bits b of u of
        masks[b], which every operand view and broadcast pattern is -- else None.  One evaluation of fn on a small host
        array: zero, the powers of two, and 192 seeded samples that check the model."""
        nb = max(1, (int(n) - 1).bit_length())
        if nb > 32:
            return None
        rng = np.random.default_rng(nb)
        samples = rng.integers(0, n, 192, dtype=np.int64)
        probe = np.concatenate([np.zeros(1, dtype=np.int64), np.int64(1) << np.arange(nb, dtype=np.int64), samples])
        r = np.asarray(fn(probe), dtype=np.int64) + np.zeros_like(probe)
        konst = int(r[0])
        masks = np.ascontiguousarray(r[1:1 + nb], dtype=np.int64)
        model = np.full(192, konst, dtype=np.int64)
        for b in range(nb):
            model |= np.where((samples >> b) & 1, masks[b], 0)
        if (r[1:1 + nb] & konst != konst).any() or not (model == r[1 + nb:]).all():
            return None
        return konst, masks.view(np.uint64), nb

    def gather_fn(self, col, n, fn):
        """out[u] = col[fn(u)] for u < n, the index map written with integer operators (&, |, <<, >>): broadcast columns and
        operand views of the hiding mode's product domains.  Maps on index bits run as one kernel (zkh_gl_gather_bits);
        anything else is evaluated with tensor operations on the device."""
        import torch
        bm = self._bit_map(fn, n)
        if bm is not None:
            out = torch.empty(n, dtype=torch.int64, device=col.device)
            self._ck(self._L.zkh_gl_gather_bits(self._h, _ptr(col), col.numel(), n, bm[0], bm[1].ctypes.data, bm[2], _ptr(out)))
            return out
        u = torch.arange(n, dtype=torch.int64, device=col.device)
        return col[fn(u)].contiguous()

    def slice(self, col, lo, n):
        return col[lo:lo + n]

    def scatter_fn(self, col, n, fn, vals):
        """col[fn(u)] = vals[u] for u < n (distinct targets); returns col.  Maps on index bits run as one kernel."""
        import torch
        bm = self._bit_map(fn, n)
        if bm is not None and vals.numel() == n:
            self._ck(self._L.zkh_gl_scatter_bits(self._h, _ptr(vals), n, bm[0], bm[1].ctypes.data, bm[2], _ptr(col), col.numel()))
            return col
        u = torch.arange(n, dtype=torch.int64, device=col.device)
        col[fn(u)] = vals
        return col

    def concat(self, cols):
        import torch
        return torch.cat(list(cols)).contiguous()

    def download(self, col):
        return to_host(col)

    def interleave(self, a, b):
        """out[2x] = a[x], out[2x+1] = b[x]: sibling-interleaved leaves of the hiding mode's fraction trees."""
        import torch
        return torch.stack([a, b], dim=1).reshape(-1).contiguous()

    def zeros(self, n):
        import torch
        return torch.zeros(n, dtype=torch.int64, device="cuda:%d" % self.device)

    def set_element(self, col, i, value):
        value = int(value) % GL_P
        col[i] = value - (1 << 64) if value >= (1 << 63) else value

    def flip_bit(self, col, b):
        """out[u] = col[u ^ (1 << b)]: the rotate-half permutation of RoPE (zkllm-src/p3_int_gadgets.cuh:1297-1298)."""
        return col.view(-1, 2, 1 << b).flip(1).reshape(-1).contiguous()

    # ---- engine interface used by prove_super ----
    def lu_counts(self, idx_list, M, pad_rows):
        """Multiplicity column of a merged lookup: histogram of all members' indices plus the
        padding rows (which hold table row 0)."""
        cnt = None
        for idx in idx_list:
            h = self.histogram(idx, M)
            cnt = h if cnt is None else cnt + h
        cnt[0] += pad_rows
        return cnt

    def lu_leaf_denominators(self, members, kp, n, gamma, shift, pad_value):
        """LQ over the merged domain u = i | (j << n): member j < k holds shift + sum_t gamma^t W_jt[i],
        pad members hold pad_value."""
        import torch
        N = 1 << n
        out = torch.empty(kp << n, dtype=torch.int64, device="cuda:%d" % self.device)
        for j in range(kp):
            sl = out[j * N:(j + 1) * N]
            if j < len(members):
                nc = len(members[j])
                ptrs = (C.c_uint64 * nc)(*[_ptr(t) for t in members[j]])
                self._ck(self._L.zkh_gl_affine(self._h, ptrs, nc, N, gamma, shift, _ptr(sl)))
            else:
                sl.fill_(pad_value - (1 << 64) if pad_value >= (1 << 63) else pad_value)
        return out

    def lu_ones(self, n):
        """All-ones numerator column of a lookup's witness side (read-only; cached per size)."""
        import torch
        cache = self.__dict__.setdefault("_ones", {})
        if n not in cache:
            if sum(cache) + n > (1 << 27):        # at most 1 GiB of cached ones
                cache.clear()
            cache[n] = torch.ones(n, dtype=torch.int64, device="cuda:%d" % self.device)
        return cache[n]

    def affine(self, cols_dev, g, addend):
        import torch
        nc = len(cols_dev)
        ptrs = (C.c_uint64 * nc)(*[_ptr(t) for t in cols_dev])
        out = torch.empty_like(cols_dev[0])
        self._ck(self._L.zkh_gl_affine(self._h, ptrs, nc, cols_dev[0].numel(), g, addend, _ptr(out)))
        return out

    # ---- logUp / GKR ----
    def histogram(self, idx_dev, M):
        """p3lu_cnts/cntg_kernel (zkllm-src/p3_logup.cuh:149-172): 64-bit multiplicities of uint32 indices
        (idx_dev: torch int32 tensor holding the uint32 bit patterns)."""
        import torch
        cnt = torch.empty(M, dtype=torch.int64, device=idx_dev.device)
        self._ck(self._L.zkh_histogram(self._h, _ptr(idx_dev), idx_dev.numel(), M, _ptr(cnt)))
        return cnt

    def inv_all_add(self, A_dev, beta):
        """p3lu::inv_all_add (zkllm-src/p3_logup.cuh:636-660)."""
        import torch
        out = torch.empty_like(A_dev)
        self._ck(self._L.zkh_gl_inv_all_add(self._h, _ptr(A_dev), A_dev.numel(), beta, _ptr(out)))
        return out

    def combine(self, cols_dev, g):
        """p3lu::combine (zkllm-src/p3_logup.cuh:663-672)."""
        import torch
        nc = len(cols_dev)
        ptrs = (C.c_uint64 * nc)(*[_ptr(t) for t in cols_dev])
        out = torch.empty_like(cols_dev[0])
        self._ck(self._L.zkh_gl_combine(self._h, ptrs, nc, cols_dev[0].numel(), g, _ptr(out)))
        return out

    def gkr_prove(self, tr, tag, p_dev, q_dev, combine_last=True):
        """p3gkr::prove_dev (zkllm-src/p3_gkr.cuh:423-429).  Returns (proof bytes, rfin, (cp, cq));
        ``tr`` advances exactly as the reference's transcript."""
        L = p_dev.numel().bit_length() - 1
        cap = self._L.zkh_gkr_proof_size(L)
        out = np.zeros(cap, dtype=np.uint8)
        rfin = np.zeros(L + 1, dtype=np.uint64)
        cpq = np.zeros(2, dtype=np.uint64)
        wr = C.c_size_t(0)
        st = _buf32(tr.state)
        self._ck(self._L.zkh_gkr_prove(self._h, _ptr(p_dev), _ptr(q_dev), L, int(combine_last), tag.encode(), st,
                                       rfin.ctypes.data, cpq.ctypes.data, out.ctypes.data, cap, C.byref(wr)))
        tr.state = bytes(st)
        nr = L if combine_last else L - 1
        return out.tobytes()[:wr.value], rfin[:nr].copy(), (int(cpq[0]), int(cpq[1]))

    # ---- sharded sumcheck: the per-GPU engine interface used by sc_prove_sharded ----
    def new_buffer(self, n):
        import torch
        return torch.zeros(n, dtype=torch.int64, device="cuda:%d" % self.device)

    def shard_begin(self, functor, nt, dcols, logn, par, tag, state):
        nc = len(dcols)
        ptrs = (C.c_uint64 * nc)(*[_ptr(t) for t in dcols])
        par_a = np.ascontiguousarray(list(par) if len(par) else [0], dtype=np.uint64)
        self._shard_shape = (nt, nc)
        self._ck(self._L.zkh_shard_begin(self._h, functor, nt, ptrs, nc, logn, par_a.ctypes.data, len(par),
                                         tag.encode(), _buf32(state)))

    def p2p_connect(self, dist, group=None):
        """Map every rank's round-exchange mailbox into this process (CUDA IPC, one process per GPU) so that
        sc_prove_sharded runs each round as one kernel with NVLink peer stores instead of an NCCL all-gather.
        Collective over ``group``.  Returns False (and leaves the NCCL path in use) when the GPUs have no
        peer access."""
        G, rank = dist.get_world_size(group), dist.get_rank(group)
        if G < 2 or G > 16:
            return False
        h = (C.c_uint8 * 64)()
        self._ck(self._L.zkh_p2p_create(self._h, h))
        handles = [None] * G
        dist.all_gather_object(handles, bytes(h), group=group)
        rc = self._L.zkh_p2p_connect(self._h, rank, G, b"".join(handles))
        oks = [None] * G
        dist.all_gather_object(oks, rc == 0, group=group)
        self.p2p_ready = all(oks)
        if not self.p2p_ready:
            self._L.zkh_p2p_disconnect(self._h)
        return self.p2p_ready

    def p2p_disconnect(self):
        self.p2p_ready = False
        self._ck(self._L.zkh_p2p_disconnect(self._h))

    def shard_round_fused(self, r):
        self._ck(self._L.zkh_shard_round_fused(self._h, r))

    def shard_local_fused(self, fin):
        self._ck(self._L.zkh_shard_local_fused(self._h, _ptr(fin)))

    def shard_prove_fused(self):
        self._ck(self._L.zkh_shard_prove_fused(self._h))

    def shard_round_local(self, r, sums):
        self._ck(self._L.zkh_shard_round_local(self._h, r, _ptr(sums)))

    def shard_round_combine(self, r, gathered, G):
        self._ck(self._L.zkh_shard_round_combine(self._h, r, _ptr(gathered), G))

    def shard_finals(self, fin):
        self._ck(self._L.zkh_shard_finals(self._h, _ptr(fin)))

    def shard_residual(self, gathered_fin, G):
        self._ck(self._L.zkh_shard_residual(self._h, _ptr(gathered_fin), G))

    def shard_end(self, rounds):
        nt, nc = self._shard_shape
        msgs = np.zeros((rounds, nt), dtype=np.uint64)
        chals = np.zeros(rounds, dtype=np.uint64)
        fin = np.zeros(nc, dtype=np.uint64)
        st = _buf32()
        self._ck(self._L.zkh_shard_end(self._h, st, msgs.ctypes.data, chals.ctypes.data, fin.ctypes.data))
        return bytes(st), msgs, chals, fin

    # ---- sumcheck ----
    def sc_prove_gpu(self, tr, tag, dcols, functor, nt, par=(), logn=None):
        """p3sg::sc_prove_gpu: appends nothing to the caller's lists; returns
        (r, msgs, finals) with r the round challenges, msgs[v, nt] the absorbed
        messages and finals the fully bound column values.  ``tr`` is advanced
        exactly as the reference's transcript is.  dcols: device tensors (left intact)."""
        nc = len(dcols)
        if logn is None:
            logn = int(dcols[0].numel()).bit_length() - 1
        ptrs = (C.c_uint64 * nc)(*[_ptr(t) for t in dcols])
        par_a = np.ascontiguousarray(list(par) if len(par) else [0], dtype=np.uint64)
        msgs = np.zeros((logn, nt), dtype=np.uint64)
        chals = np.zeros(logn, dtype=np.uint64)
        fin = np.zeros(nc, dtype=np.uint64)
        st = _buf32(tr.state)
        self._ck(self._L.zkh_sumcheck(self._h, functor, nt, ptrs, nc, logn, par_a.ctypes.data, len(par),
                                      tag.encode(), st, msgs.ctypes.data, chals.ctypes.data,
                                      fin.ctypes.data))
        tr.state = bytes(st)
        return chals, msgs, fin

    def sc5_run(self, tr, tag, dcols, functor, lam):
        """p3hwl::sc5_run / sc5_prove (zkllm-src/p3_hawkeye.cuh:1016-1033, :641-700), non-zk, for the fp8
        gadget's constraint summands F_HW_*: quartic zero-check over device columns with the random
        coefficients ``lam``.  Returns (r, msgs[v, 5], finals); ``tr`` advances as the reference's does."""
        nc = len(dcols)
        logn = int(dcols[0].numel()).bit_length() - 1
        ptrs = (C.c_uint64 * nc)(*[_ptr(t) for t in dcols])
        lam_a = np.ascontiguousarray(lam, dtype=np.uint64)
        msgs = np.zeros((logn, 5), dtype=np.uint64)
        chals = np.zeros(logn, dtype=np.uint64)
        fin = np.zeros(nc, dtype=np.uint64)
        st = _buf32(tr.state)
        self._ck(self._L.zkh_sumcheck_wide(self._h, functor, ptrs, nc, logn, lam_a.ctypes.data, len(lam_a),
                                           tag.encode(), st, msgs.ctypes.data, chals.ctypes.data, fin.ctypes.data))
        tr.state = bytes(st)
        return chals, msgs, fin

    def sc_prove_zc(self, tr, tag, dcols, terms, konst=0):
        """Eq-weighted zero-check with a programmable summand (the non-zk path of p3hwl::sc5z / sc5_prove,
        zkllm-src/p3_hawkeye.cuh:641-700, for the integer-layer gadgets): proves the sumcheck of
            dcols[0] * (konst + sum_j coef_j * prod_k dcols[idx_jk])
        with ``terms`` = [(coef, (idx, ...)), ...], one to three column indices per term.  Five evaluations per
        round.  Returns (r, msgs[v, 5], finals)."""
        nc = len(dcols)
        logn = int(dcols[0].numel()).bit_length() - 1
        ptrs = (C.c_uint64 * nc)(*[_ptr(t) for t in dcols])
        prog = zc_program(terms, konst)
        msgs = np.zeros((logn, 5), dtype=np.uint64)
        chals = np.zeros(logn, dtype=np.uint64)
        fin = np.zeros(nc, dtype=np.uint64)
        st = _buf32(tr.state)
        self._ck(self._L.zkh_sumcheck_zerocheck(self._h, ptrs, nc, logn, prog.ctypes.data, len(prog), tag.encode(), st,
                                                msgs.ctypes.data, chals.ctypes.data, fin.ctypes.data))
        tr.state = bytes(st)
        return chals, msgs, fin

    def sc_prove_zc_blind(self, tr, tag, dcols, terms, konst, table):
        """The zero-check chain under a structured Libra blind (the structured branch of p3hwl::sc5z, zkllm-src/p3_hawkeye.cuh:
        1329-1331 with sb_fix :1092-1110).  table: per round [c0..c4 of g_rd, A_rd, B_rd]; the message of round rd gains
        A_rd * (pref + g_rd(t)) + B_rd on the device.  Returns (r, msgs, finals, g(r))."""
        nc = len(dcols)
        logn = int(dcols[0].numel()).bit_length() - 1
        ptrs = (C.c_uint64 * nc)(*[_ptr(t) for t in dcols])
        prog = zc_program(terms, konst)
        fix = np.ascontiguousarray(table, dtype=np.uint64).reshape(logn, 7)
        msgs = np.zeros((logn, 5), dtype=np.uint64)
        chals = np.zeros(logn, dtype=np.uint64)
        fin = np.zeros(nc, dtype=np.uint64)
        pref = C.c_uint64(0)
        st = _buf32(tr.state)
        self._ck(self._L.zkh_sumcheck_zerocheck_blind(self._h, ptrs, nc, logn, prog.ctypes.data, len(prog), fix.ctypes.data,
                                                      tag.encode(), st, msgs.ctypes.data, chals.ctypes.data, fin.ctypes.data,
                                                      C.byref(pref)))
        tr.state = bytes(st)
        return chals, msgs, fin, int(pref.value)

    def sc_prove_zc_partial(self, tr, tag, dcols, terms, konst, rounds, table=None, pref=0):
        """The first ``rounds`` rounds of a zero-check chain (zkh_sumcheck_zerocheck_partial): returns (r, msgs, left, pref) with
        left[k] the values column k still holds after the last bind.  table: the structured blind's rows of these rounds."""
        nc = len(dcols)
        logn = int(dcols[0].numel()).bit_length() - 1
        ptrs = (C.c_uint64 * nc)(*[_ptr(t) for t in dcols])
        prog = zc_program(terms, konst)
        fix = np.ascontiguousarray(table, dtype=np.uint64).reshape(rounds, 7) if table is not None else None
        msgs = np.zeros((rounds, 5), dtype=np.uint64)
        chals = np.zeros(rounds, dtype=np.uint64)
        left = np.zeros((nc, (1 << logn) >> rounds), dtype=np.uint64)
        pout = C.c_uint64(0)
        st = _buf32(tr.state)
        self._ck(self._L.zkh_sumcheck_zerocheck_partial(self._h, ptrs, nc, logn, rounds, prog.ctypes.data, len(prog),
                                                        fix.ctypes.data if fix is not None else 0, int(pref), tag.encode(), st,
                                                        msgs.ctypes.data, chals.ctypes.data, left.ctypes.data, C.byref(pout)))
        tr.state = bytes(st)
        return chals, msgs, left, int(pout.value) if fix is not None else int(pref)

    def sc_prove_host(self, tr, tag, cols, functor, nt, par=()):
        """Same through host columns (numpy uint64): upload + prove + download in one call."""
        arrs = [np.ascontiguousarray(c, dtype=np.uint64) for c in cols]
        nc = len(arrs)
        logn = int(len(arrs[0])).bit_length() - 1
        ptrs = (C.c_uint64 * nc)(*[a.ctypes.data for a in arrs])
        par_a = np.ascontiguousarray(list(par) if len(par) else [0], dtype=np.uint64)
        msgs = np.zeros((logn, nt), dtype=np.uint64)
        chals = np.zeros(logn, dtype=np.uint64)
        fin = np.zeros(nc, dtype=np.uint64)
        st = _buf32(tr.state)
        self._ck(self._L.zkh_sumcheck_host(self._h, functor, nt, ptrs, nc, logn, par_a.ctypes.data,
                                           len(par), tag.encode(), st, msgs.ctypes.data,
                                           chals.ctypes.data, fin.ctypes.data))
        tr.state = bytes(st)
        return chals, msgs, fin


def sc_prove_sharded(engine, tr, tag, dcols, functor, nt, dist=None, par=(), group=None, rendezvous=True):
    """p3sg::sc_prove_gpu over several GPUs of one node: the hypercube is split on its top
    log2(G) variables, rank g holding slice g of every column (``dcols``: this rank's slices).
    Per round the ranks exchange their nt partial sums (nt*8 bytes each); every rank adds
    them mod p in rank order, runs the same transcript step and binds its own slice.  After the local
    rounds the G per-rank values of each column are exchanged and every rank finishes the
    last log2(G) rounds.  Returns (r, msgs, finals) exactly as sc_prove_gpu would on the
    concatenated columns; ``tr`` advances identically on every rank.

    With the peer exchange connected (Prover.p2p_connect) the whole proof is device code: one kernel per
    round with the sums crossing NVLink as peer stores, the last kernel also exchanging the bound values
    and running the residual rounds; no collective call is made.  The device waits are bounded to about
    a second, so ``rendezvous`` (default) first completes this rank's stream and meets the other ranks at
    a host barrier; a caller that issues proofs back to back passes rendezvous=False for all but the
    first of the series (only kernel skew separates the ranks then).
    Without the peer exchange every round is all-gathered with ``dist``.

    ``engine``: a Prover (CUDA) -- or, in the CPU tests of this host logic, an object with the
    same shard_* methods.  ``dist``: torch.distributed (initialised) or None for one rank."""
    G = dist.get_world_size(group) if (dist is not None and dist.is_initialized()) else 1
    if G & (G - 1):
        raise ValueError("the number of ranks must be a power of two")
    nc = len(dcols)
    logn = int(dcols[0].numel()).bit_length() - 1
    if logn < 1:
        raise ValueError("each rank needs at least two elements per column")
    k = G.bit_length() - 1

    def all_gather(out, inp):
        if G == 1:
            out.copy_(inp)
        else:
            dist.all_gather_into_tensor(out, inp, group=group)

    if G > 1 and getattr(engine, "p2p_ready", False):
        if rendezvous:
            engine.sync()
            dist.barrier(group=group)
        engine.shard_begin(functor, nt, dcols, logn, par, tag, tr.state)
        engine.shard_prove_fused()
    else:
        engine.shard_begin(functor, nt, dcols, logn, par, tag, tr.state)
        fin, gfin = engine.new_buffer(nc), engine.new_buffer(G * nc)
        sums, gathered = engine.new_buffer(nt), engine.new_buffer(G * nt)
        for r in range(logn):
            engine.shard_round_local(r, sums)
            all_gather(gathered, sums)
            engine.shard_round_combine(r, gathered, G)
        engine.shard_finals(fin)
        all_gather(gfin, fin)
        engine.shard_residual(gfin, G)
    state, msgs, chals, finals = engine.shard_end(logn + k)
    tr.state = state
    return chals, msgs, finals


def commit_columns_sharded(engine, cols, R, dist=None, group=None, device=None):
    """Commitments of K independent columns over the GPUs of one node: column j belongs to rank j mod G,
    which encodes and hashes it (p3bf::commit_gpu_rootonly); the 32-byte roots are all-gathered so every
    rank (in particular the transcript owner) ends with all K roots in column order.  The reference commits
    its thousands of per-layer columns one after another on one GPU; columns are independent, so no data
    moves between GPUs except the roots.  ``cols[j]`` is this rank's buffer for column j when it owns it and
    may be None otherwise."""
    import torch
    G = dist.get_world_size(group) if (dist is not None and dist.is_initialized()) else 1
    rank = dist.get_rank(group) if G > 1 else 0
    K = len(cols)
    per = (K + G - 1) // G
    mine = torch.zeros((per, 32), dtype=torch.uint8)
    for slot, j in enumerate(range(rank, K, G)):
        if cols[j] is None:
            raise ValueError("rank %d owns column %d but holds no data for it" % (rank, j))
        mine[slot] = torch.frombuffer(bytearray(engine.commit_gpu_rootonly(cols[j], R)), dtype=torch.uint8)
    if G == 1:
        allr = mine.unsqueeze(0)
    else:
        if device is not None:
            mine = mine.to(device)
        allr = torch.zeros((G, per, 32), dtype=torch.uint8, device=mine.device)
        dist.all_gather_into_tensor(allr.view(-1), mine.view(-1), group=group)
        allr = allr.cpu()
    return [bytes(allr[j % G, j // G].numpy().tobytes()) for j in range(K)]


def lu_counts_sharded(engine, idx_local, M, pad_rows, dist=None, group=None):
    """Multiplicity column of a lookup whose index arrays are split over the GPUs of one node: every rank histograms the
    index arrays it holds (p3lu_cnts/cntg_kernel, zkllm-src/p3_logup.cuh:149-172) and the 64-bit partial counts are summed
    with one all-reduce (plain integer sum: counts stay far below 2^63), so every rank ends with the full column; the
    padding rows (table row 0) are added once.  idx_local: this rank's index arrays (possibly empty)."""
    import torch
    cnt = None
    for idx in idx_local:
        h = engine.histogram(idx, M)
        cnt = h if cnt is None else cnt + h
    G = dist.get_world_size(group) if (dist is not None and dist.is_initialized()) else 1
    if cnt is None:
        raise ValueError("lu_counts_sharded: every rank needs at least one (possibly empty) index array")
    if G > 1:
        dist.all_reduce(cnt, group=group)
    cnt[0] += pad_rows
    return cnt


def run_independent(items, fn, dist=None, group=None):
    """Independent proofs (e.g. one layer proof per transcript) placed on separate GPUs: rank g runs
    fn(item) for items g, g+G, g+2G, ... and every rank receives all results in item order."""
    G = dist.get_world_size(group) if (dist is not None and dist.is_initialized()) else 1
    rank = dist.get_rank(group) if G > 1 else 0
    local = [(i, fn(items[i])) for i in range(rank, len(items), G)]
    if G == 1:
        return [r for _, r in local]
    gathered = [None] * G
    dist.all_gather_object(gathered, local, group=group)
    out = [None] * len(items)
    for part in gathered:
        for i, r in part:
            out[i] = r
    return out


def _ser_gkr_group(m, c, root_cnt, gkT, subs):
    import struct
    b = struct.pack("<III", m, c, len(subs)) + root_cnt + gkT
    for n, k, gk, mem in subs:
        b += struct.pack("<II", n, k) + gk
        for yW, yv, extra in mem:
            b += struct.pack("<I", len(yW)) + np.array(yW, dtype=np.uint64).tobytes()
            b += struct.pack("<I", len(yv)) + np.array(yv, dtype=np.uint64).tobytes()
            b += struct.pack("<I", len(extra)) + np.array(extra, dtype=np.uint64).tobytes()
    return b


def prove_super(engine, tr, table_cols, table_id, subgroups, R, strict=True):
    """p3lu::prove_super (zkllm-src/p3_logup.cuh:1357-1881), non-zk: ONE merged logUp instance for all
    lookups into one table.

    table_cols: c columns of 2^m rows (engine buffers); table_id: its 32-byte binding hash
    (p3lu::make_table).  subgroups: list, in flush order, of (n, members); a member is
    (cols, roots, idx) with c witness columns of 2^n rows, their commitment roots (None for a
    virtual column) and the uint32 row indices into the table; an optional fourth element is the member's bind
    callback (p3lu::PBind, p3_logup.cuh:451-456): called as bind(pm, y_virt) after the member's own claims, it returns
    further opening claims (column, root, point, value) that tie the virtual columns to commitments, or a pair
    (claims, extra) when values ride in the proof (LuMember::extra).
    Returns (proof bytes, claims, cnt column).  claims = the opening-ledger additions in the
    reference's order: (column, root, point, value) for every committed member column at the
    subgroup's shared point, then the multiplicity column at the table-side point.
    ``tr`` advances exactly as the reference's transcript."""
    import struct
    c = len(table_cols)
    M = int(table_cols[0].numel())
    m = M.bit_length() - 1
    tr.absorb("lug-tab", table_id)
    tr.absorb("lug-sdims", struct.pack("<III", len(subgroups), m, c))
    pad_rows, idx_all = 0, []
    for n, members in subgroups:
        k = len(members)
        g = (k - 1).bit_length()
        tr.absorb("lug-dims", struct.pack("<IIII", n, g, k, c))
        for cols, roots, idx, *_ in members:
            if len(cols) != c or any(int(t.numel()) != (1 << n) for t in cols) or int(idx.numel()) != (1 << n):
                raise ValueError("p3lu: group member size")
            for r in roots:
                if r is not None:
                    tr.absorb("lug-W", r)
                else:
                    tr.absorb("lug-Wv", b"virt")
            idx_all.append(idx)
        pad_rows += ((1 << g) - k) << n
    cnt = engine.lu_counts(idx_all, M, pad_rows)           # raises on an index outside the table
    root_cnt = engine.commit_gpu_rootonly(cnt, R)
    tr.absorb("lug-cnt", root_cnt)
    gamma, beta = tr.chal(), tr.chal()
    gp = [pow(gamma, t, GL_P) for t in range(c)]
    row0 = [int(engine.element(col, 0)) for col in table_cols]
    a0 = sum(g_ * r for g_, r in zip(gp, row0)) % GL_P
    accP, accQ = 0, 1
    subs, claims = [], []
    for n, members in subgroups:
        k = len(members)
        g = (k - 1).bit_length()
        LQ = engine.lu_leaf_denominators([mb[0] for mb in members], 1 << g, n, gamma, beta, (a0 + beta) % GL_P)
        LP = engine.lu_ones(1 << (n + g))
        gk, rA, _ = engine.gkr_prove(tr, "lug-gA", LP, LQ, True)
        P, Q = (int(x) for x in np.frombuffer(gk[:16], dtype=np.uint64))
        accP, accQ = (accP * Q + P * accQ) % GL_P, accQ * Q % GL_P
        pm = np.array(rA[:n], dtype=np.uint64)
        mem = []
        for cols, roots, idx, *bind in members:
            yW, yv = [], []
            for col, r in zip(cols, roots):
                y = engine.eval_h_gpu(col, pm)
                if r is not None:
                    yW.append(y)
                    tr.absorb("lug-yW", struct.pack("<Q", y))
                    claims.append((col, r, pm, y))
                else:
                    yv.append(y)
                    tr.absorb("lug-yv", struct.pack("<Q", y))
            extra = []
            if bind and bind[0] is not None:
                more = bind[0](pm, yv)
                if isinstance(more, tuple):       # (claims, values that ride in the proof as LuMember::extra)
                    more, extra = more
                claims.extend(more)
            mem.append((yW, yv, extra))
        subs.append((n, k, gk, mem))
    LQT = engine.affine(table_cols, gamma, beta)
    gkT, rT, (cpT, _cq) = engine.gkr_prove(tr, "lug-gT", cnt, LQT, True)
    PT, QT = (int(x) for x in np.frombuffer(gkT[:16], dtype=np.uint64))
    if strict and accP * QT % GL_P != PT * accQ % GL_P:
        raise ValueError("p3lu: witness not in table")
    claims.append((cnt, root_cnt, np.array(rT, dtype=np.uint64), cpT))
    return _ser_gkr_group(m, c, root_cnt, gkT, subs), claims, cnt


class Ledger:
    """p3bo::PLedger (zkllm-src/p3_batchopen.cuh:144-178): opening claims grouped by size class in
    order of first appearance; points deduplicated per class in order."""

    def __init__(self):
        self.cls = []          # [v, pts(list of np arrays), ents(list of (col, root, zid)), ys]

    def add(self, col, root, z, y):
        z = np.ascontiguousarray(z, dtype=np.uint64)
        for c in self.cls:
            if c[0] == len(z):
                keys = [p.tobytes() for p in c[1]]
                if z.tobytes() not in keys:
                    c[1].append(z)
                    keys.append(z.tobytes())
                c[2].append((col, root, keys.index(z.tobytes())))
                c[3].append(y)
                return
        self.cls.append([len(z), [z], [(col, root, 0)], [y]])


def commit_cols(engine, cols, R):
    """(column, root) pairs of several columns; engines that can queue many commitments before synchronising do so."""
    if hasattr(engine, "commit_many"):
        return list(zip(cols, engine.commit_many(cols, R)))
    return [(c, engine.commit_gpu_rootonly(c, R)) for c in cols]


def claimc(engine, tr, ledger, col, root, z):
    """p3hwl::claimc (zkllm-src/p3_hawkeye.cuh:800-838): evaluate, absorb under "hwl-y", defer the opening."""
    import struct
    y = engine.eval_h_gpu(col, np.ascontiguousarray(z, dtype=np.uint64))
    tr.absorb("hwl-y", struct.pack("<Q", y))
    ledger.add(col, root, z, y)
    return y


def tail_prove(engine, tr, ledger, R, Q, tag):
    """p3ig::tail_prove (zkllm-src/p3_int_gadgets.cuh:190-197) without deferred lookups: one batched
    opening per size class, labelled tag + index."""
    return [engine.prove_class(tr, np.stack(c[1]), c[2], R, Q, "%s%d" % (tag, i)) for i, c in enumerate(ledger.cls)]


S_J, S_A, S_I, S_C = 0, 1, 2, 3      # p3imm bit sources: contraction index, free index, Y's i index, constant


def view_offsets(view, lj, la):
    """p3imm::op_off (zkllm-src/p3_int_gadgets.cuh:448-459) for all (a, j): element index inside the committed
    column of entry (j, a) of the operand view; result shape [2^la][2^lj]."""
    j = np.arange(1 << lj, dtype=np.int64)[None, :]
    a = np.arange(1 << la, dtype=np.int64)[:, None]
    idx = np.zeros((1 << la, 1 << lj), dtype=np.int64)
    for t, (src, bit) in enumerate(view):
        b = ((j >> bit) & 1) if src == S_J else ((a >> bit) & 1) if src == S_A else (bit if src == S_C else 0)
        idx |= b << t
    return idx


def view_point(view, r_first, r_second, first=S_J, second=S_A):
    """p3imm::op_pt / y_pt (zkllm-src/p3_int_gadgets.cuh:473-497): the claim point on the committed column."""
    return [r_first[bit] if src == first else r_second[bit] if src == second else (bit if src == S_C else 0)
            for src, bit in view]


def imm_prove(engine, tr, X, W, Y, lj, lk, li, R, Q, ledger=None, views=None):
    """p3imm::prove (zkllm-src/p3_int_gadgets.cuh:546-605), non-zk, direct layouts: proves
    Y(i,k) = sum_j X(i,j) W(j,k) for committed columns X = [j | i<<lj], W = [k | j<<lk], Y = [k | i<<lk].
    X, W, Y: (device column, 32-byte root).

    The reference materialises three broadcast columns of 2^(lj+lk+li) elements and runs a cubic
    sumcheck over them.  The summand eq(z;k,i) X(j,i) W(j,k) factors over the index groups, so the
    identical round messages are produced from three short product sumchecks: over j on the vectors
    X(j,zi) and W(j,zk), then over k, then over i, each after a partial evaluation of X / W (matrix-
    vector products).  Work is O(|X| + |W|) instead of O(2^(lj+lk+li)); the proof bytes are the same.
    Returns the serialised p3imm::Proof (u32 lj, lk, li | messages (lj+lk+li)*40 | yY yX yW |
    u32 batches, each u32 length + BatchProof) -- the tail is present when no shared ledger is given."""
    import struct
    own = ledger is None
    if own:
        ledger = Ledger()
    tr.absorb("imm-dims", struct.pack("<III", lj, lk, li))
    tr.absorb("imm-X", X[1])
    tr.absorb("imm-W", W[1])
    tr.absorb("imm-Y", Y[1])
    z = [tr.chal() for _ in range(lk + li)]
    zk_, zi_ = z[:lk], z[lk:]
    Xfull, Wfull = X, W
    if views is None:
        yY = claimc(engine, tr, ledger, Y[0], Y[1], z)
    else:
        # operand views into larger committed columns (per-head attention matmuls): gather the dense operands,
        # prove on them, and place every claim on the committed column at the view's point
        xv, wv, yv = views
        yY = claimc(engine, tr, ledger, Y[0], Y[1], view_point(yv, zk_, zi_, S_A, S_I))
        X = (engine.gather(X[0], view_offsets(xv, lj, li).reshape(-1)), None)          # [i][j]
        W = (engine.gather(W[0], view_offsets(wv, lj, lk).T.reshape(-1)), None)        # [j][k]
    J, K, I = 1 << lj, 1 << lk, 1 << li
    eq_i, eq_k = engine.build_eq_gpu(np.array(zi_, dtype=np.uint64)), engine.build_eq_gpu(np.array(zk_, dtype=np.uint64))
    msgs, r = [], []
    # rounds over j: sum_j X(j, zi) * W(j, zk)
    Xz = engine.matvec(X[0], I, J, eq_i, False)
    Wz = engine.matvec(W[0], J, K, eq_k, True)
    if lj:
        rj, m, _ = engine.sc_prove_gpu(tr, "imm-sc", [Xz, Wz], F_PROD2, 5)
        msgs.append(m)
        rj = [int(x) for x in rj]
    else:
        rj = []
    eq_rj = engine.build_eq_gpu(np.array(rj, dtype=np.uint64))
    X1 = engine.matvec(X[0], I, J, eq_rj, True)       # X(rj, i)
    W1 = engine.matvec(W[0], J, K, eq_rj, False)      # W(rj, k)
    # rounds over k: [sum_i eq(zi,i) X(rj,i)] * sum_k eq(zk,k) W(rj,k)
    SX = engine.eval_h_gpu(X1, np.array(zi_, dtype=np.uint64))
    if lk:
        rk, m, fin = engine.sc_prove_gpu(tr, "imm-sc", [engine.scale(eq_k, SX), W1], F_PROD2, 5)
        msgs.append(m)
        rk, Wrr = [int(x) for x in rk], int(fin[1])
    else:
        rk, Wrr = [], engine.element(W1, 0)
    eqk_r = 1
    for a, b in zip(rk, zk_):
        eqk_r = eqk_r * ((a * b + (1 - a) * (1 - b)) % GL_P) % GL_P
    # rounds over i: eq(zk,rk) W(rj,rk) * sum_i eq(zi,i) X(rj,i)
    if li:
        ri, m, _ = engine.sc_prove_gpu(tr, "imm-sc", [engine.scale(eq_i, eqk_r * Wrr % GL_P), X1], F_PROD2, 5)
        msgs.append(m)
        ri = [int(x) for x in ri]
    else:
        ri = []
    if views is None:
        yX = claimc(engine, tr, ledger, X[0], X[1], rj + ri)
        yW = claimc(engine, tr, ledger, W[0], W[1], rk + rj)
    else:
        yX = claimc(engine, tr, ledger, Xfull[0], Xfull[1], view_point(views[0], rj, ri))
        yW = claimc(engine, tr, ledger, Wfull[0], Wfull[1], view_point(views[1], rj, rk))
    out = struct.pack("<III", lj, lk, li) + b"".join(np.ascontiguousarray(m, dtype=np.uint64).tobytes() for m in msgs)
    out += struct.pack("<QQQ", yY, yX, yW)
    batches = tail_prove(engine, tr, ledger, R, Q, "imm-bo") if own else []
    out += struct.pack("<I", len(batches)) + b"".join(struct.pack("<I", len(b)) + b for b in batches)
    return out


LU_GCAP = 25   # zkllm-src/p3_logup.cuh:1891


def make_table(cols):
    """p3lu::make_table (zkllm-src/p3_logup.cuh:413-421): host columns + the binding hash of a public table."""
    import hashlib
    cols = [np.ascontiguousarray(c, dtype=np.uint64) for c in cols]
    h = hashlib.sha256(np.uint64(len(cols)).tobytes() + np.uint64(len(cols[0])).tobytes())
    for c in cols:
        h.update(c.tobytes())
    return {"cols": cols, "id": h.digest(), "dev": {}}


def table_columns(engine, tab):
    """The table's columns as buffers of ``engine`` (uploaded once per engine and cached in the table object)."""
    key = id(engine)
    if key not in tab["dev"]:
        tab["dev"][key] = [engine.upload(c) for c in tab["cols"]]
    return tab["dev"][key]


def range_table(b, off):
    """p3ig::range_table (zkllm-src/p3_int_gadgets.cuh:60-64): rows j + off as field elements, j < 2^b."""
    v = np.arange(1 << b, dtype=np.int64) + off
    return make_table([np.where(v < 0, v.astype(object) + GL_P, v.astype(object)).astype(np.uint64)])


def lu_flush(engine, tr, luq, ledger, R, strict=True):
    """p3lu::lu_flush (zkllm-src/p3_logup.cuh:1940-1956): group the deferred lookups by (table, log-rows)
    in first-appearance order (groups capped at 2^LU_GCAP stacked rows), bundle the groups by table,
    prove one merged instance per table.  luq entries: {"W": [(col, root or None), ...], "idx": indices,
    "tab": make_table(...)} plus an optional "bind" callback (see prove_super).  Opening claims go to ``ledger``.  Returns the list of GroupProof bytes."""
    groups = []                                    # lu_groups
    for i, o in enumerate(luq):
        n = int(o["idx"].numel()).bit_length() - 1
        for g in groups:
            if g[0] == o["tab"]["id"] and g[1] == n:
                g[2].append(i)
                break
        else:
            groups.append([o["tab"]["id"], n, [i]])
    split = []
    for tid, n, mem in groups:
        cap = 1 if n >= LU_GCAP else 1 << (LU_GCAP - n)
        for off in range(0, len(mem), cap):
            split.append((tid, n, mem[off:off + cap]))
    supers = []                                    # lu_supers
    for tid, n, mem in split:
        for sp in supers:
            if sp[0] == tid:
                sp[1].append((n, mem))
                break
        else:
            supers.append([tid, [(n, mem)]])
    out = []
    for tid, subs in supers:
        tab = luq[subs[0][1][0]]["tab"]
        sg = [(n, [([w[0] for w in luq[j]["W"]], [w[1] for w in luq[j]["W"]], luq[j]["idx"], luq[j].get("bind")) for j in mem]) for n, mem in subs]
        pf, claims, _cnt = prove_super(engine, tr, table_columns(engine, tab), tid, sg, R, strict)
        for col, root, pt, y in claims:
            ledger.add(col, root, pt, y)
        out.append(pf)
    del luq[:]
    return out


def irs_prove(engine, tr, tables, X, Y, wit, le, sf, rng, R, Q, ledger=None, luq=None, tag="irs"):
    """p3irs::prove (zkllm-src/p3_int_gadgets.cuh:291-340), non-zk: Y = round-half-up(X / 2^sf) with the
    remainder limbs and Y range-checked by lookups.  X, Y: (column, root) committed operands of 2^le rows;
    wit = (limb columns, limb indices, y indices) from engine.irs_witness; tables: {"R16","R14","RTOP",
    "RS16","RS20"} as make_table objects.  With ledger/luq given the gadget only records its claims and
    lookups; otherwise it runs the tail itself (lookup flush + batched openings, tags tag-bo<i>).
    Proof: u32 le, sf, nl, rng | limb roots nl*32 | messages le*40 | yX yY yL[nl] |
    u32 groups, each u32 len + GroupProof | u32 batches, each u32 len + BatchProof."""
    import struct
    own = ledger is None
    if own:
        ledger, luq = Ledger(), []
    L, iL, iY = wit
    nl = 1 if sf <= 16 else 2
    tr.absorb("irs-dims", struct.pack("<IIII", le, sf, nl, rng))
    tr.absorb("irs-X", X[1])
    tr.absorb("irs-Y", Y[1])
    rL = [engine.commit_gpu_rootonly(L[l], R) for l in range(nl)]
    for l in range(nl):
        tr.absorb("irs-L", rL[l])
    for l in range(nl):
        tab = (tables["R14"] if sf == 14 else tables["R16"]) if l == 0 else (tables["R16"] if sf == 32 else tables["RTOP"])
        luq.append({"W": [(L[l], rL[l])], "idx": iL[l], "tab": tab})
    if rng:
        luq.append({"W": [(Y[0], Y[1])], "idx": iY, "tab": tables["RS20"] if rng == 1 else tables["RS16"]})
    zE = np.array([tr.chal() for _ in range(le)], dtype=np.uint64)
    E = engine.build_eq_gpu(zE)
    rE, m, _ = engine.sc_prove_gpu(tr, "irs-sc", [E, X[0], Y[0]] + list(L[:nl]), F_IRS1 if nl == 1 else F_IRS2, 5,
                                   [1 << (sf - 1), 1 << sf])
    rE = [int(x) for x in rE]
    yX = claimc(engine, tr, ledger, X[0], X[1], rE)
    yY = claimc(engine, tr, ledger, Y[0], Y[1], rE)
    yL = [claimc(engine, tr, ledger, L[l], rL[l], rE) for l in range(nl)]
    out = struct.pack("<IIII", le, sf, nl, rng) + b"".join(rL) + np.ascontiguousarray(m, dtype=np.uint64).tobytes()
    out += struct.pack("<QQ", yX, yY) + b"".join(struct.pack("<Q", v) for v in yL)
    lug, batches = [], []
    if own:
        lug = lu_flush(engine, tr, luq, ledger, R)
        batches = tail_prove(engine, tr, ledger, R, Q, tag + "-bo")
    out += struct.pack("<I", len(lug)) + b"".join(struct.pack("<I", len(b)) + b for b in lug)
    out += struct.pack("<I", len(batches)) + b"".join(struct.pack("<I", len(b)) + b for b in batches)
    return out


def col_sum(engine, col):
    """Sum of a power-of-two column through its multilinear extension: sum = 2^v * c~(1/2, ..., 1/2)."""
    v = int(col.numel()).bit_length() - 1
    half = (GL_P + 1) // 2
    return engine.eval_h_gpu(col, np.full(v, half, dtype=np.uint64)) * pow(2, v, GL_P) % GL_P


def lu_prove(engine, tr, W, idx, tab, R, Q, label, strict=True):
    """p3lu::prove / prove_v (zkllm-src/p3_logup.cuh:754-765, :932-1163), non-zk, standalone openings: the
    classic logUp with committed helper columns hA = 1/(A+beta), hT = cnt/(Tc+beta), two cubic sumchecks
    ("lu-scA", "lu-scT") and one Basefold opening per committed column.
    W: [(column, root) or (column, None) for a virtual column]; idx: row indices; tab: make_table(...).
    Returns (proof bytes, rA).  Serialised LookupProof: u32 n, m, c | root_cnt root_hA root_hT | S |
    msgsA n*32 | msgsT m*32 | u32 len, open_hA | u32 count, (u32 len, open_W)* | u32 count, y_virt* |
    u32 len, open_hT | u32 len, open_cnt."""
    import struct
    N, M = int(idx.numel()), len(tab["cols"][0])
    n, m, c = N.bit_length() - 1, M.bit_length() - 1, len(W)
    if (1 << n) != N or (1 << m) != M:
        raise ValueError("p3lu: pow2")
    if len(tab["cols"]) != c:
        raise ValueError("p3lu: col count")
    tcols = table_columns(engine, tab)
    tr.absorb("lu-tab", tab["id"])
    for col, root in W:
        if root is not None:
            tr.absorb("lu-W", root)
        else:
            tr.absorb("lu-Wv", b"virt")
    cnt = engine.lu_counts([idx], M, 0)
    root_cnt = engine.commit_gpu_rootonly(cnt, R)
    tr.absorb("lu-cnt", root_cnt)
    gamma, beta = tr.chal(), tr.chal()
    A = engine.combine([w[0] for w in W], gamma)
    Tc = engine.combine(tcols, gamma)
    hA = engine.inv_all_add(A, beta)
    hT = engine.mul(cnt, engine.inv_all_add(Tc, beta))
    SA, ST = col_sum(engine, hA), col_sum(engine, hT)
    if strict and SA != ST:
        raise ValueError("p3lu: witness not in table: " + label)
    root_hA, root_hT = engine.commit_gpu_rootonly(hA, R), engine.commit_gpu_rootonly(hT, R)
    tr.absorb("lu-hA", root_hA)
    tr.absorb("lu-hT", root_hT)
    tr.absorb("lu-S", struct.pack("<Q", SA))
    zA = np.array([tr.chal() for _ in range(n)], dtype=np.uint64)
    lamA = tr.chal()
    rA, msgsA, _ = engine.sc_prove_gpu(tr, "lu-scA", [hA, A, engine.build_eq_gpu(zA), engine.lu_ones(N)], F_LOGUP, 4,
                                       [lamA, beta])
    y_hA = engine.eval_h_gpu(hA, rA)
    open_hA = engine.prove_eval_dev(hA, rA, y_hA, R, Q, None, label + "-hA")
    open_W, y_virt = [], []
    for k, (col, root) in enumerate(W):
        y = engine.eval_h_gpu(col, rA)
        if root is not None:
            open_W.append(engine.prove_eval_dev(col, rA, y, R, Q, None, label + "-W%d" % k))
        else:
            y_virt.append(y)
            tr.absorb("lu-yv", struct.pack("<Q", y))
    zT = np.array([tr.chal() for _ in range(m)], dtype=np.uint64)
    lamT = tr.chal()
    rT, msgsT, _ = engine.sc_prove_gpu(tr, "lu-scT", [hT, Tc, engine.build_eq_gpu(zT), cnt], F_LOGUP, 4, [lamT, beta])
    y_hT, y_cnt = engine.eval_h_gpu(hT, rT), engine.eval_h_gpu(cnt, rT)
    open_hT = engine.prove_eval_dev(hT, rT, y_hT, R, Q, None, label + "-hT")
    open_cnt = engine.prove_eval_dev(cnt, rT, y_cnt, R, Q, None, label + "-cnt")
    for y in (y_hA, y_hT, y_cnt):
        tr.absorb("lu-ends", struct.pack("<Q", y))
    blob = lambda b: struct.pack("<I", len(b)) + b
    out = struct.pack("<III", n, m, c) + root_cnt + root_hA + root_hT + struct.pack("<Q", SA)
    out += np.ascontiguousarray(msgsA, dtype=np.uint64).tobytes() + np.ascontiguousarray(msgsT, dtype=np.uint64).tobytes()
    out += blob(open_hA) + struct.pack("<I", len(open_W)) + b"".join(blob(b) for b in open_W)
    out += struct.pack("<I", len(y_virt)) + b"".join(struct.pack("<Q", y) for y in y_virt)
    out += blob(open_hT) + blob(open_cnt)
    return out, rA
