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
F_PROD2, F_PROD3, F_GKR, F_LOGUP = 0, 1, 2, 3
FUNCTOR_NC = {F_PROD2: 2, F_PROD3: 3, F_GKR: 5, F_LOGUP: 4}


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
        self._L = load_library()
        h = C.c_void_p()
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
        self._ck(self._L.zkh_ctx_set_stream(self._h, C.c_void_p(stream or 0)))

    def sync(self):
        self._ck(self._L.zkh_ctx_sync(self._h))

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

    def bind(self, in_dev, a, out=None, n=None):
        import torch
        n = n if n is not None else in_dev.numel()
        if out is None:
            out = torch.empty(n // 2, dtype=torch.int64, device=in_dev.device)
        self._ck(self._L.zkh_gl_bind(self._h, _ptr(in_dev), _ptr(out), n, a))
        return out

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
