"""The drop-in claim at the engine boundary: the reference's own gadget provers, compiled UNCHANGED with
include/p3_scgpu_zkh.cuh force-included (its GPU sumcheck engine p3sg::sc_prove_gpu redirected to this library), give the
bytes of the stock reference build.  Both builds come from the same translation unit under oracle/."""
import ctypes as C
import os

import numpy as np
import pytest

from imm_helpers import matmul_instance
from lu_helpers import table_id
from test_lookup_gpu import gpu_groups, make_lookup

pytestmark = pytest.mark.gpu
u64p, u32p = C.POINTER(C.c_uint64), C.POINTER(C.c_uint32)


@pytest.fixture(scope="module")
def ref_zkh(ref):
    path = os.path.join(os.path.dirname(ref.path), "libp3ref_zkh.so")
    if not os.path.exists(path):
        pytest.skip("oracle/_ref/libp3ref_zkh.so not built (make -C oracle ref_zkh)")
    if not ref.gpu_available():
        pytest.skip("reference shim sees no GPU")
    lib = C.CDLL(path)
    lib.ref_zkh_sumcheck_calls.restype = C.c_longlong
    assert lib.ref_zkh_sumcheck_calls() >= 0
    return lib


def imm(lib, st0, X, W, Y, roots, lj, lk, li, R, Q):
    st = (C.c_uint8 * 32)(*st0)
    out = (C.c_uint8 * (8 << 20))()
    ms = C.c_double(0)
    f = lib.ref_imm_prove
    f.restype = C.c_size_t
    n = f(st, X.ctypes.data_as(u64p), W.ctypes.data_as(u64p), Y.ctypes.data_as(u64p), roots[0], roots[1], roots[2],
          C.c_uint32(lj), C.c_uint32(lk), C.c_uint32(li), C.c_uint32(R), C.c_uint32(Q), out, C.c_size_t(8 << 20), C.byref(ms))
    return bytes(out)[:n], bytes(st)


def test_reference_matmul_prover_over_this_library(orc, ref, ref_zkh, zk, prover):
    lj, lk, li, R, Q = 6, 6, 5, 1, 24             # 2^17-point chain: the reference sends it to its GPU engine
    X, W, Y = matmul_instance(orc, lj, lk, li, 321)
    roots = [prover.commit_gpu_rootonly(zk.p3.to_device(c), R) for c in (X, W, Y)]
    st0 = zk.Transcript("imm-ref").state
    want = imm(ref.lib, st0, X, W, Y, roots, lj, lk, li, R, Q)
    before = ref_zkh.ref_zkh_sumcheck_calls()
    got = imm(ref_zkh, st0, X, W, Y, roots, lj, lk, li, R, Q)
    assert ref_zkh.ref_zkh_sumcheck_calls() > before, "the matmul chain did not go through the library"
    assert len(want[0]) > 0 and got == want


def test_reference_lookup_prover_over_this_library(orc, ref, ref_zkh, zk, prover):
    R, Q = 1, 24
    m, shapes = 8, [(12, 2), (10, 3)]
    tcols, subs = make_lookup(orc, m, shapes, 99)
    groups, roots_flat, committed = gpu_groups(zk, prover, subs, R)
    tarr = [np.ascontiguousarray(t) for t in tcols]
    tp = (u64p * len(tarr))(*[a.ctypes.data_as(u64p) for a in tarr])
    wcols = [np.ascontiguousarray(c) for n, members in subs for cols, idx in members for c in cols]
    wp = (u64p * len(wcols))(*[a.ctypes.data_as(u64p) for a in wcols])
    idxs = [np.ascontiguousarray(idx) for n, members in subs for cols, idx in members]
    ip = (u32p * len(idxs))(*[a.ctypes.data_as(u32p) for a in idxs])
    sub_n = np.array([n for n, _ in subs], dtype=np.uint32)
    sub_k = np.array([len(mm) for _, mm in subs], dtype=np.uint32)

    def run(lib):
        st = (C.c_uint8 * 32)(*zk.Transcript("lu-ref").state)
        out = (C.c_uint8 * (1 << 20))()
        ms = C.c_double(0)
        f = lib.ref_lu_prove_super
        f.restype = C.c_size_t
        n = f(st, tp, C.c_uint32(m), C.c_uint32(len(tarr)), C.c_uint32(len(subs)), sub_n.ctypes.data_as(C.c_void_p),
              sub_k.ctypes.data_as(C.c_void_p), wp, roots_flat, ip, C.c_uint32(R), C.c_uint32(Q), out, C.c_size_t(1 << 20),
              C.byref(ms))
        return bytes(out)[:n], bytes(st)
    want = run(ref.lib)
    got = run(ref_zkh)
    assert len(want[0]) > 0 and got == want
