"""Byte comparison with the reference's own CUDA provers at the benchmark's full shapes: the int8 matmul proof
128 x 768 . 768 x 768 (padded to 128 x 1024 . 1024 x 1024, seed 0) with the rescale of its output by 2^16, and the
lookup proof of 2^24 queries into a 2^16-row table with two columns.  The small shapes of the other test files pin
every branch; these pin the sizes the published numbers are quoted on."""
import ctypes as C

import numpy as np
import pytest

from lu_helpers import table_id

pytestmark = pytest.mark.gpu

P = 0xFFFFFFFF00000001
u64p, u32p = C.POINTER(C.c_uint64), C.POINTER(C.c_uint32)


def lift(a):
    a = a.reshape(-1).astype(np.int64)
    return np.where(a < 0, a.astype(np.uint64) + np.uint64(P), a.astype(np.uint64))


@pytest.fixture(scope="module")
def refgpu(ref):
    if not ref.gpu_available():
        pytest.skip("reference shim sees no GPU")
    return ref


@pytest.fixture(scope="module")
def matmul_c1(zk, prover):
    rng = np.random.default_rng(0)
    Xi = np.zeros((128, 1024), dtype=np.int64)
    Wi = np.zeros((1024, 1024), dtype=np.int64)
    Xi[:, :768] = rng.integers(-127, 128, (128, 768))
    Wi[:768, :768] = rng.integers(-127, 128, (768, 768))
    host = [lift(Xi), lift(Wi), lift(Xi @ Wi)]
    dev = [zk.p3.to_device(c) for c in host]
    roots = [prover.commit_gpu_rootonly(x, 1) for x in dev]
    return host, dev, roots


def test_int8_matmul_proof_equals_reference_prover(refgpu, zk, prover, matmul_c1):
    (X, W, Y), d, roots = matmul_c1
    lj, lk, li, R, Q = 10, 10, 7, 1, 24
    tr = zk.Transcript("imm")
    pf = zk.p3.imm_prove(prover, tr, (d[0], roots[0]), (d[1], roots[1]), (d[2], roots[2]), lj, lk, li, R, Q)
    st = (C.c_uint8 * 32)(*zk.Transcript("imm").state)
    out = (C.c_uint8 * (16 << 20))()
    ms = C.c_double(0)
    f = refgpu.lib.ref_imm_prove
    f.restype = C.c_size_t
    n = f(st, X.ctypes.data_as(u64p), W.ctypes.data_as(u64p), Y.ctypes.data_as(u64p), roots[0], roots[1], roots[2],
          C.c_uint32(lj), C.c_uint32(lk), C.c_uint32(li), C.c_uint32(R), C.c_uint32(Q), out, C.c_size_t(16 << 20),
          C.byref(ms))
    assert n > 0 and bytes(out)[:n] == pf and bytes(st) == tr.state


def test_rescale_proof_of_the_matmul_output_equals_reference_prover(refgpu, zk, prover, matmul_c1):
    (_, _, Y), d, roots = matmul_c1
    le, sf, rg, R, Q = 17, 16, 2, 1, 24
    tabs = {"R16": zk.p3.range_table(16, 0), "R14": zk.p3.range_table(14, 0), "RTOP": zk.p3.range_table(1, 0),
            "RS16": zk.p3.range_table(16, -(1 << 15)), "RS20": zk.p3.range_table(20, -(1 << 19))}
    tr = zk.Transcript("irs")
    y, L, iL, iY = prover.irs_witness(d[2], sf, rg)
    ry = prover.commit_gpu_rootonly(y, R)
    pf = zk.p3.irs_prove(prover, tr, tabs, (d[2], roots[2]), (y, ry), (L, iL, iY), le, sf, rg, R, Q)
    st = (C.c_uint8 * 32)(*zk.Transcript("irs").state)
    out = (C.c_uint8 * (16 << 20))()
    ms = C.c_double(0)
    f = refgpu.lib.ref_irs_prove
    f.restype = C.c_size_t
    n = f(st, Y.ctypes.data_as(u64p), roots[2], ry, C.c_uint32(le), C.c_uint32(sf), C.c_int(rg), C.c_uint32(R),
          C.c_uint32(Q), out, C.c_size_t(16 << 20), C.byref(ms))
    assert n > 0 and bytes(out)[:n] == pf and bytes(st) == tr.state


def test_lookup_proof_of_2_24_queries_equals_reference_prover(refgpu, zk, prover):
    import torch
    m, n, R, Q = 16, 24, 1, 24
    xs = np.arange(-32768, 32768, dtype=np.int64)
    silu = np.rint(65536.0 * (xs / 65536.0) / (1.0 + np.exp(-xs / 65536.0))).astype(np.int64)
    tcols = [lift(xs), lift(silu)]
    idx = (np.clip(np.rint(np.random.default_rng(0).normal(0, 1 << 10, 1 << n)), -32768, 32767).astype(np.int64)
           + 32768).astype(np.uint32)
    wcols = [np.ascontiguousarray(tc[idx]) for tc in tcols]
    dT = [zk.p3.to_device(t) for t in tcols]
    dW = [zk.p3.to_device(w) for w in wcols]
    didx = torch.from_numpy(idx.view(np.int32)).cuda()
    wroots = [prover.commit_gpu_rootonly(x, R) for x in dW]
    tr = zk.Transcript("lu")
    pf, claims, _ = zk.p3.prove_super(prover, tr, dT, table_id(tcols), [(n, [(dW, wroots, didx)])], R)
    tp = (u64p * 2)(*[a.ctypes.data_as(u64p) for a in tcols])
    wp = (u64p * 2)(*[a.ctypes.data_as(u64p) for a in wcols])
    ip = (u32p * 1)(idx.ctypes.data_as(u32p))
    sub_n, sub_k = np.array([n], dtype=np.uint32), np.array([1], dtype=np.uint32)
    st = (C.c_uint8 * 32)(*zk.Transcript("lu").state)
    out = (C.c_uint8 * (1 << 20))()
    ms = C.c_double(0)
    f = refgpu.lib.ref_lu_prove_super
    f.restype = C.c_size_t
    nb = f(st, tp, C.c_uint32(m), C.c_uint32(2), C.c_uint32(1), sub_n.ctypes.data_as(C.c_void_p),
           sub_k.ctypes.data_as(C.c_void_p), wp, b"".join(wroots), ip, C.c_uint32(R), C.c_uint32(Q), out,
           C.c_size_t(1 << 20), C.byref(ms))
    assert nb > 0 and bytes(out)[:nb] == pf and bytes(st) == tr.state
