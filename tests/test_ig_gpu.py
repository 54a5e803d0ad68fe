"""Integer-layer gadgets on CUDA: the proof bytes of the Prover-backed run equal the oracle-backed run of the same
host logic and the reference's own provers (witness replay on the host, commitments / lookups / openings on the
GPU) on the same inputs."""
import ctypes as C
import os

import numpy as np
import pytest

from ig_helpers import OracleGadgetEngine, arr, commit, ref_prove2

pytestmark = pytest.mark.gpu
R, Q = 1, 24


@pytest.fixture(scope="module")
def tables(zk):
    return zk.ig.build_tables(zk.load_library(), 64, 12)


class Dev:
    """Upload helpers for the CUDA engine mirroring ig_helpers.arr / commit."""

    def __init__(self, zk, prover):
        self.zk, self.p = zk, prover

    def col(self, a):
        import torch
        a = np.ascontiguousarray(a)
        if a.dtype == np.uint32:
            return torch.from_numpy(a.view(np.int32)).cuda()
        return self.zk.p3.to_device(a)

    def commit(self, a):
        c = self.col(a)
        return (c, self.p.commit_gpu_rootonly(c, R))


def both(zk, prover, orc, fn):
    """fn(engine, col, commit) -> proof bytes on a fresh transcript; run on CUDA and on the oracle engine."""
    d = Dev(zk, prover)
    tr1 = zk.Transcript("ig")
    pf1 = fn(prover, tr1, d.col, d.commit)
    eng = OracleGadgetEngine(orc)
    tr2 = zk.Transcript("ig")
    pf2 = fn(eng, tr2, lambda a: arr(eng, a), lambda a: commit(eng, arr(eng, a), R))
    assert pf1 == pf2 and tr1.state == tr2.state
    return pf1, tr1.state


def test_iadd(orc, ref_or_none, zk, prover, tables):
    ig, le = zk.ig, 11
    g = np.random.default_rng(1)
    a, b = ig.lift(g.integers(-(1 << 18), 1 << 18, 1 << le)), ig.lift(g.integers(-(1 << 18), 1 << 18, 1 << le))
    out, idxO = ig.iadd_witness(a, b)
    roots = {}

    def run(eng, tr, col, com):
        A, B, O = com(a), com(b), com(out)
        roots["r"] = [A[1], B[1], O[1]]
        return ig.iadd_prove(eng, tr, tables, A, B, O, col(idxO), le, R, Q)
    pf, st = both(zk, prover, orc, run)
    if ref_or_none is not None and ref_or_none.gpu_available():
        rpf, rst, _ = ref_prove2(ref_or_none, "ref_iadd_prove", zk.Transcript("ig").state, a, b, roots["r"], le, R, Q)
        assert rpf == pf and rst == st


def test_iswg(orc, ref_or_none, zk, prover, tables):
    ig, le = zk.ig, 10
    g = np.random.default_rng(2)
    gv, uv = ig.lift(g.integers(-(1 << 19), 1 << 19, 1 << le)), ig.lift(g.integers(-(1 << 15), 1 << 15, 1 << le))
    sil, rem, mo, iG, iR, iM = ig.iswg_witness(gv, uv, tables)
    roots = {}

    def run(eng, tr, col, com):
        G, U, MO = com(gv), com(uv), com(mo)
        roots["r"] = [G[1], U[1], MO[1]]
        return ig.iswg_prove(eng, tr, tables, G, U, MO, (col(sil), col(rem), col(iG), col(iR), col(iM)), le, R, Q)
    pf, st = both(zk, prover, orc, run)
    if ref_or_none is not None and ref_or_none.gpu_available():
        rpf, rst, _ = ref_prove2(ref_or_none, "ref_iswg_prove", zk.Transcript("ig").state, gv, uv, roots["r"], le, R, Q)
        assert rpf == pf and rst == st


def test_irope(orc, ref_or_none, zk, prover, tables):
    ig = zk.ig
    lseq, ldh, lnh = 4, 3, 1
    ld, lT = ldh + lnh, lseq
    le = lT + ld
    g = np.random.default_rng(3)
    ct = g.integers(-(1 << 14), (1 << 14) + 1, (1 << lseq, 1 << (ldh - 1))).astype(np.int32)
    sn = g.integers(-(1 << 14), (1 << 14) + 1, (1 << lseq, 1 << (ldh - 1))).astype(np.int32)
    q = ig.lift(g.integers(-(1 << 17), 1 << 17, 1 << le))
    y, rem, iR, iY, Cc, S2 = ig.irope_witness(q, ct, sn, lseq, ldh, lT, ld)
    roots = {}

    def run(eng, tr, col, com):
        Qc, Y = com(q), com(y)
        roots["r"] = [Qc[1], Y[1]]
        return ig.irope_prove(eng, tr, tables, (col(ig.lift(Cc)), col(ig.lift(S2)), ldh), Qc, Y, (col(rem), col(iR), col(iY)), lT, ld, R, Q)
    pf, st = both(zk, prover, orc, run)
    if ref_or_none is not None and ref_or_none.gpu_available():
        s = (C.c_uint8 * 32)(*zk.Transcript("ig").state)
        out = (C.c_uint8 * (32 << 20))()
        f = ref_or_none.lib.ref_irope_prove
        f.restype = C.c_size_t
        n = f(s, q.ctypes.data_as(C.c_void_p), ct.ctypes.data_as(C.c_void_p), sn.ctypes.data_as(C.c_void_p), C.c_uint32(lseq),
              C.c_uint32(ldh), roots["r"][0], roots["r"][1], C.c_uint32(lT), C.c_uint32(ld), C.c_uint32(R), C.c_uint32(Q), out,
              C.c_size_t(32 << 20), None)
        assert bytes(out)[:n] == pf and bytes(s) == st


def test_irms(orc, ref_or_none, zk, prover):
    ig = zk.ig
    lT, ld = 4, 5
    T = ig.build_tables(zk.load_library(), 1 << ld, 12)
    g = np.random.default_rng(4)
    x = ig.lift(g.integers(-(1 << 17), 1 << 17, 1 << (lT + ld)))
    gains = ig.lift(g.integers(1 << 15, 1 << 17, 1 << ld))
    w = ig.irms_witness(x, gains, T, lT, ld)
    roots = {}

    def run(eng, tr, col, com):
        X, G, Y = com(x), com(gains), com(w["y"])
        roots["r"] = [X[1], G[1], Y[1]]
        wit = {k: (col(v) if isinstance(v, np.ndarray) else [col(c) for c in v]) for k, v in w.items()}
        return ig.irms_prove(eng, tr, T, X, G, Y, wit, lT, ld, R, Q)
    pf, st = both(zk, prover, orc, run)
    if ref_or_none is not None and ref_or_none.gpu_available():
        s = (C.c_uint8 * 32)(*zk.Transcript("ig").state)
        out = (C.c_uint8 * (32 << 20))()
        f = ref_or_none.lib.ref_irms_prove
        f.restype = C.c_size_t
        n = f(s, x.ctypes.data_as(C.c_void_p), gains.ctypes.data_as(C.c_void_p), roots["r"][0], roots["r"][1], roots["r"][2],
              C.c_uint32(lT), C.c_uint32(ld), C.c_uint32(R), C.c_uint32(Q), out, C.c_size_t(32 << 20), None)
        assert bytes(out)[:n] == pf and bytes(s) == st


def test_ismx(orc, ref_or_none, zk, prover, tables):
    ig = zk.ig
    la, lseq = 1, 4
    g = np.random.default_rng(5)
    z = ig.lift(g.integers(-3000, 3000, 1 << (la + 2 * lseq)))
    w = ig.ismx_witness(z, tables, la, lseq)
    roots = {}

    def run(eng, tr, col, com):
        Z, P = com(z), com(w["p"])
        roots["r"] = [Z[1], P[1]]
        wit = {k: (col(v) if isinstance(v, np.ndarray) else [col(c) for c in v]) for k, v in w.items() if k != "p"}
        return ig.ismx_prove(eng, tr, tables, Z, P, wit, la, lseq, R, Q)
    pf, st = both(zk, prover, orc, run)
    if ref_or_none is not None and ref_or_none.gpu_available():
        s = (C.c_uint8 * 32)(*zk.Transcript("ig").state)
        out = (C.c_uint8 * (32 << 20))()
        f = ref_or_none.lib.ref_ismx_prove
        f.restype = C.c_size_t
        n = f(s, z.ctypes.data_as(C.c_void_p), roots["r"][0], roots["r"][1], C.c_uint32(la), C.c_uint32(lseq), C.c_uint32(R),
              C.c_uint32(Q), out, C.c_size_t(32 << 20), None)
        assert bytes(out)[:n] == pf and bytes(s) == st


@pytest.mark.parametrize("nb0,nb1,I,J,K", [(1, 1, 16, 32, 16), (1, 1, 130, 70, 67), (2, 4, 64, 16, 64), (1, 3, 256, 512, 64), (1, 1, 512, 2048, 128)])
def test_integer_matmul_kernel_equals_int64_products(zk, prover, nb0, nb1, I, J, K):
    """zkh_ig_matmul (the witness chain's exact integer products, p3imm::matmul_i64 in the reference) against int64 numpy products:
    plain row-major operands, transposed B (the score product's view), and head-sliced (batch, position, head, lane) views."""
    import torch
    from ig_helpers import StridedMatmulEngine
    rng = np.random.default_rng(I * 131 + J)
    P = 0xFFFFFFFF00000001
    lift = lambda a: np.where(a < 0, a.astype(np.int64).view(np.uint64) - np.uint64(0xFFFFFFFF), a.astype(np.int64).view(np.uint64))
    chk = StridedMatmulEngine()
    nb = nb0 * nb1
    layouts = [((nb1 * I * J, I * J, J, 1), (nb1 * J * K, J * K, K, 1), (nb1 * I * K, I * K, K, 1)),           # row-major, batched
               ((nb1 * I * J, I * J, J, 1), (nb1 * J * K, J * K, 1, J), (nb1 * I * K, I * K, K, 1)),           # B stored transposed
               ((I * nb1 * J, J, nb1 * J, 1), (J * nb1 * K, K, nb1 * K, 1), (I * nb1 * K, K, nb1 * K, 1))]     # (b0, row, b1, col)
    for sa, sb, sc in layouts:
        A = lift(rng.integers(-(1 << 19) + 1, 1 << 19, nb * I * J))
        B = lift(rng.integers(-(1 << 19) + 1, 1 << 19, nb * J * K))
        want = torch.zeros(nb * I * K, dtype=torch.int64)
        chk.ig_matmul(torch.from_numpy(A.view(np.int64)), sa, torch.from_numpy(B.view(np.int64)), sb, want, sc, nb0, nb1, I, J, K)
        got = torch.zeros(nb * I * K, dtype=torch.int64, device="cuda")
        prover.ig_matmul(zk.p3.to_device(A), sa, zk.p3.to_device(B), sb, got, sc, nb0, nb1, I, J, K)
        assert (got.cpu() == want).all()
        assert bool(((zk.p3.to_host(got) < P)).all())
    big = A.copy()
    big[3] = 1 << 30                                     # an operand outside the range is refused, not wrapped
    with pytest.raises(zk.ZkhError):
        prover.ig_matmul(zk.p3.to_device(big), sa, zk.p3.to_device(B), sb, got, sc, nb0, nb1, I, J, K)


def test_integer_matmul_tensor_core_and_integer_pipe_paths_agree(zk, tmp_path):
    """The same products through the tensor-core kernel (three 7-bit limbs, int32 accumulators in tensor memory) and through
    the integer-pipe kernel, forced with ZKH_IG_MATMUL in fresh processes, against int64 numpy products: full-size tiles,
    several k-tiles (the shared-memory stages are reused), transposed B, head-sliced views, operands at the limb boundaries."""
    import subprocess
    import sys
    import textwrap
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    prog = textwrap.dedent('''
        import sys, numpy as np, torch
        sys.path.insert(0, %r); sys.path.insert(0, %r); sys.path.insert(0, %r)
        import zkh_import
        from ig_helpers import StridedMatmulEngine
        zk = zkh_import.load()
        prover = zk.Prover(0, torch.cuda.current_stream().cuda_stream)
        lift = lambda a: np.where(a < 0, a.astype(np.int64).view(np.uint64) - np.uint64(0xFFFFFFFF), a.astype(np.int64).view(np.uint64))
        rng = np.random.default_rng(5)
        chk = StridedMatmulEngine()
        for nb0, nb1, I, J, K in [(1, 1, 128, 64, 64), (1, 1, 256, 512, 128), (1, 2, 128, 192, 64), (2, 2, 128, 128, 192), (1, 1, 512, 2048, 256)]:
            nb = nb0 * nb1
            for sa, sb, sc in [((nb1 * I * J, I * J, J, 1), (nb1 * J * K, J * K, K, 1), (nb1 * I * K, I * K, K, 1)),
                               ((nb1 * I * J, I * J, J, 1), (nb1 * J * K, J * K, 1, J), (nb1 * I * K, I * K, K, 1)),
                               ((I * nb1 * J, J, nb1 * J, 1), (J * nb1 * K, K, nb1 * K, 1), (I * nb1 * K, K, nb1 * K, 1))]:
                a = rng.integers(-(1 << 20) + 1, 1 << 20, nb * I * J)
                b = rng.integers(-(1 << 20) + 1, 1 << 20, nb * J * K)
                a[:8] = [(1 << 20) - 1, -(1 << 20) + 1, 127, 128, -128, -129, 16383, -16384]
                b[:4] = [-(1 << 20) + 1, (1 << 20) - 1, 16384, -1]
                A, B = lift(a), lift(b)
                want = torch.zeros(nb * I * K, dtype=torch.int64)
                chk.ig_matmul(torch.from_numpy(A.view(np.int64)), sa, torch.from_numpy(B.view(np.int64)), sb, want, sc, nb0, nb1, I, J, K)
                got = torch.zeros(nb * I * K, dtype=torch.int64, device="cuda")
                prover.ig_matmul(zk.p3.to_device(A), sa, zk.p3.to_device(B), sb, got, sc, nb0, nb1, I, J, K)
                assert (got.cpu() == want).all(), (nb0, nb1, I, J, K, sa)
        print("OK")
    ''') % (root, os.path.join(root, "oracle"), os.path.join(root, "tests"))
    for path in ("tc", "imad"):
        env = dict(os.environ, ZKH_IG_MATMUL=path)
        r = subprocess.run([sys.executable, "-c", prog], capture_output=True, text=True, env=env, timeout=600)
        assert r.returncode == 0 and "OK" in r.stdout, (path, r.stdout[-2000:], r.stderr[-2000:])
