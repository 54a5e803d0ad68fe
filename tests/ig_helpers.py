"""CPU stand-in engine and reference windows for the integer-layer gadgets (test infrastructure)."""
import ctypes as C

import numpy as np

from irs_helpers import OracleStandaloneLuEngine
from lu_helpers import _Arr
from zc_helpers import zc_sumcheck

GL_P = 0xFFFFFFFF00000001


class OracleGadgetEngine(OracleStandaloneLuEngine):
    """Everything the gadget host logic asks of an engine, on the CPU oracle."""

    def bcast_rows(self, col, ld):
        return _Arr(np.repeat(col.a, 1 << ld))

    def bcast_cols(self, col, lT):
        return _Arr(np.tile(col.a, 1 << lT))

    def causal_mask(self, la, lseq):
        u = np.arange(1 << (la + 2 * lseq), dtype=np.int64)
        seq = 1 << lseq
        return _Arr(((u & (seq - 1)) <= ((u >> lseq) & (seq - 1))).astype(np.uint64))

    def gather(self, col, idx):
        return _Arr(col.a[np.asarray(idx, dtype=np.int64)])

    def flip_bit(self, col, b):
        return _Arr(col.a.reshape(-1, 2, 1 << b)[:, ::-1, :].reshape(-1).copy())

    def sc_prove_zc(self, tr, tag, cols, terms, konst=0):
        st, m, r, fin = zc_sumcheck(self.orc, tr.state, tag, [c.a for c in cols], terms, konst)
        tr.state = st
        return r, m, fin


def arr(engine, a):
    return _Arr(np.ascontiguousarray(a))


def commit(engine, col, R):
    return (col, engine.commit_gpu_rootonly(col, R))


def ref_table(ref, which, d=64, btop=12):
    rows, nc = {0: (1 << 17, 2), 1: (1 << 20, 2), 2: (1 << 16, 2), 3: (32, 3)}[which]
    cols = [np.zeros(rows, dtype=np.uint64) for _ in range(nc)]
    u64p = C.POINTER(C.c_uint64)
    ptrs = (u64p * nc)(*[c.ctypes.data_as(u64p) for c in cols])
    tid = (C.c_uint8 * 32)()
    assert ref.lib.ref_ig_table(C.c_uint32(d), C.c_uint32(btop), which, ptrs, tid) == nc
    return cols, bytes(tid)


def ref_verify3(ref, name, st, roots, le, R, Q, proof):
    """ref_iadd_verify / ref_iswg_verify: three operand roots, (le, R, Q)."""
    s = (C.c_uint8 * 32)(*st)
    ok = getattr(ref.lib, name)(s, roots[0], roots[1], roots[2], C.c_uint32(le), C.c_uint32(R), C.c_uint32(Q), bytes(proof),
                                C.c_size_t(len(proof)))
    return bool(ok), bytes(s)


def ref_prove2(ref, name, st, a, b, roots, le, R, Q):
    """ref_iadd_prove / ref_iswg_prove (GPU): two input columns, three operand roots."""
    s = (C.c_uint8 * 32)(*st)
    cap = 64 << 20
    out = (C.c_uint8 * cap)()
    ms = C.c_double(0)
    f = getattr(ref.lib, name)
    f.restype = C.c_size_t
    a, b = np.ascontiguousarray(a, dtype=np.uint64), np.ascontiguousarray(b, dtype=np.uint64)
    n = f(s, a.ctypes.data_as(C.c_void_p), b.ctypes.data_as(C.c_void_p), roots[0], roots[1], roots[2], C.c_uint32(le),
          C.c_uint32(R), C.c_uint32(Q), out, C.c_size_t(cap), C.byref(ms))
    return bytes(out)[:n], bytes(s), ms.value


def layer_inputs(ig, c, seed, wscale=0.9):
    return ig.random_layer_inputs(c, seed, wscale)


def ref_itf_verify(ref, st, c, x0, rX0, wroots, Wt, out, R, Q, proof):
    s = (C.c_uint8 * 32)(*st)
    dims = (C.c_uint32 * 6)(c.seq, c.d, c.nh, c.dh, c.dff, c.batch)
    vp = lambda a: np.ascontiguousarray(a).ctypes.data_as(C.c_void_p)
    x0c, outc, ct, sn = (np.ascontiguousarray(a) for a in (x0, out, Wt["ct"], Wt["st"]))
    ok = ref.lib.ref_itf_verify(s, dims, vp(x0c), rX0, b"".join(wroots), vp(ct), vp(sn), vp(outc), C.c_uint32(R), C.c_uint32(Q),
                                bytes(proof), C.c_size_t(len(proof)))
    if not ok and hasattr(ref.lib, "ref_last_why"):
        ref.lib.ref_last_why.restype = C.c_char_p
        ref.last_why = (ref.lib.ref_last_why() or b"").decode()
    return bool(ok), bytes(s)


def ref_itf_prove(ref, st, c, x0, Wt, R, Q):
    s = (C.c_uint8 * 32)(*st)
    dims = (C.c_uint32 * 6)(c.seq, c.d, c.nh, c.dh, c.dff, c.batch)
    u64p = C.POINTER(C.c_uint64)
    ws = [np.ascontiguousarray(w, dtype=np.uint64) for w in Wt["w"]]
    wp = (u64p * 7)(*[w.ctypes.data_as(u64p) for w in ws])
    vp = lambda a: a.ctypes.data_as(C.c_void_p)
    x0c, g1, g2, ct, sn = (np.ascontiguousarray(a) for a in (x0, Wt["g1"], Wt["g2"], Wt["ct"], Wt["st"]))
    cap = 256 << 20
    out = (C.c_uint8 * cap)()
    grid = np.zeros(len(x0c), dtype=np.uint64)
    ms = (C.c_double * 3)()
    f = ref.lib.ref_itf_prove
    f.restype = C.c_size_t
    n = f(s, dims, vp(x0c), wp, vp(g1), vp(g2), vp(ct), vp(sn), C.c_uint32(R), C.c_uint32(Q), out, C.c_size_t(cap), vp(grid), ms)
    return bytes(out[:n]), bytes(s), grid, list(ms)


class StridedMatmulEngine:
    """CPU stand-in for Prover.ig_matmul (the strided exact integer products of the device witness chain): the views are
    rebuilt with numpy strides over the signed values, multiplied in int64 and written back lifted."""

    def ig_matmul(self, A, a_str, B, b_str, Cc, c_str, nb0, nb1, I, J, K):
        def signed(t):
            a = t.numpy().view(np.uint64)
            return np.where(a >> np.uint64(63), a + np.uint64(0xFFFFFFFF), a).view(np.int64)

        def view(a, st, rows, cols):
            return np.lib.stride_tricks.as_strided(a, shape=(nb0, nb1, rows, cols), strides=[8 * int(x) for x in st])
        y = np.einsum("abij,abjk->abik", view(signed(A), a_str, I, J), view(signed(B), b_str, J, K))
        out = Cc.numpy()
        view(out, c_str, I, K)[...] = np.where(y < 0, y.view(np.uint64) - np.uint64(0xFFFFFFFF), y.view(np.uint64)).view(np.int64)
