"""Test-side stand-ins and helpers for the merged lookup (test infrastructure)."""
import ctypes as C
import hashlib

import numpy as np

GL_P = 0xFFFFFFFF00000001


class _Arr:
    """numpy-backed column with the two torch methods prove_super touches."""

    def __init__(self, a):
        self.a = np.ascontiguousarray(a)

    def numel(self):
        return len(self.a)


class OracleLookupEngine:
    """CPU engine for zk_hillclimb_b200.p3.prove_super built on the oracle."""

    def __init__(self, orc):
        self.orc = orc

    def lu_counts(self, idx_list, M, pad_rows):
        cnt = np.zeros(M, dtype=np.uint64)
        for idx in idx_list:
            cnt += self.orc.histogram(idx.a, M)
        cnt[0] += np.uint64(pad_rows)
        return _Arr(cnt)

    def commit_gpu_rootonly(self, col, R):
        return self.orc.merkle_root(self.orc.rs_encode(col.a, R))

    def element(self, col, i):
        return int(col.a[i])

    def lu_leaf_denominators(self, members, kp, n, gamma, shift, pad_value):
        N = 1 << n
        out = np.empty(kp << n, dtype=np.uint64)
        for j in range(kp):
            if j < len(members):
                comb = self.orc.combine([c.a for c in members[j]], gamma)
                out[j * N:(j + 1) * N] = ((comb.astype(object) + shift) % GL_P).astype(np.uint64)
            else:
                out[j * N:(j + 1) * N] = np.uint64(pad_value)
        return _Arr(out)

    def lu_ones(self, n):
        return _Arr(np.ones(n, dtype=np.uint64))

    def affine(self, cols, g, addend):
        comb = self.orc.combine([c.a for c in cols], g)
        return _Arr(((comb.astype(object) + addend) % GL_P).astype(np.uint64))

    def gkr_prove(self, tr, tag, P, Q, combine_last):
        st, pf, rfin, cpq = self.orc.gkr_prove(tr.state, tag, P.a, Q.a, combine_last)
        tr.state = st
        return pf, rfin, cpq

    def eval_h_gpu(self, col, z):
        return self.orc.mle_eval(col.a, z)


def table_id(cols):
    """p3lu::make_table's binding hash: SHA-256 over (ncols, M, columns) (zkllm-src/p3_logup.cuh:413-421)."""
    h = hashlib.sha256()
    h.update(np.uint64(len(cols)).tobytes() + np.uint64(len(cols[0])).tobytes())
    for c in cols:
        h.update(np.ascontiguousarray(c, dtype=np.uint64).tobytes())
    return h.digest()


def make_lookup(orc, m, shapes, seed, c=2):
    """A c-column table of 2^m rows and, per subgroup (n, k), k members whose rows are table rows."""
    rng = np.random.default_rng(seed)
    t0, s = orc.lcg(1 << m, seed)
    tcols = [t0] + [orc.lcg(1 << m, s + t)[0] for t in range(1, c)]
    subgroups = []
    for n, k in shapes:
        members = []
        for _ in range(k):
            idx = np.clip(np.rint(rng.normal((1 << m) / 2, max((1 << m) / 16, 1), 1 << n)), 0, (1 << m) - 1).astype(np.uint32)
            members.append(([tc[idx] for tc in tcols], idx))
        subgroups.append((n, members))
    return tcols, subgroups


def verify_with_reference(ref, st, tcols, subgroups_meta, roots_flat, committed_flat, R, Q, proof, max_claims=256):
    """p3lu::verify_super through the reference shim.  Returns (ok, new state, ledger claims)."""
    u64p = C.POINTER(C.c_uint64)
    c = len(tcols)
    m = len(tcols[0]).bit_length() - 1
    arrs = [np.ascontiguousarray(t, dtype=np.uint64) for t in tcols]
    tp = (u64p * c)(*[a.ctypes.data_as(u64p) for a in arrs])
    ns = len(subgroups_meta)
    sub_n = np.array([x[0] for x in subgroups_meta], dtype=np.uint32)
    sub_k = np.array([x[1] for x in subgroups_meta], dtype=np.uint32)
    s = (C.c_uint8 * 32)(*st)
    ncl = C.c_uint32(0)
    croots = (C.c_uint8 * (32 * max_claims))()
    cvlen = np.zeros(max_claims, dtype=np.uint32)
    cpts = np.zeros(max_claims * 64, dtype=np.uint64)
    cy = np.zeros(max_claims, dtype=np.uint64)
    ok = ref.lib.ref_lu_verify_super(s, tp, C.c_uint32(m), C.c_uint32(c), C.c_uint32(ns),
                                     sub_n.ctypes.data_as(C.c_void_p), sub_k.ctypes.data_as(C.c_void_p),
                                     bytes(roots_flat), bytes(committed_flat), C.c_uint32(R), C.c_uint32(Q),
                                     bytes(proof), C.c_size_t(len(proof)), C.byref(ncl), croots,
                                     cvlen.ctypes.data_as(C.c_void_p), cpts.ctypes.data_as(u64p),
                                     cy.ctypes.data_as(u64p), C.c_uint32(max_claims))
    claims = []
    for i in range(ncl.value):
        v = int(cvlen[i])
        claims.append((bytes(croots[32 * i:32 * i + 32]), cpts[64 * i:64 * i + v].copy(), int(cy[i])))
    return bool(ok), bytes(s), claims
