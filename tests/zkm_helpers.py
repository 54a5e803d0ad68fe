"""CPU stand-in engine and reference windows for the hiding mode (test infrastructure)."""
import ctypes as C

import numpy as np

from ig_helpers import OracleGadgetEngine
from lu_helpers import _Arr

GL_P = 0xFFFFFFFF00000001


class OracleZkEngine(OracleGadgetEngine):
    """What zk_hillclimb_b200.zkm asks of an engine, on the CPU oracle."""

    def zk_fill_chain(self, s0, n, k0=0):
        return _Arr(self.orc.zprng_fill(s0, k0 + n)[k0:])

    def zk_augment(self, col, e, mask_seed):
        n = len(col.a)
        return _Arr(np.concatenate([col.a, self.orc.zprng_fill(mask_seed, (n << e) - n)]))

    def commit_salted(self, col, R, sseed, keep=False):
        root = bytes(self.orc.merkle_build_salted(self.orc.rs_encode(col.a, R), sseed)[-32:])
        return (root, None, None) if keep else root

    def concat(self, cols):
        return _Arr(np.concatenate([c.a for c in cols]))

    def slice(self, col, lo, n):
        return _Arr(col.a[lo:lo + n])

    def download(self, col):
        return col.a

    def zk_fill_at(self, seed, n, i0=0):
        """p3zkc::zprng_at stream, vectorised (checked against the C restatement in the tests)."""
        with np.errstate(over="ignore"):
            z = np.uint64(seed) + np.uint64(0x9E3779B97F4A7C15) * (np.arange(i0, i0 + n, dtype=np.uint64) + np.uint64(1))
            z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
            z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
            z ^= z >> np.uint64(31)
        return _Arr(z % np.uint64(GL_P))

    def interleave(self, a, b):
        return _Arr(np.stack([a.a, b.a], axis=1).reshape(-1))

    def zeros(self, n):
        return _Arr(np.zeros(n, dtype=np.uint64))

    def set_element(self, col, i, value):
        col.a[i] = np.uint64(int(value) % GL_P)

    def matmul(self, A, B, I, J, K):
        a, b = A.a.astype(object).reshape(I, J), B.a.astype(object).reshape(J, K)
        return _Arr(np.array([int(x) % GL_P for x in a.dot(b).reshape(-1)], dtype=np.uint64))

    def scatter_fn(self, col, n, fn, vals):
        col.a[fn(np.arange(n, dtype=np.int64))] = vals.a
        return col

    def gather_fn(self, col, n, fn):
        return _Arr(col.a[fn(np.arange(n, dtype=np.int64))])

    def prove_class_salted(self, tr, pts, ents, R, Q, label):
        pf, st = self.orc.bo_prove_class_salted(tr.state, pts, [e[0].a for e in ents], [e[1] for e in ents],
                                                [e[2] for e in ents], [e[3] for e in ents], R, Q, label)
        tr.state = st
        return pf

    def sc_prove_zc_partial(self, tr, tag, cols, terms, konst, rounds, table=None, pref=0):
        """The first rounds of a zero-check chain, optionally under the structured blind's table rows of these rounds."""
        return _partial(self, tr, tag, cols, terms, konst, rounds, table, pref)

    def sc_prove_zc_blind(self, tr, tag, cols, terms, konst, table):
        """The zero-check whose round messages gain A * (pref + g(t)) + B from the table rows [c0..c4, A, B]."""
        geval = lambda c, t: sum(int(c[k]) * pow(t, k, GL_P) for k in range(5)) % GL_P
        cur = [c.a for c in cols]
        msgs, chals, pref = [], [], 0
        while len(cur[0]) > 1:
            row = table[len(msgs)]
            s = [(m + int(row[5]) * ((pref + geval(row, t)) % GL_P) + int(row[6])) % GL_P
                 for t, m in enumerate(_round_message(cur, terms, konst))]
            tr.absorb(tag, np.array(s, dtype=np.uint64).tobytes())
            a = tr.chal()
            pref = (pref + geval(row, a)) % GL_P
            msgs.append(s)
            chals.append(a)
            cur = [np.array([(int(c[2 * i]) + a * (int(c[2 * i + 1]) - int(c[2 * i]))) % GL_P for i in range(len(c) // 2)],
                            dtype=np.uint64) for c in cur]
        return (np.array(chals, dtype=np.uint64), np.array(msgs, dtype=np.uint64), np.array([c[0] for c in cur], dtype=np.uint64),
                pref)


def _partial(engine, tr, tag, cols, terms, konst, rounds, table, pref):
    geval = lambda c, t: sum(int(c[k]) * pow(t, k, GL_P) for k in range(5)) % GL_P
    cur = [c.a for c in cols]
    msgs, chals = [], []
    for rd in range(rounds):
        s = _round_message(cur, terms, konst)
        if table is not None:
            row = table[rd]
            s = [(m + int(row[5]) * ((pref + geval(row, t)) % GL_P) + int(row[6])) % GL_P for t, m in enumerate(s)]
        tr.absorb(tag, np.array(s, dtype=np.uint64).tobytes())
        a = tr.chal()
        if table is not None:
            pref = (pref + geval(table[rd], a)) % GL_P
        msgs.append(s)
        chals.append(a)
        cur = [np.array([(int(c[2 * i]) + a * (int(c[2 * i + 1]) - int(c[2 * i]))) % GL_P for i in range(len(c) // 2)], dtype=np.uint64)
               for c in cur]
    return np.array(chals, dtype=np.uint64), np.array(msgs, dtype=np.uint64), np.stack(cur), pref


def _round_message(cols, terms, konst):
    h = len(cols[0]) // 2
    s = [0] * 5
    tt = [(int(t[0]) % GL_P, tuple(t[1]), bool(len(t) > 2 and t[2])) for t in terms]
    for i in range(h):
        lo = [int(c[2 * i]) for c in cols]
        df = [int(c[2 * i + 1]) - int(c[2 * i]) for c in cols]
        for t in range(5):
            v = [(l + t * d) % GL_P for l, d in zip(lo, df)]
            acc, free = int(konst) % GL_P, 0
            for coef, idx, outside in tt:
                p = coef
                for k in idx:
                    p = p * v[k] % GL_P
                if outside:
                    free += p
                else:
                    acc += p
            s[t] = (s[t] + v[0] * (acc % GL_P) + free) % GL_P
    return s


def ref_zk(ref, on, Q=24, seed=1, sblind_min=22):
    ref.lib.ref_zk_set(C.c_int(1 if on else 0), C.c_uint32(Q), C.c_uint64(seed), C.c_uint32(sblind_min))


def ref_imm_verify_zk(ref, st, roots, lj, lk, li, R, Q, proof, sblind_min=22):
    """p3imm::verify with the reference's zk switch on (the switch is put back)."""
    ref_zk(ref, True, Q, 1, sblind_min)
    try:
        s = (C.c_uint8 * 32)(*st)
        ok = ref.lib.ref_imm_verify(s, roots[0], roots[1], roots[2], C.c_uint32(lj), C.c_uint32(lk), C.c_uint32(li),
                                    C.c_uint32(R), C.c_uint32(Q), bytes(proof), C.c_size_t(len(proof)))
    finally:
        ref_zk(ref, False)
    return bool(ok), bytes(s)


def ref_imm_prove_zk(ref, st, X, W, lj, lk, li, R, Q, seed, sblind_min=22):
    """The reference's zk matmul prover (GPU): returns (proof bytes, state, roots X W Y, ms)."""
    s = (C.c_uint8 * 32)(*st)
    cap = 256 << 20
    out = (C.c_uint8 * cap)()
    roots = (C.c_uint8 * 96)()
    ms = C.c_double(0)
    f = ref.lib.ref_imm_prove_zk
    f.restype = C.c_size_t
    Xc, Wc = np.ascontiguousarray(X, dtype=np.uint64), np.ascontiguousarray(W, dtype=np.uint64)
    n = f(s, Xc.ctypes.data_as(C.c_void_p), Wc.ctypes.data_as(C.c_void_p), C.c_uint32(lj), C.c_uint32(lk), C.c_uint32(li),
          C.c_uint32(R), C.c_uint32(Q), C.c_uint64(seed), C.c_uint32(sblind_min), out, C.c_size_t(cap), roots, C.byref(ms))
    rb = bytes(roots)
    return bytes(out[:n]), bytes(s), [rb[0:32], rb[32:64], rb[64:96]], ms.value


def ref_irs_verify_zk(ref, st, rootX, rootY, le, sf, rng, R, Q, proof, sblind_min=22):
    """p3irs::verify with the reference's zk switch on."""
    ref_zk(ref, True, Q, 1, sblind_min)
    try:
        s = (C.c_uint8 * 32)(*st)
        ok = ref.lib.ref_irs_verify(s, rootX, rootY, C.c_uint32(le), C.c_uint32(sf), C.c_int(rng), C.c_uint32(R),
                                    C.c_uint32(Q), bytes(proof), C.c_size_t(len(proof)))
    finally:
        ref_zk(ref, False)
    return bool(ok), bytes(s)


def ref_irs_prove_zk(ref, st, acc, le, sf, rng, R, Q, seed, sblind_min=22):
    """The reference's zk rescale prover (GPU): returns (proof bytes, state, roots X Y, ms)."""
    s = (C.c_uint8 * 32)(*st)
    cap = 256 << 20
    out = (C.c_uint8 * cap)()
    roots = (C.c_uint8 * 64)()
    ms = C.c_double(0)
    f = ref.lib.ref_irs_prove_zk
    f.restype = C.c_size_t
    a = np.ascontiguousarray(acc, dtype=np.uint64)
    n = f(s, a.ctypes.data_as(C.c_void_p), C.c_uint32(le), C.c_uint32(sf), C.c_int(rng), C.c_uint32(R), C.c_uint32(Q),
          C.c_uint64(seed), C.c_uint32(sblind_min), out, C.c_size_t(cap), roots, C.byref(ms))
    rb = bytes(roots)
    return bytes(out[:n]), bytes(s), [rb[0:32], rb[32:64]], ms.value
