"""CPU restatement of the reference's BLS12-381 Fr sumcheck path with Python integers.

TEST INFRASTRUCTURE ONLY: imported by tests/ and by __graft_entry__.smoke(); never by the package.

The reference's first proof stack keeps every tensor as plain integers below
    p = 0x73eda753299d7d483339d80809a1d80553bda402fffe5bfeffffffff00000001
(limb constant at zkllm-src/bls12-381.cu:4) and reaches the transcript only with plain values, so exact
integer arithmetic mod p restates it.  Functions follow:
    fs transcript / challenge      zkllm-src/fs_transcript.hpp:115-166, vrf_common.cuh:219-244
    eq tensor                      zkllm-src/zkob_lookup.cuh:202-212, :247-268
    FrTensor folds                 zkllm-src/fr-tensor.cu:542-652
    inner-product rounds           zkllm-src/zkfc.cu:94-127, zkob_fc.cu:290-332
    Hadamard / bracket rounds      zkllm-src/zkob_lookup.cuh:214-318, :321-425
    lagrange3 / lagrange4          zkllm-src/vrf_common.cuh:130-140

Pin status: the reference's own implementation of this stack needs a GPU even for scalar arithmetic
(h_scalar launches a one-thread kernel, vrf_common.cuh:100-104), so it cannot run where there is no
GPU.  On a GPU machine this restatement is pinned against the UNMODIFIED reference compiled into
oracle/_ref/libfrref.so (ReferenceFr below; tests/test_fr_reference_gpu.py compares fold, eq tensor,
partial_me, operator()(u), the inner-product rounds, fs_hadamard and fs_quartic value for value,
transcript state included).  Without a GPU only the transcript half is pinned (shared fs::Transcript
golden vectors); the field half is exact integer arithmetic on the published modulus.
"""
import hashlib
import struct

P = 0x73eda753299d7d483339d80809a1d80553bda402fffe5bfeffffffff00000001
TOP = 0x73eda753     # top limb of p (vrf_common.cuh:241)


def to_bytes(x):
    return int(x).to_bytes(32, "little")


def from_bytes(b):
    return int.from_bytes(b, "little")


class Transcript:
    """fs::Transcript (zkllm-src/fs_transcript.hpp:115-166)."""

    def __init__(self, seed):
        self.state = hashlib.sha256(seed.encode() if isinstance(seed, str) else seed).digest()

    def absorb(self, label, data):
        lb = label.encode()
        self.state = hashlib.sha256(self.state + struct.pack("<I", len(lb)) + lb + struct.pack("<Q", len(data)) + data).digest()

    def challenge_bytes(self):
        out = hashlib.sha256(self.state + b"chal").digest()
        self.state = hashlib.sha256(self.state + b"rtch").digest()
        return out

    def absorb_fr(self, label, x):
        self.absorb(label, to_bytes(x))

    def challenge_fr(self):
        """fs_challenge_fr: eight LE limbs of the challenge bytes, top limb mod TOP, redraw on zero."""
        while True:
            b = self.challenge_bytes()
            limbs = list(struct.unpack("<8I", b))
            limbs[7] %= TOP
            x = sum(l << (32 * i) for i, l in enumerate(limbs))
            if x:
                return x


def eq_build(u):
    E = [1]
    for c in u:                       # bit i is the new top bit
        E = [(1 - c) * e % P for e in E] + [c * e % P for e in E]
    return E


def mle_eval(t, u):
    """Fr_me: pairs (2i, 2i+1) with u[0] first."""
    t = list(t)
    for x in u:
        t = [(t[2 * i] + x * (t[2 * i + 1] - t[2 * i])) % P for i in range(len(t) // 2)]
    return t[0]


def partial_me(t, other, logd, window, u):
    """FrTensor::partial_me on [other][2^logd][window], u[0] pairs adjacent windows."""
    D = 1 << logd
    t = list(t)
    for x in u[:logd]:
        Dn = D // 2
        out = [0] * (other * Dn * window)
        for o in range(other):
            for d in range(Dn):
                for w in range(window):
                    a = t[(o * D + 2 * d) * window + w]
                    b = t[(o * D + 2 * d + 1) * window + w]
                    out[(o * Dn + d) * window + w] = (a + x * (b - a)) % P
        t, D = out, Dn
    return t


def fold(t, w):
    h = len(t) // 2
    return [(t[i] + w * (t[i + h] - t[i])) % P for i in range(h)]


def lagrange(evals, x):
    """Value at x of the polynomial with the given evaluations at 0..len-1 (lagrange3 / lagrange4)."""
    n, acc = len(evals), 0
    for i, y in enumerate(evals):
        num, den = 1, 1
        for j in range(n):
            if j != i:
                num = num * (x - j) % P
                den = den * (i - j) % P
        acc = (acc + y * num * pow(den, -1, P)) % P
    return acc


def product_sumcheck(tr, cols, labels):
    """Round loop shared by zkob_fc (2 columns), fs_hadamard (3) and fs_quartic (4): top variable first,
    evaluations at t = 0..nc absorbed one by one under `labels`, challenge by fs_challenge_fr.
    Returns (evals per round, challenges, final column values)."""
    cols = [list(c) for c in cols]
    nc, nt = len(cols), len(cols) + 1
    evals, chals = [], []
    while len(cols[0]) > 1:
        h = len(cols[0]) // 2
        ev = []
        for t in range(nt):
            s = 0
            for i in range(h):
                prod = 1
                for c in cols:
                    prod = prod * (c[i] + t * (c[i + h] - c[i])) % P
                s += prod
            ev.append(s % P)
        for lb, e in zip(labels, ev):
            tr.absorb_fr(lb, e)
        x = tr.challenge_fr()
        evals.append(ev)
        chals.append(x)
        cols = [fold(c, x) for c in cols]
    return evals, chals, [c[0] for c in cols]


class ReferenceFr:
    """ctypes window on oracle/_ref/libfrref.so: the unmodified reference's Fr stack (GPU machine only)."""

    PATH = __import__("os").path.join(__import__("os").path.dirname(__import__("os").path.abspath(__file__)), "_ref", "libfrref.so")

    @classmethod
    def available(cls):
        import os
        return os.path.exists(cls.PATH)

    def __init__(self):
        import ctypes
        self.C = ctypes
        self.lib = ctypes.CDLL(self.PATH)
        self.ms = ctypes.c_double(0)      # duration of the last timed reference call, milliseconds

    def gpu_available(self):
        return bool(self.lib.refA_gpu_available())

    @staticmethod
    def _pack(vals):
        if hasattr(vals, "tobytes"):            # numpy limb array [n, 8] uint32
            return vals.tobytes()
        return b"".join(to_bytes(v) for v in vals)

    @staticmethod
    def _unpack(buf, n):
        b = bytes(buf)
        return [from_bytes(b[32 * i:32 * i + 32]) for i in range(n)]

    def _out(self, n):
        return (self.C.c_uint8 * (32 * max(n, 1)))()

    def fold(self, t, w):
        out = self._out(len(t) // 2)
        assert self.lib.refA_fold(self._pack(t), len(t), to_bytes(w), out) == 0
        return self._unpack(out, len(t) // 2)

    def eq_build(self, u):
        out = self._out(1 << len(u))
        assert self.lib.refA_eq(self._pack(u), len(u), out) == 0
        return self._unpack(out, 1 << len(u))

    def partial_me(self, t, u, cur_dim, window):
        out = self._out(len(t))
        n = self.lib.refA_partial_me(self._pack(t), len(t), self._pack(u), len(u), cur_dim, window, out, self.C.byref(self.ms))
        assert n >= 0
        return self._unpack(out, n)

    def mle_eval(self, t, u):
        out = self._out(1)
        assert self.lib.refA_me(self._pack(t), len(t), self._pack(u), len(u), out) == 0
        return self._unpack(out, 1)[0]

    def _rounds(self, fn, st, cols, nt, *pre):
        n = len(cols[0])
        logn = n.bit_length() - 1
        s = (self.C.c_uint8 * 32)(*st)
        ev, ws, fin = self._out(logn * nt), self._out(logn), self._out(len(cols))
        assert fn(s, *pre, *[self._pack(c) for c in cols], n, ev, ws, fin, self.C.byref(self.ms)) == 0
        e = self._unpack(ev, logn * nt)
        return bytes(s), [e[i * nt:(i + 1) * nt] for i in range(logn)], self._unpack(ws, logn), self._unpack(fin, len(cols))

    def ip_rounds(self, st, a, b):
        return self._rounds(self.lib.refA_ip_rounds, st, [a, b], 3)

    def hadamard(self, st, E, S, U):
        """fs_hadamard: terminals are S and U only (E's is verifier-computed)."""
        n = len(E)
        logn = n.bit_length() - 1
        s = (self.C.c_uint8 * 32)(*st)
        ev, ws, fin = self._out(logn * 4), self._out(logn), self._out(2)
        assert self.lib.refA_hadamard(s, self._pack(E), self._pack(S), self._pack(U), n, ev, ws, fin, self.C.byref(self.ms)) == 0
        e = self._unpack(ev, logn * 4)
        return bytes(s), [e[i * 4:(i + 1) * 4] for i in range(logn)], self._unpack(ws, logn), self._unpack(fin, 2)

    def lookup(self, st, S, T, m, alpha, beta, u):
        """tlookup_inv_kernel + fs_phase1/fs_phase2: returns (state, A, evals, ws, terminals)."""
        D, N = len(S), len(m)
        logD = D.bit_length() - 1
        s = (self.C.c_uint8 * 32)(*st)
        Ao, ev, ws, term = self._out(D), self._out(logD * 4), self._out(logD), self._out(5)
        assert self.lib.refA_lookup(s, self._pack(S), self._pack(T), self._pack(m), D, N, to_bytes(alpha), to_bytes(beta),
                                    self._pack(u), Ao, ev, ws, term, self.C.byref(self.ms)) == 0
        e = self._unpack(ev, logD * 4)
        return (bytes(s), self._unpack(Ao, D), [e[i * 4:(i + 1) * 4] for i in range(logD)], self._unpack(ws, logD),
                tuple(self._unpack(term, 5)))

    def quartic(self, st, tag, E, A, B, Cc):
        n = len(E)
        logn = n.bit_length() - 1
        s = (self.C.c_uint8 * 32)(*st)
        ev, ws, fin = self._out(logn * 5), self._out(logn), self._out(3)
        assert self.lib.refA_quartic(s, tag.encode(), self._pack(E), self._pack(A), self._pack(B), self._pack(Cc), n,
                                     ev, ws, fin, self.C.byref(self.ms)) == 0
        e = self._unpack(ev, logn * 5)
        return bytes(s), [e[i * 5:(i + 1) * 5] for i in range(logn)], self._unpack(ws, logn), self._unpack(fin, 3)


# ---- tLookup: logUp over Fr (zkllm-src/tlookup.cu:184-296, zkob_lookup.cuh:143-198) ----
def inv_add(vals, beta):
    """tlookup_inv_kernel: 1/(x+beta), Fermat's inverse of 0 being 0."""
    return [pow((x + beta) % P, P - 2, P) for x in vals]


def _poly_eval(coef, x):
    acc = 0
    for c in reversed(coef):
        acc = (acc * x + c) % P
    return acc


def _poly_mul(a, b):
    out = [0] * (len(a) + len(b) - 1)
    for i, x in enumerate(a):
        for j, y in enumerate(b):
            out[i + j] = (out[i + j] + x * y) % P
    return out


def _poly_add(a, b):
    n = max(len(a), len(b))
    return [((a[i] if i < len(a) else 0) + (b[i] if i < len(b) else 0)) % P for i in range(n)]


def _eq_poly(u):
    return [(1 - u) % P, (2 * u - 1) % P]            # Polynomial::eq(u): (1-u) + (2u-1) t


def _eval_coeffs(X, Y, scale, beta, u_):
    """tLookup_phase*_poly_eval_kernel + MLE evaluation at u_: coefficients in t of
    sum_i eq(u_, i) * scale * X_i(t) * (Y_i(t) + beta), pairs (i, i+h)."""
    h = len(X) // 2
    t0 = [scale * X[i] * (Y[i] + beta) % P for i in range(h)]
    t1 = [scale * ((X[i + h] - X[i]) * (Y[i] + beta) + X[i] * (Y[i + h] - Y[i])) % P for i in range(h)]
    t2 = [scale * (X[i + h] - X[i]) * (Y[i + h] - Y[i]) % P for i in range(h)]
    return [mle_eval(t0, u_), mle_eval(t1, u_), mle_eval(t2, u_)]


def lookup_sumcheck(tr, A, S, B, T, m, alpha, beta, C, u):
    """fs_phase1 followed by fs_phase2 (non-strict): returns (evals per round [p(0..3)], challenges,
    terminals (A_f, S_f, B_f, T_f, m_f)).  D = len(A) = len(S), N = len(B) = len(T) = len(m)."""
    A, S, B, T, m = list(A), list(S), list(B), list(T), list(m)
    D, N = len(A), len(m)
    inv_ratio = N * pow(D, -1, P) % P
    alpha_run, alpha_sq = alpha, alpha * alpha % P
    inv2 = pow(2, -1, P)
    u = list(u)
    evals, ws = [], []
    while u:
        u_, ul = u[:-1], u[-1]
        h = len(A) // 2
        if len(A) != len(m):                          # phase 1
            p0 = _eval_coeffs(A, S, alpha_run, beta, u_)
            p1 = [sum(A[:h]) % P, (sum(A[h:]) - sum(A[:h])) % P]
            poly = _poly_add(_poly_add(_poly_mul(p0, _eq_poly(ul)), p1), [C * inv2 % P])
        else:                                         # phase 2
            p0 = _poly_add(_eval_coeffs(A, S, alpha_run, beta, u_), _eval_coeffs(B, T, inv_ratio * alpha_sq % P, beta, u_))
            p1 = [sum(A[:h]) % P, (sum(A[h:]) - sum(A[:h])) % P]
            p2 = [sum(m[i] * B[i] for i in range(h)) % P,
                  sum((m[i + h] - m[i]) * B[i] + m[i] * (B[i + h] - B[i]) for i in range(h)) % P,
                  sum((m[i + h] - m[i]) * (B[i + h] - B[i]) for i in range(h)) % P]
            poly = _poly_add(_poly_add(_poly_mul(p0, _eq_poly(ul)), p1), [(-inv_ratio * c) % P for c in p2])
        e = [_poly_eval(poly, t) for t in range(4)]
        for lb, x in zip(("p0", "p1", "p2", "p3"), e):
            tr.absorb_fr(lb, x)
        v = tr.challenge_fr()
        evals.append(e)
        ws.append(v)
        eqv = (ul * v + (1 - ul) * (1 - v)) % P
        if len(A) != len(m):
            C = C * inv2 % P
        else:
            B, T, m = fold(B, v), fold(T, v), fold(m, v)
            alpha_sq = alpha_sq * eqv % P
        A, S = fold(A, v), fold(S, v)
        alpha_run = alpha_run * eqv % P
        u = u_
    return evals, ws, (A[0], S[0], B[0], T[0], m[0])
