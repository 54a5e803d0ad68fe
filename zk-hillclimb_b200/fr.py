"""Host-side mirror of the reference's BLS12-381 Fr prover pieces (its first proof stack) over the C ABI.

Elements are the reference's Fr_t: eight little-endian 32-bit limbs holding a plain integer below P.
Device arrays are torch int32 tensors of shape [n, 8]; points, challenges and results are Python ints.
Names follow the reference: build_eq_tensor, k_fr_fold, FrTensor.partial_me / operator()(u),
fs_hadamard, fs_quartic, the zkob_fc inner-product rounds (zkllm-src/zkob_lookup.cuh, fr-tensor.cu,
zkob_fc.cu).  There is no CPU path: every function calls the CUDA library.
"""
import ctypes as C

import numpy as np

from ._lib import ZkhError  # noqa: F401

P = 0x73eda753299d7d483339d80809a1d80553bda402fffe5bfeffffffff00000001


def pack(vals):
    """ints -> numpy uint32 [n, 8] limb array."""
    out = np.empty((len(vals), 8), dtype=np.uint32)
    for i, x in enumerate(vals):
        out[i] = np.frombuffer(int(x).to_bytes(32, "little"), dtype=np.uint32)
    return out


def unpack(arr):
    a = np.ascontiguousarray(arr, dtype=np.uint32).reshape(-1, 8)
    return [int.from_bytes(row.tobytes(), "little") for row in a]


def to_device(vals, device="cuda:0"):
    import torch
    a = vals if isinstance(vals, np.ndarray) else pack(vals)
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.uint32).view(np.int32)).to(device)


def to_host(t):
    return unpack(t.detach().cpu().numpy().view(np.uint32))


def _pt(u):
    return np.ascontiguousarray(pack(u)) if len(u) else np.zeros((1, 8), dtype=np.uint32)


def _new(prover, n):
    import torch
    return torch.empty((n, 8), dtype=torch.int32, device="cuda:%d" % prover.device)


def build_eq_tensor(prover, u):
    """E[b] = prod_i (bit_i(b) ? u[i] : 1-u[i])  (zkllm-src/zkob_lookup.cuh:247-268)."""
    out = _new(prover, 1 << len(u))
    a = _pt(u)
    prover._ck(prover._L.zkh_fr_eq_build(prover._h, a.ctypes.data, len(u), out.data_ptr()))
    return out


def fr_fold(prover, t, w):
    """k_fr_fold: out[i] = t[i] + w*(t[i+h]-t[i])."""
    h = t.shape[0] // 2
    out = _new(prover, h)
    a = _pt([w])
    prover._ck(prover._L.zkh_fr_fold(prover._h, t.data_ptr(), h, a.ctypes.data, out.data_ptr()))
    return out


def partial_me(prover, t, u, cur_dim, window_size):
    """FrTensor::partial_me(u, cur_dim, window_size) for cur_dim == 2^len(u)."""
    if cur_dim != 1 << len(u):
        raise ValueError("partial_me: cur_dim must equal 2^len(u)")
    n = t.shape[0]
    if n % (cur_dim * window_size):
        raise ValueError("partial_me: size not divisible by cur_dim*window_size")
    other = n // (cur_dim * window_size)
    out = _new(prover, other * window_size)
    a = _pt(u)
    prover._ck(prover._L.zkh_fr_partial_me(prover._h, t.data_ptr(), other, len(u), window_size, a.ctypes.data,
                                           out.data_ptr()))
    return out


def mle_eval(prover, t, u):
    """FrTensor::operator()(u): multilinear extension of t at u, u[0] pairing adjacent elements."""
    if t.shape[0] != 1 << len(u):
        raise ValueError("mle_eval: size must equal 2^len(u)")
    a = _pt(u)
    out = (C.c_uint8 * 32)()
    prover._ck(prover._L.zkh_fr_mle_eval(prover._h, t.data_ptr(), a.ctypes.data, len(u), out))
    return int.from_bytes(bytes(out), "little")


def multi_dim_me(prover, t, us, shape):
    """FrTensor::multi_dim_me (zkllm-src/fr-tensor.cu:634-643): fold the last dimension first."""
    if len(us) != len(shape):
        raise ValueError("Incompatible dimensions")
    for u, d in zip(reversed(us[1:]), reversed(shape[1:])):
        t = partial_me(prover, t, u, d, 1)
    return mle_eval(prover, t, us[0]) if us else to_host(t[:1])[0]


def product_sumcheck(prover, tr, cols, labels):
    """The round loop of zkob_fc's inner product (2 columns; labels p0 p1 p2), fs_hadamard (3; hp0..hp3)
    and fs_quartic (4; tag+p0..p4): returns (evals[rounds][nt], challenges, finals) as ints and
    advances ``tr`` exactly as the reference's transcript advances."""
    nc = len(cols)
    n = cols[0].shape[0]
    logn = n.bit_length() - 1
    if n != 1 << logn or len(labels) != nc + 1:
        raise ValueError("product_sumcheck: power-of-two columns and nc+1 labels")
    ptrs = (C.c_void_p * nc)(*[c.data_ptr() for c in cols])
    labs = (C.c_char_p * (nc + 1))(*[l.encode() for l in labels])
    ev = np.zeros((logn, nc + 1, 8), dtype=np.uint32)
    ch = np.zeros((logn, 8), dtype=np.uint32)
    fin = np.zeros((nc, 8), dtype=np.uint32)
    st = (C.c_uint8 * 32)(*tr.state)
    prover._ck(prover._L.zkh_fr_sumcheck(prover._h, ptrs, nc, logn, labs, st, ev.ctypes.data, ch.ctypes.data,
                                         fin.ctypes.data))
    tr.state = bytes(st)
    return [unpack(e) for e in ev], unpack(ch), unpack(fin)


def inv_add(prover, t, beta):
    """tlookup_inv_kernel (zkllm-src/tlookup.cu:50-62): 1/(t[i] + beta), 0 for a zero denominator."""
    out = _new(prover, t.shape[0])
    b = _pt([beta])                       # keep the host arrays alive across the call
    prover._ck(prover._L.zkh_fr_inv_add(prover._h, t.data_ptr(), t.shape[0], b.ctypes.data, out.data_ptr()))
    return out


def mul(prover, a, b):
    """Element-wise product a * b (FrTensor::operator*, zkllm-src/fr-tensor.cu:343-350)."""
    out = _new(prover, a.shape[0])
    prover._ck(prover._L.zkh_fr_mul(prover._h, out.data_ptr(), a.data_ptr(), b.data_ptr(), a.shape[0]))
    return out


def dot(prover, a, b):
    """(a * b).sum() over Fr."""
    out = (C.c_uint8 * 32)()
    prover._ck(prover._L.zkh_fr_dot(prover._h, a.data_ptr(), b.data_ptr(), a.shape[0], out))
    return int.from_bytes(bytes(out), "little")


def lookup_sumcheck(prover, tr, A, S, Bv, T, m, alpha, beta, Cc, u):
    """fs_phase1 + fs_phase2 (zkllm-src/zkob_lookup.cuh:143-198): the logUp sumcheck over A = 1/(S+beta) (D entries),
    Bv = 1/(T+beta), the table T and the multiplicities m (N entries), u the logD-entry point.  Claim alpha + alpha^2,
    Cc = alpha^2 - sum(Bv*m).  Returns (evals[rounds][4], challenges, (A_f, S_f, B_f, T_f, m_f)); ``tr`` advances as
    the reference's transcript (labels p0..p3 per round)."""
    D, N = A.shape[0], m.shape[0]
    logD, logN = D.bit_length() - 1, N.bit_length() - 1
    if D != 1 << logD or N != 1 << logN or len(u) != logD or S.shape[0] != D or Bv.shape[0] != N or T.shape[0] != N:
        raise ValueError("lookup_sumcheck: power-of-two sizes, len(u) == log2(D)")
    ev = np.zeros((logD, 4, 8), dtype=np.uint32)
    ws = np.zeros((logD, 8), dtype=np.uint32)
    term = np.zeros((5, 8), dtype=np.uint32)
    st = (C.c_uint8 * 32)(*tr.state)
    a_, b_, c_, u_ = _pt([alpha]), _pt([beta]), _pt([Cc]), _pt(u)      # keep the host arrays alive across the call
    prover._ck(prover._L.zkh_fr_lookup_sumcheck(prover._h, A.data_ptr(), S.data_ptr(), Bv.data_ptr(), T.data_ptr(),
                                                m.data_ptr(), logD, logN, a_.ctypes.data, b_.ctypes.data,
                                                c_.ctypes.data, u_.ctypes.data, st, ev.ctypes.data,
                                                ws.ctypes.data, term.ctypes.data))
    tr.state = bytes(st)
    return [unpack(e) for e in ev], unpack(ws), tuple(unpack(term))


def mul_throughput(prover, iters=4096):
    """Montgomery products per second (in 10^9) measured on the prover's GPU."""
    out = C.c_double(0)
    prover._ck(prover._L.zkh_fr_mul_throughput(prover._h, iters, C.byref(out)))
    return out.value


def g1_pedersen_commit(prover, gens, scalars, m, n):
    """Commitment::commit (zkllm-src/commitment.cu:41-103): m row commitments over n generators.  gens: uint8 device tensor of
    n * 144 bytes (Jacobian triples), scalars: packed Fr tensor of m * n elements (pack / to_device); returns m * 144 bytes."""
    import torch
    out = torch.empty(m * 144, dtype=torch.uint8, device=gens.device)
    prover._ck(prover._L.zkh_g1_pedersen_commit(prover._h, gens.data_ptr(), scalars.data_ptr(), m, n, out.data_ptr()))
    return out


# ------------------------------------------------------------------------------------------------------------------------
# G1 openings (zkllm-src/vrf_common.cuh).  Points are 144-byte Jacobian triples: `bytes` on the host, uint8 tensors of
# n * 144 bytes on the device.
def g1_msm(prover, gens, scalars, n):
    """dev_msm (vrf_common.cuh:165-184): <g, a> over n points (n a power of two), the reference's triple."""
    out = (C.c_uint8 * 144)()
    prover._ck(prover._L.zkh_g1_msm(prover._h, gens.data_ptr(), scalars.data_ptr(), n, out))
    return bytes(out)


def g1_fold_chain(prover, src, size, us, orientation):
    """fold_chain (vrf_common.cuh:144-163): orientation 0 folds commitments (k_com_me), 1 generators (k_gen_fold)."""
    out = (C.c_uint8 * 144)()
    a = _pt(us)
    prover._ck(prover._L.zkh_g1_fold_chain(prover._h, src.data_ptr(), size, a.ctypes.data, len(us), orientation, out))
    return bytes(out)


def ipa_prove(prover, a, b, gens, Q, n, state):
    """ipa_prove (vrf_common.cuh:302-336).  a, b: packed Fr device tensors of n scalars; gens: n points on the device;
    Q: 144 bytes; state: the transcript state (32 bytes).  Returns (L, R, a_final, new_state): lists of 144-byte points."""
    rounds = n.bit_length() - 1
    L = (C.c_uint8 * (144 * max(rounds, 1)))()
    R = (C.c_uint8 * (144 * max(rounds, 1)))()
    af = (C.c_uint8 * 32)()
    st = (C.c_uint8 * 32).from_buffer_copy(state)
    q = (C.c_uint8 * 144).from_buffer_copy(Q)
    prover._ck(prover._L.zkh_g1_ipa_prove(prover._h, a.data_ptr(), b.data_ptr(), gens.data_ptr(), q, n, st, L, R, af))
    Lb, Rb = bytes(L), bytes(R)
    return ([Lb[144 * r:144 * r + 144] for r in range(rounds)], [Rb[144 * r:144 * r + 144] for r in range(rounds)],
            int.from_bytes(bytes(af), "little"), bytes(st))


def ipa_verify(prover, gens, n, Q, P0, u_b, L, R, a_final, state):
    """ipa_verify (vrf_common.cuh:340-371).  Returns (accepted, new_state).  The shape checks of the reference (round
    counts, n = 2^rounds = 2^len(u_b)) reject before any device work."""
    rounds = len(L)
    if rounds != len(R) or n != (1 << rounds) or len(u_b) != rounds or not 0 <= a_final < P:
        return False, bytes(state)
    st = (C.c_uint8 * 32).from_buffer_copy(state)
    q = (C.c_uint8 * 144).from_buffer_copy(Q)
    p0 = (C.c_uint8 * 144).from_buffer_copy(P0)
    Lb = (C.c_uint8 * (144 * max(rounds, 1))).from_buffer_copy(b"".join(L).ljust(144, b"\0"))
    Rb = (C.c_uint8 * (144 * max(rounds, 1))).from_buffer_copy(b"".join(R).ljust(144, b"\0"))
    af = (C.c_uint8 * 32).from_buffer_copy(int(a_final).to_bytes(32, "little"))
    ub = _pt(u_b)
    acc = C.c_int(0)
    prover._ck(prover._L.zkh_g1_ipa_verify(prover._h, gens.data_ptr(), n, q, p0, ub.ctypes.data, Lb, Rb, af, st, C.byref(acc)))
    return bool(acc.value), bytes(st)


def g1_rows_check(prover, lhs, a, s, b, rows):
    """The affine link of the rescaling verifier (zkllm-src/zkob_rescale.cu:226-241): the number of rows j with
    lhs[j] != s * a[j] + b[j] as group elements.  lhs, a, b: device tensors of rows * 144 bytes; s: an integer below P."""
    sv = _pt([s])
    bad = C.c_uint32(0)
    prover._ck(prover._L.zkh_g1_rows_check(prover._h, lhs.data_ptr(), a.data_ptr(), sv.ctypes.data, b.data_ptr(), rows, C.byref(bad)))
    return bad.value
