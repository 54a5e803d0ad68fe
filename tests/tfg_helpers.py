"""Reference windows and seeded inputs for the bf16 gadgets of the fp8 transformer layer (test infrastructure)."""
import ctypes as C
import os
import tempfile

import numpy as np

_vp = lambda a: a.ctypes.data_as(C.c_void_p)
_ART_LD = {}


def load_art(ref, zk, ld=6):
    """Build the pinned table artefact with the package's generator and hand it to the reference through the file its own
    loader reads; returns the artefact dict."""
    art = zk.tfart.build_art(ld)
    if _ART_LD.get("ld") != ld:
        with tempfile.NamedTemporaryFile(suffix=".bin", delete=False) as f:
            f.write(zk.tfart.art_bytes(art))
        try:
            assert ref.lib.ref_tf_load_art(f.name.encode()) == 1
        finally:
            os.unlink(f.name)
        _ART_LD["ld"] = ld
    return art


def bf16_patterns(rng, n, scale=1.0, zeros=0.05):
    """Seeded bf16 patterns of N(0, scale) values with a share of signed zeros."""
    x = rng.normal(0, scale, size=n).astype(np.float32)
    p = (x.view(np.uint32) >> 16).astype(np.uint16)
    z = rng.random(n) < zeros
    p[z] = np.where(rng.random(int(z.sum())) < 0.5, 0, 0x8000).astype(np.uint16)
    return p


def ref_swg_verify(ref, st, roots3, n, R, Q, proof):
    s = (C.c_uint8 * 32)(*st)
    ok = ref.lib.ref_swg_verify(s, roots3[0], roots3[1], roots3[2], C.c_uint32(n), C.c_uint32(R), C.c_uint32(Q), bytes(proof),
                                C.c_size_t(len(proof)))
    return bool(ok), bytes(s)


def ref_swg_prove(ref, st, gate, up, R, Q, gpu=True):
    s = (C.c_uint8 * 32)(*st)
    n = len(gate)
    cap = 64 << 20
    out, roots, M = (C.c_uint8 * cap)(), (C.c_uint8 * 96)(), np.zeros(n, dtype=np.uint16)
    f = ref.lib.ref_swg_prove
    f.restype = C.c_size_t
    g, u = np.ascontiguousarray(gate, dtype=np.uint16), np.ascontiguousarray(up, dtype=np.uint16)
    w = f(s, _vp(g), _vp(u), C.c_uint32(n), C.c_uint32(R), C.c_uint32(Q), int(gpu), roots, _vp(M), out, C.c_size_t(cap))
    rb = bytes(roots)
    return bytes(out[:w]), bytes(s), [rb[i * 32:(i + 1) * 32] for i in range(3)], M


def ref_verify3(ref, fn, st, roots3, n, R, Q, proof):
    """ref_swg_verify / ref_bfa_verify: three operand roots and the element count."""
    s = (C.c_uint8 * 32)(*st)
    ok = getattr(ref.lib, fn)(s, roots3[0], roots3[1], roots3[2], C.c_uint32(n), C.c_uint32(R), C.c_uint32(Q), bytes(proof),
                              C.c_size_t(len(proof)))
    return bool(ok), bytes(s)


def ref_prove2(ref, fn, st, a, b, R, Q, gpu=True):
    """ref_swg_prove / ref_bfa_prove: two bf16 input arrays -> (proof, state, three roots, output patterns)."""
    s = (C.c_uint8 * 32)(*st)
    n = len(a)
    cap = 128 << 20
    out, roots, O = (C.c_uint8 * cap)(), (C.c_uint8 * 96)(), np.zeros(n, dtype=np.uint16)
    f = getattr(ref.lib, fn)
    f.restype = C.c_size_t
    a, b = np.ascontiguousarray(a, dtype=np.uint16), np.ascontiguousarray(b, dtype=np.uint16)
    w = f(s, _vp(a), _vp(b), C.c_uint32(n), C.c_uint32(R), C.c_uint32(Q), int(gpu), roots, _vp(O), out, C.c_size_t(cap))
    rb = bytes(roots)
    return bytes(out[:w]), bytes(s), [rb[i * 32:(i + 1) * 32] for i in range(3)], O


def bf16_add_cases(rng, n):
    """bf16 pairs covering the add gadget's branches: near/far exponent gaps, cancellation, zeros, equal exponents."""
    a = bf16_patterns(rng, n, 1.0)
    b = bf16_patterns(rng, n, 1.0)
    k = n // 8
    if k:
        b[:k] = a[:k] ^ 0x8000                                   # exact cancellation
        b[k:2 * k] = a[k:2 * k]                                   # doubling
        b[2 * k:3 * k] = bf16_patterns(rng, k, 1e-4)              # far addend
        b[3 * k:4 * k] = (a[3 * k:4 * k] & 0xFF80) | rng.integers(0, 128, size=k).astype(np.uint16)   # same binade
    return a, b


def ref_verify_roots(ref, fn, st, roots, dims, R, Q, proof, pre=()):
    """ref_qnt_verify / ref_rms_verify (roots concatenated, two dims) and, with leading array arguments, the rope / softmax forms."""
    s = (C.c_uint8 * 32)(*st)
    args = [s] + [_vp(np.ascontiguousarray(a)) for a in pre] + [b"".join(roots)] + [C.c_uint32(v) for v in dims] + \
        [C.c_uint32(R), C.c_uint32(Q), bytes(proof), C.c_size_t(len(proof))]
    ok = getattr(ref.lib, fn)(*args)
    return bool(ok), bytes(s)
