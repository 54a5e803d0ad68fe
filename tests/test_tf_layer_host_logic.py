"""The composed fp8 transformer layer (p3tf, non-zk) through the host logic in zk_hillclimb_b200.tfg on CPU: the witness
chain reproduces every activation the reference's Python layer model traces (golden fixture), and the layer proof is
accepted by the reference's own host-only layer verifier on the same transcript."""
import ctypes as C
import os

import numpy as np
import pytest

from hwl_helpers import OracleHwlEngine, host_col
from tfg_helpers import load_art

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def golden_layer():
    g = np.load(os.path.join(ROOT, "tests", "golden", "tf_tiny_layer.npz"))
    W = {"w": [(g["w%s_codes" % n].reshape(-1), g["w%s_scales" % n]) for n in "qkvogud"], "g1": g["g1"], "g2": g["g2"],
         "cos": g["cos"].reshape(-1), "sin": g["sin"].reshape(-1)}
    return g, W


def test_witness_chain_reproduces_reference_trace(zk):
    tfg = zk.tfg
    g, W = golden_layer()
    c = tfg.TfConfig(4, 64, 2, 32, 128, 1)
    art = zk.tfart.build_art(c.ld)
    w = tfg.tf_build_witness(c, g["x0"].reshape(-1), W, art)
    same = lambda a, b: (np.asarray(a).reshape(-1) == np.asarray(b).reshape(-1)).all()
    assert same(w["rms"][0]["Y"], g["trace_rms1"]) and same(w["mmY"][c.mmWQ], g["trace_q"]) and same(w["mmY"][c.mmWK], g["trace_k"])
    assert same(w["mmY"][c.mmWV], g["trace_v"])
    for h in range(2):
        assert same(w["rp"][2 * h]["OUT"], g["trace_ropeq%d" % h]) and same(w["rp"][2 * h + 1]["OUT"], g["trace_ropek%d" % h])
        assert same(w["mmY"][c.mmQK(h)], g["trace_scores%d" % h]) and same(w["sm"][h]["P"], g["trace_probs%d" % h])
        assert same(w["mmY"][c.mmPV(h)], g["trace_attnout%d" % h])
    assert same(w["mmY"][c.mmWO], g["trace_oproj"]) and same(w["res"][0]["O"], g["trace_resid1"])
    assert same(w["rms"][1]["Y"], g["trace_rms2"]) and same(w["mmY"][c.mmWG], g["trace_gate"]) and same(w["mmY"][c.mmWU], g["trace_up"])
    assert same(w["sw"]["M"], g["trace_swiglu"]) and same(w["mmY"][c.mmWD], g["trace_down"])
    assert same(w["out"], g["out"])


def ref_tf_verify(ref, st, c, x0, rX0, wroots, W, out, R, Q, proof, wmax=23):
    s = (C.c_uint8 * 32)(*st)
    dims = (C.c_uint32 * 6)(*c.dims())
    vp = lambda a: np.ascontiguousarray(a, dtype=np.uint16).ctypes.data_as(C.c_void_p)
    keep = [np.ascontiguousarray(a, dtype=np.uint16) for a in (x0, W["cos"], W["sin"], out)]
    ok = ref.lib.ref_tf_verify(s, dims, keep[0].ctypes.data_as(C.c_void_p), rX0, b"".join(wroots), keep[1].ctypes.data_as(C.c_void_p),
                               keep[2].ctypes.data_as(C.c_void_p), keep[3].ctypes.data_as(C.c_void_p), C.c_uint32(wmax), C.c_uint32(R),
                               C.c_uint32(Q), bytes(proof), C.c_size_t(len(proof)))
    return bool(ok), bytes(s)


def ref_tf_prove(ref, st, c, x0, W, R, Q, wmax=23):
    """The reference's own build_witness (host) + commit_all + prove (CUDA): (proof bytes, state, output patterns, [ms])."""
    s = (C.c_uint8 * 32)(*st)
    dims = (C.c_uint32 * 6)(*c.dims())
    codes = [np.ascontiguousarray(w[0], dtype=np.uint8) for w in W["w"]]
    scales = [np.ascontiguousarray(w[1], dtype=np.uint32) for w in W["w"]]
    pc = (C.c_void_p * 7)(*[a.ctypes.data for a in codes])
    ps = (C.c_void_p * 7)(*[a.ctypes.data for a in scales])
    keep = [np.ascontiguousarray(a, dtype=np.uint16) for a in (x0, W["g1"], W["g2"], W["cos"], W["sin"])]
    cap = 1 << 30
    out = (C.c_uint8 * cap)()
    act = np.zeros(c.T * c.d, dtype=np.uint16)
    ms = (C.c_double * 3)()
    f = ref.lib.ref_tf_prove
    f.restype = C.c_size_t
    n = f(s, dims, *[a.ctypes.data_as(C.c_void_p) for a in keep[:1]], pc, ps, *[a.ctypes.data_as(C.c_void_p) for a in keep[1:]],
          C.c_uint32(wmax), C.c_uint32(R), C.c_uint32(Q), out, C.c_size_t(cap), act.ctypes.data_as(C.c_void_p), ms)
    return bytes(out[:n]), bytes(s), act, list(ms)


def small_layer(zk, c, seed):
    """Seeded weights as the reference's tiny layer draws them: random e4m3 codes, log-normal fp32 row scales around 0.02."""
    rng = np.random.default_rng(seed)

    def wmat(n, k, extra=1.0):
        return rng.integers(0, 256, n * k).astype(np.uint8), (np.exp(rng.normal(0, 0.3, n)) * 0.02 * extra).astype(np.float32).view(np.uint32)
    d, dff, dh, seq = c.d, c.dff, c.dh, c.seq
    to_bf = np.vectorize(zk.tfart.bf_from_f64, otypes=[np.uint16])
    half = dh // 2
    ang = np.arange(seq, dtype=np.float64)[:, None] * (10000.0 ** (-np.arange(half, dtype=np.float64) / half))[None, :]
    W = {"w": [wmat(d, d, 1.0 / np.sqrt(dh)), wmat(d, d), wmat(d, d), wmat(d, d), wmat(dff, d), wmat(dff, d), wmat(d, dff)],
         "g1": to_bf(1.0 + rng.normal(0, 0.1, d)), "g2": to_bf(1.0 + rng.normal(0, 0.1, d)),
         "cos": to_bf(np.cos(ang)).reshape(-1), "sin": to_bf(np.sin(ang)).reshape(-1)}
    x0 = to_bf(rng.normal(0, 1.0, c.T * d))
    return x0, W


@pytest.mark.parametrize("dims", [(2, 16, 2, 8, 32, 1), (2, 16, 2, 8, 16, 2)])
def test_layer_accepted_by_reference_verifier(orc, ref, zk, dims):
    R, Q = 1, 24
    tfg = zk.tfg
    c = tfg.TfConfig(*dims)
    art = load_art(ref, zk, c.ld)
    T = tfg.tf_tables(art)
    x0, W = small_layer(zk, c, 5)
    w = tfg.tf_build_witness(c, x0, W, art)
    eng = OracleHwlEngine(orc, ref)
    o = tfg.tf_commit_all(eng, w, R, host_col)
    wroots = tfg.tf_weight_roots(eng, c, W, R, host_col)
    assert wroots[0] == o["mm"][c.mmWQ]["W"][1] and wroots[14] == o["rms"][0]["G"][1]
    tr = zk.Transcript("tf-layer")
    pf = tfg.tf_prove(eng, tr, w, o, T, art, R, Q, host_col)
    st0 = zk.Transcript("tf-layer").state
    rX0 = o["rms"][0]["X"][1]
    ok, st = ref_tf_verify(ref, st0, c, x0, rX0, wroots, W, w["out"], R, Q, pf)
    assert ok and st == tr.state
    bad_out = w["out"].copy()
    bad_out[3] ^= 1
    assert not ref_tf_verify(ref, st0, c, x0, rX0, wroots, W, bad_out, R, Q, pf)[0]
    assert not ref_tf_verify(ref, st0, c, x0, rX0, wroots[1:] + wroots[:1], W, w["out"], R, Q, pf)[0]
    for off in (30, len(pf) // 2, len(pf) - 9):
        bad = bytearray(pf)
        bad[off] ^= 1
        assert not ref_tf_verify(ref, st0, c, x0, rX0, wroots, W, w["out"], R, Q, bytes(bad))[0]


def ref_mdl_verify(ref, st, c, nlayers, vocab, ids, roots, W, logits, R, Q, proof, wmax=23):
    s = (C.c_uint8 * 32)(*st)
    dims = (C.c_uint32 * 6)(*c.dims())
    keep = [np.ascontiguousarray(ids, dtype=np.uint32)] + [np.ascontiguousarray(a, dtype=np.uint16) for a in (W["cos"], W["sin"], logits)]
    p = [a.ctypes.data_as(C.c_void_p) for a in keep]
    ok = ref.lib.ref_mdl_verify(s, dims, C.c_uint32(nlayers), C.c_uint32(vocab), p[0], b"".join(roots), p[1], p[2], p[3], C.c_uint32(wmax),
                                C.c_uint32(R), C.c_uint32(Q), bytes(proof), C.c_size_t(len(proof)))
    return bool(ok), bytes(s)


def small_model(zk, c, nlayers, vocab, seed):
    rng = np.random.default_rng(seed)
    to_bf = np.vectorize(zk.tfart.bf_from_f64, otypes=[np.uint16])
    layers = []
    for li in range(nlayers):
        _x, W = small_layer(zk, c, seed + 10 * li)
        layers.append(W)
    MW = {"vocab": vocab, "emb": to_bf(rng.normal(0, 1.0, vocab * c.d)), "layers": layers, "gF": to_bf(1.0 + rng.normal(0, 0.1, c.d)),
          "wh": (rng.integers(0, 256, vocab * c.d).astype(np.uint8), (np.exp(rng.normal(0, 0.3, vocab)) * 0.02).astype(np.float32).view(np.uint32))}
    ids = rng.integers(0, vocab, c.T)
    return MW, ids


def test_two_layer_model_accepted_by_reference_verifier(orc, ref, zk):
    """Embedding gather, two chained layers (shared commitments, no public activations), final RMSNorm, LM head, public logits."""
    R, Q = 1, 24
    tfg = zk.tfg
    c = tfg.TfConfig(2, 16, 2, 8, 16, 1)
    nlayers, vocab = 2, 8
    art = load_art(ref, zk, c.ld)
    T = tfg.tf_tables(art)
    MW, ids = small_model(zk, c, nlayers, vocab, 21)
    w = tfg.mdl_build_witness(c, ids, MW, art)
    eng = OracleHwlEngine(orc, ref)
    o = tfg.mdl_commit(eng, w, MW, R, host_col)
    assert o["lay"][1]["rms"][0]["X"][1] == o["lay"][0]["res"][1]["OUT"][1]
    roots = tfg.mdl_roots(eng, c, MW, R, host_col)
    tr = zk.Transcript("mdl")
    pf = tfg.mdl_prove(eng, tr, w, o, T, art, R, Q, host_col)
    st0 = zk.Transcript("mdl").state
    W0 = MW["layers"][0]
    ok, st = ref_mdl_verify(ref, st0, c, nlayers, vocab, ids, roots, W0, w["logits"], R, Q, pf)
    assert ok and st == tr.state
    bad_logits = w["logits"].copy()
    bad_logits[2] ^= 1
    assert not ref_mdl_verify(ref, st0, c, nlayers, vocab, ids, roots, W0, bad_logits, R, Q, pf)[0]
    bad_ids = np.array(ids).copy()
    bad_ids[0] = (bad_ids[0] + 1) % vocab
    assert not ref_mdl_verify(ref, st0, c, nlayers, vocab, bad_ids, roots, W0, w["logits"], R, Q, pf)[0]
    assert not ref_mdl_verify(ref, st0, c, nlayers, vocab, ids, roots[:4] + roots[20:] + roots[4:20], W0, w["logits"], R, Q, pf)[0]
