"""The bf16 gadgets and the composed fp8 transformer layer on CUDA: the CUDA engine gives the bytes the CPU stand-in engine
gives (same host logic, different engine), and the reference's host-only verifiers accept."""
import numpy as np
import pytest

from hwl_helpers import OracleHwlEngine, host_col
from test_tf_layer_host_logic import golden_layer, ref_tf_prove, ref_tf_verify, small_layer
from tfg_helpers import bf16_add_cases, bf16_patterns, load_art, ref_verify3, ref_verify_roots

pytestmark = pytest.mark.gpu


def dev_kw(prover):
    return {"device": "cuda:%d" % prover.device, "inverse": lambda t: prover.inv_all_add(t.contiguous(), 0)}


ident = lambda t: t


def test_swiglu_and_add_gadgets(orc, ref, zk, prover):
    R, Q = 1, 24
    tfg = zk.tfg
    art = load_art(ref, zk)
    rng = np.random.default_rng(3)
    n = 1 << 10
    gate, up = bf16_patterns(rng, n, 2.0), bf16_patterns(rng, n, 1.0)
    wt = tfg.swg_witness(gate, up, art, **dev_kw(prover))
    assert (wt["M"] == tfg.swg_witness(gate, up, art)["M"]).all()
    ops = tfg.swg_commit_operands(prover, wt, R, ident)
    tr = zk.Transcript("swg")
    pf = tfg.swg_prove(prover, tr, wt, tfg.swg_tables(art), ops, R, Q, ident)
    ok, st = ref_verify3(ref, "ref_swg_verify", zk.Transcript("swg").state, [ops[k][1] for k in ("GATE", "UP", "M")], n, R, Q, pf)
    assert ok and st == tr.state
    a, b = bf16_add_cases(rng, n)
    wt = tfg.bfa_witness(a, b, **dev_kw(prover))
    ops = tfg.bfa_commit_operands(prover, wt, R, ident)
    tr = zk.Transcript("bfa")
    pf = tfg.bfa_prove(prover, tr, wt, tfg.bfa_tables(), ops, R, Q, ident)
    ok, st = ref_verify3(ref, "ref_bfa_verify", zk.Transcript("bfa").state, [ops[k][1] for k in ("X1", "X2", "OUT")], n, R, Q, pf)
    assert ok and st == tr.state


def test_rope_softmax_rmsnorm_quant_gadgets(orc, ref, zk, prover):
    R, Q = 1, 24
    tfg = zk.tfg
    rng = np.random.default_rng(4)
    art = load_art(ref, zk, 6)
    # RMSNorm + quantise, 16 rows of 64
    x = bf16_patterns(rng, 16 * 64, 1.5)
    g = zk.tfart  # gains around 1
    gains = np.vectorize(g.bf_from_f64, otypes=[np.uint16])(1.0 + rng.normal(0, 0.1, 64))
    wt = tfg.rms_witness(x, gains, 16, art, **dev_kw(prover))
    ops = tfg.rms_commit_operands(prover, wt, R, ident)
    tr = zk.Transcript("rms")
    pf = tfg.rms_prove(prover, tr, wt, tfg.rms_tables(art), art, ops, R, Q, ident)
    ok, st = ref_verify_roots(ref, "ref_rms_verify", zk.Transcript("rms").state, [ops[k][1] for k in ("X", "G", "Y")], (16, 6), R, Q, pf)
    assert ok and st == tr.state
    wq = tfg.qnt_witness(wt["Y"], 16, 6, art, **dev_kw(prover))
    ops = tfg.qnt_commit_operands(prover, wq, R, ident)
    tr = zk.Transcript("qnt")
    pf = tfg.qnt_prove(prover, tr, wq, tfg.qnt_tables(art), ops, R, Q, ident)
    ok, st = ref_verify_roots(ref, "ref_qnt_verify", zk.Transcript("qnt").state, [ops[k][1] for k in ("X", "CODES", "SCALES")], (16, 6), R, Q, pf)
    assert ok and st == tr.state
    # RoPE 16 x 32, softmax 16 x 16 causal
    seq, dh = 16, 32
    half = dh // 2
    ang = np.arange(seq, dtype=np.float64)[:, None] * (10000.0 ** (-np.arange(half, dtype=np.float64) / half))[None, :]
    to_bf = np.vectorize(zk.tfart.bf_from_f64, otypes=[np.uint16])
    cos, sin = to_bf(np.cos(ang)).reshape(-1), to_bf(np.sin(ang)).reshape(-1)
    q = bf16_patterns(rng, seq * dh, 1.0)
    wr = tfg.rope_witness(q, cos, sin, seq, dh, art, **dev_kw(prover))
    ops = tfg.rope_commit_operands(prover, wr, R, ident)
    tr = zk.Transcript("rope")
    pf = tfg.rope_prove(prover, tr, wr, tfg.rope_tables(art), ops, R, Q, ident)
    ok, st = ref_verify_roots(ref, "ref_rope_verify", zk.Transcript("rope").state, [ops["Q"][1], ops["OUT"][1]], (seq, dh), R, Q, pf, pre=(cos, sin))
    assert ok and st == tr.state
    s = bf16_patterns(rng, seq * seq, 2.0)
    msk = np.tril(np.ones((seq, seq), dtype=np.uint8)).reshape(-1)
    ws = tfg.smx_witness(s, msk, seq, 4, art, **dev_kw(prover))
    ops = tfg.smx_commit_operands(prover, ws, R, ident)
    tr = zk.Transcript("smx")
    pf = tfg.smx_prove(prover, tr, ws, tfg.smx_tables(art), art, ops, R, Q, ident)
    ok, st = ref_verify_roots(ref, "ref_smx_verify", zk.Transcript("smx").state, [ops["S"][1], ops["P"][1]], (seq, seq, 23), R, Q, pf, pre=(msk,))
    assert ok and st == tr.state


def test_layer_witness_on_device_reproduces_reference_trace(zk, prover):
    tfg = zk.tfg
    g, W = golden_layer()
    c = tfg.TfConfig(4, 64, 2, 32, 128, 1)
    art = zk.tfart.build_art(c.ld)
    w = tfg.tf_build_witness(c, g["x0"].reshape(-1), W, art, device="cuda:%d" % prover.device, engine=prover)
    assert (w["out"] == g["out"].reshape(-1)).all() and (w["mmY"][c.mmWD] == g["trace_down"].reshape(-1)).all()
    assert (w["sm"][1]["P"] == g["trace_probs1"].reshape(-1)).all()


@pytest.mark.parametrize("dims", [(2, 16, 2, 8, 32, 1), (8, 64, 2, 32, 128, 2)])
def test_layer_proof_same_bytes_as_cpu_engine_and_verifies(orc, ref, zk, prover, dims):
    R, Q = 1, 24
    tfg = zk.tfg
    c = tfg.TfConfig(*dims)
    art = load_art(ref, zk, c.ld)
    T = tfg.tf_tables(art)
    x0, W = small_layer(zk, c, 6)
    w = tfg.tf_build_witness(c, x0, W, art, device="cuda:%d" % prover.device, engine=prover)
    o = tfg.tf_commit_all(prover, w, R, ident)
    wroots = tfg.tf_weight_roots(prover, c, W, R, ident)
    tr = zk.Transcript("tf-layer")
    pf = tfg.tf_prove(prover, tr, w, o, T, art, R, Q, ident)
    st0 = zk.Transcript("tf-layer").state
    ok, st = ref_tf_verify(ref, st0, c, x0, o["rms"][0]["X"][1], wroots, W, w["out"], R, Q, pf)
    assert ok and st == tr.state
    if ref.gpu_available():                           # the reference's own CUDA layer prover: identical bytes
        rpf, rst, ract, _ms = ref_tf_prove(ref, st0, c, x0, W, R, Q)
        assert (ract == w["out"]).all() and rpf == pf and rst == tr.state
    if dims[0] == 2:                                  # the CPU stand-in engine on the CPU witness: identical bytes
        wh = tfg.tf_build_witness(c, x0, W, art)
        eng = OracleHwlEngine(orc, ref)
        oh = tfg.tf_commit_all(eng, wh, R, host_col)
        trh = zk.Transcript("tf-layer")
        assert tfg.tf_prove(eng, trh, wh, oh, T, art, R, Q, host_col) == pf and trh.state == tr.state


def test_two_layer_model_on_device_accepted_by_reference_verifier(orc, ref, zk, prover):
    """p3mdl on the GPU engine: embedding gather, two chained layers, final RMSNorm, LM head, public logits; the proof is the
    one the CPU stand-in engine gives for the same model and the reference's model verifier accepts it."""
    from test_tf_layer_host_logic import ref_mdl_verify, small_model
    R, Q = 1, 24
    tfg = zk.tfg
    c = tfg.TfConfig(2, 16, 2, 8, 16, 1)
    nlayers, vocab = 2, 8
    art = load_art(ref, zk, c.ld)
    T = tfg.tf_tables(art)
    MW, ids = small_model(zk, c, nlayers, vocab, 21)
    dev = "cuda:%d" % prover.device
    to_dev = lambda t: t if t.is_cuda else t.to(dev)          # the model's host-side columns (embedding, head) are uploaded here
    w = tfg.mdl_build_witness(c, ids, MW, art, device=dev, engine=prover)
    o = tfg.mdl_commit(prover, w, MW, R, to_dev)
    roots = tfg.mdl_roots(prover, c, MW, R, to_dev)
    tr = zk.Transcript("mdl")
    pf = tfg.mdl_prove(prover, tr, w, o, T, art, R, Q, to_dev)
    st0 = zk.Transcript("mdl").state
    logits = np.asarray(w["logits"].cpu() if hasattr(w["logits"], "cpu") else w["logits"])
    ok, st = ref_mdl_verify(ref, st0, c, nlayers, vocab, ids, roots, MW["layers"][0], logits, R, Q, pf)
    assert ok and st == tr.state
    bad = logits.copy()
    bad[1] ^= 1
    assert not ref_mdl_verify(ref, st0, c, nlayers, vocab, ids, roots, MW["layers"][0], bad, R, Q, pf)[0]
    wh = tfg.mdl_build_witness(c, ids, MW, art)
    eng = OracleHwlEngine(orc, ref)
    oh = tfg.mdl_commit(eng, wh, MW, R, host_col)
    trh = zk.Transcript("mdl")
    assert tfg.mdl_prove(eng, trh, wh, oh, T, art, R, Q, host_col) == pf and trh.state == tr.state
