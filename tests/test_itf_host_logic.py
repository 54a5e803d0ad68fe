"""One decoder layer (p3itf::prove, non-zk) through the host logic in zk_hillclimb_b200.ig on CPU: witness chain,
commitments, 24 + 2A sub-proofs, merged lookups, public I/O bindings and batched openings; the proof must be
accepted by the reference's own host-only layer verifier on the same transcript."""
import numpy as np
import pytest

from ig_helpers import OracleGadgetEngine, StridedMatmulEngine, arr, layer_inputs, ref_itf_verify


@pytest.mark.parametrize("dims", [(4, 8, 2, 4, 16, 1), (4, 8, 2, 4, 8, 2)])
def test_layer_accepted_by_reference_verifier(tmp_path, orc, ref, zk, dims):
    R, Q = 1, 24
    ig = zk.ig
    c = ig.Config(*dims)
    T = ig.build_tables(zk.load_library(), c.d, c.btop)
    x0, Wt = layer_inputs(ig, c, 11)
    w = ig.itf_build_witness(c, x0, Wt, T)
    eng = OracleGadgetEngine(orc)
    col = lambda a: arr(eng, a)
    o = ig.itf_commit_all(eng, w, Wt, R, col)
    tr = zk.Transcript("itf-layer")
    pf = ig.itf_prove(eng, tr, c, w, o, Wt, T, R, Q, col)
    wroots = [x[1] for x in o["w"]] + [o["g1"][1], o["g2"][1]]
    st0 = zk.Transcript("itf-layer").state
    ok, st = ref_itf_verify(ref, st0, c, x0, o["x0"][1], wroots, Wt, w["out"], R, Q, pf)
    assert ok and st == tr.state
    # a wrong public output, a wrong weight root and a flipped proof byte are rejected
    bad_out = w["out"].copy()
    bad_out[3] = (int(bad_out[3]) + 1) % 0xFFFFFFFF00000001
    assert not ref_itf_verify(ref, st0, c, x0, o["x0"][1], wroots, Wt, bad_out, R, Q, pf)[0]
    assert not ref_itf_verify(ref, st0, c, x0, o["x0"][1], wroots[1:] + wroots[:1], Wt, w["out"], R, Q, pf)[0]
    for off in (30, len(pf) // 2, len(pf) - 9):
        bad = bytearray(pf)
        bad[off] ^= 1
        assert not ref_itf_verify(ref, st0, c, x0, o["x0"][1], wroots, Wt, w["out"], R, Q, bytes(bad))[0]
    native_layer_verifier_agrees(tmp_path, dims, x0, Wt, o, w, pf, R, Q)


def native_layer_verifier_agrees(tmp_path, dims, x0, Wt, o, w, pf, R, Q):
    """The C++ host verifier (include/zkh_p3_layer_verify.hpp through the program zkh_p3_layer; no GPU, no reference) gives the
    reference verifier's answers on the same proof: accept, and reject for a wrong output, a wrong weight root, a flipped byte."""
    import os
    import subprocess
    from test_cxx_layer_gpu import EXE, write_inputs
    if not os.path.exists(EXE):
        pytest.skip("zkh_p3_layer not built")
    inp, outp = str(tmp_path / "in.i32"), str(tmp_path / "proof.bin")
    write_inputs(inp, x0, Wt)
    roots = [o["x0"][1]] + [x[1] for x in o["w"]] + [o["g1"][1], o["g2"][1]]
    pub = b"".join(roots) + np.ascontiguousarray(w["out"], dtype=np.uint64).tobytes()
    args = [EXE, "verify", inp, outp] + [str(d) for d in dims] + [str(R), str(Q), "itf-layer"]

    def run(proof, pubdata):
        open(outp, "wb").write(proof)
        open(outp + ".pub", "wb").write(pubdata)
        r = subprocess.run(args, capture_output=True, text=True, timeout=600)
        assert r.returncode in (0, 1), r.stderr
        return r.returncode == 0, r.stdout.strip()
    ok, why = run(pf, pub)
    assert ok, why
    bad_pub = bytearray(pub)
    bad_pub[320 + 3 * 8] ^= 1                       # public output entry 3
    assert not run(pf, bytes(bad_pub))[0]
    swapped = b"".join([roots[0]] + roots[2:8] + roots[1:2] + roots[8:]) + pub[320:]
    assert not run(pf, swapped)[0]
    for off in (30, len(pf) // 2, len(pf) - 9):
        bad = bytearray(pf)
        bad[off] ^= 1
        assert not run(bytes(bad), pub)[0]


def _flat(v):
    import torch
    if isinstance(v, dict):
        return [x for k in sorted(v) for x in _flat(v[k])]
    if isinstance(v, (list, tuple)):
        return [x for e in v for x in _flat(e)]
    if v is None:
        return [None]
    if isinstance(v, torch.Tensor):
        v = v.cpu().numpy()
    v = np.asarray(v)
    return [v.view(np.uint64) if v.dtype == np.int64 else v.astype(np.uint64)]


@pytest.mark.parametrize("dims", [(4, 8, 2, 4, 16, 2), (8, 16, 2, 8, 32, 1)])
def test_tensor_witness_chain_equals_numpy_chain(zk, dims):
    """The tensor-arithmetic witness chain (ig_dev, here on the CPU) gives every column and index array of the numpy chain."""
    from zk_hillclimb_b200 import ig_dev
    ig = zk.ig
    c = ig.Config(*dims)
    T = ig.build_tables(zk.load_library(), c.d, c.btop)
    x0, Wt = layer_inputs(ig, c, 9)
    w = ig.itf_build_witness(c, x0, Wt, T)
    wd = ig_dev.itf_build_witness(c, x0, Wt, T, device="cpu", engine=StridedMatmulEngine())
    for k, v in w.items():
        a, b = _flat(v), _flat(wd[k])
        assert len(a) == len(b), k
        for x, y in zip(a, b):
            assert (x is None and y is None) or (x.shape == y.shape and (x == y).all()), k
