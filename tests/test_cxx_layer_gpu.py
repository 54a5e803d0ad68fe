"""The integer decoder layer proved from C++ (include/zkh_p3_layer.hpp, program zkh_p3_layer): same proof bytes as the
Python host over the same library, accepted by the reference's layer verifier, equal to the reference's own layer prover."""
import os
import subprocess

import numpy as np
import pytest

from ig_helpers import layer_inputs, ref_itf_prove, ref_itf_verify

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "zk-hillclimb_b200", "zkh_p3_layer")


def signed32(a):
    """field-lifted column -> the signed 32-bit integers a weight loader would hold."""
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint64:
        a = np.where(a >> np.uint64(63), a + np.uint64(0xFFFFFFFF), a).view(np.int64)
    return a.astype(np.int32)


def write_inputs(path, x0, Wt):
    with open(path, "wb") as f:
        for a in [x0] + list(Wt["w"]) + [Wt["g1"], Wt["g2"], Wt["ct"], Wt["st"]]:
            f.write(signed32(np.asarray(a).reshape(-1)).tobytes())


@pytest.mark.parametrize("dims", [(4, 8, 2, 4, 16, 1), (16, 32, 2, 16, 64, 2), (64, 256, 4, 64, 1024, 1)])
def test_cxx_layer_prover_same_bytes(tmp_path, ref_or_none, zk, prover, dims):
    if not os.path.exists(EXE):
        pytest.skip("zkh_p3_layer not built")
    from zk_hillclimb_b200 import ig_dev
    R, Q = 1, 24
    ig = zk.ig
    c = ig.Config(*dims)
    T = ig.build_tables(zk.load_library(), c.d, c.btop)
    x0, Wt = layer_inputs(ig, c, 11)
    inp, outp = str(tmp_path / "in.i32"), str(tmp_path / "proof.bin")
    write_inputs(inp, x0, Wt)
    r = subprocess.run([EXE, inp, outp] + [str(d) for d in dims] + [str(R), str(Q), "itf-layer"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    got = open(outp, "rb").read()
    # the C++ host verifier (no GPU work, no reference): accepts the proof, rejects a flipped byte and a wrong output grid
    vargs = [EXE, "verify", inp, outp] + [str(d) for d in dims] + [str(R), str(Q), "itf-layer"]
    v = subprocess.run(vargs, capture_output=True, text=True, timeout=600)
    assert v.returncode == 0 and "ACCEPT" in v.stdout, v.stdout + v.stderr
    if dims[1] <= 32:
        for pos in (40, len(got) // 3, len(got) - 50):
            bad = bytearray(got)
            bad[pos] ^= 1
            open(outp, "wb").write(bytes(bad))
            v = subprocess.run(vargs, capture_output=True, text=True, timeout=600)
            assert v.returncode == 1 and "REJECT" in v.stdout, (pos, v.stdout, v.stderr)
        open(outp, "wb").write(got)
        pubp = outp + ".pub"
        pb = bytearray(open(pubp, "rb").read())
        keep = bytes(pb)
        pb[320] ^= 1                                  # first element of the public output grid
        open(pubp, "wb").write(bytes(pb))
        v = subprocess.run(vargs, capture_output=True, text=True, timeout=600)
        assert v.returncode == 1 and "REJECT" in v.stdout
        open(pubp, "wb").write(keep)
        gold = os.environ.get("ZKH_WRITE_LAYER_GOLDEN")
        if gold and dims[0] == 4:                     # fixture for the CPU test of the verifier (tests/golden/make_itf_layer_golden.py)
            os.makedirs(gold, exist_ok=True)
            for src, name in ((inp, "in.i32"), (outp, "proof.bin"), (pubp, "proof.bin.pub")):
                open(os.path.join(gold, name), "wb").write(open(src, "rb").read())
    # the Python host over the same library
    w = ig_dev.itf_build_witness(c, x0, Wt, T, engine=prover)
    ident = lambda a: a
    o = ig.itf_commit_all(prover, w, w["dev_W"], R, ident)
    tr = zk.Transcript("itf-layer")
    pf = ig.itf_prove(prover, tr, c, w, o, Wt, T, R, Q, ident)
    if got != pf:                                  # say where the two proofs part (sub-proofs are length-prefixed after 24 bytes)
        n = min(len(got), len(pf))
        first = next((i for i in range(n) if got[i] != pf[i]), n)
        pytest.fail("C++ and Python layer proofs differ: lengths %d / %d, first difference at byte %d" % (len(got), len(pf), first))
    if ref_or_none is not None:
        wroots = [x[1] for x in o["w"]] + [o["g1"][1], o["g2"][1]]
        out_host = zk.p3.to_host(w["out"])
        ok, st = ref_itf_verify(ref_or_none, zk.Transcript("itf-layer").state, c, x0, o["x0"][1], wroots, Wt, out_host, R, Q, got)
        assert ok and st == tr.state
        if ref_or_none.gpu_available() and dims[1] <= 32:
            rpf, rst, grid, ms = ref_itf_prove(ref_or_none, zk.Transcript("itf-layer").state, c, x0, Wt, R, Q)
            assert rpf == got
