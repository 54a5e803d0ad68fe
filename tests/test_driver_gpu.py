"""The driver executable on the GPU: selftest, a proved and verified two-obligation walk through the serve loop, and the
proof bytes against the package's Python host logic on the same inputs (which is pinned to the reference's provers)."""
import json
import os
import subprocess

import numpy as np
import pytest

from irs_helpers import irs_tables, lift

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "zk-hillclimb_b200")
EXE = os.path.join(PKG, "zkob_p3fc")
R, Q = 1, 24


def test_driver_selftest():
    r = subprocess.run([EXE, "selftest"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "SELFTEST OK" in r.stdout and "WRONG" not in r.stdout, r.stdout + r.stderr


def test_prove_walk_then_verify_walk(zk, prover, tmp_path):
    from zk_hillclimb_b200 import p3walk
    p3 = zk.p3
    run = tmp_path / "run"
    (run / "registration").mkdir(parents=True)
    g = np.random.default_rng(77)
    shapes = [("layer0.attn.q_proj", 24, 48, 40, 8, None), ("layer0.attn.o_proj", 24, 40, 64, 9, "layer0.attn.q_proj")]
    x0 = g.integers(-127, 128, (24, 48)).astype(np.int32)
    x0.tofile(run / "registration" / "input.i32")
    obs, ws = [], []
    for k, (prefix, B, IN, OUT, sf, src) in enumerate(shapes):
        w = g.integers(-127, 128, (IN, OUT)).astype(np.int32)
        w.tofile(run / "registration" / ("w%d.i32" % k))
        ws.append(w)
        r = subprocess.run([EXE, "commit", str(run / "registration" / ("w%d.i32" % k)), str(IN), str(OUT), str(R),
                            str(run / "registration" / ("w%d.root" % k))], capture_output=True, text=True)
        assert r.returncode == 0, r.stderr
        obs.append({"prefix": prefix, "B": B, "IN": IN, "OUT": OUT, "sf": sf, "weight": "registration/w%d.i32" % k,
                    "weight_root": "registration/w%d.root" % k, "input_from": src})
    r = subprocess.run([EXE, "commit", str(run / "registration" / "input.i32"), "24", "48", str(R), str(run / "registration" / "input.root")],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    pub = {"R": R, "Q": Q, "input": "registration/input.i32", "input_root": "registration/input.root", "obligations": obs}
    (run / "public.json").write_text(json.dumps(pub, indent=1))
    quiet = lambda *a, **k: None
    secs = p3walk.prove_walk(str(run), log=quiet)
    assert set(secs) == {s[0] for s in shapes}
    out = tmp_path / "transcript.json"
    tr = p3walk.verify_walk(str(run), None, str(out), log=quiet)
    assert tr["verdict"] == "ACCEPT" and len(tr["checked"]) == 6, tr
    # the first obligation's proof equals the Python host logic's composition on the same padded inputs
    _, run_seed = p3walk.load_public(str(run / "public.json"))
    prefix, B, IN, OUT, sf, _ = shapes[0]
    li, lj, lk = 5, 6, 6
    xp = np.zeros((1 << li, 1 << lj), dtype=np.int64)
    wp = np.zeros((1 << lj, 1 << lk), dtype=np.int64)
    xp[:B, :IN], wp[:IN, :OUT] = x0, ws[0]
    com = lambda a: (lambda d: (d, prover.commit_gpu_rootonly(d, R)))(p3.to_device(lift(a.reshape(-1))))
    X, W, Y = com(xp), com(wp), com(xp @ wp)
    tr_ = zk.Transcript("%s:%s" % (run_seed, prefix))
    ledger, luq = p3.Ledger(), []
    p1 = p3.imm_prove(prover, tr_, X, W, Y, lj, lk, li, R, Q, ledger)
    yo, L, iL, iY = prover.irs_witness(Y[0], sf, 1)
    Yo = (yo, prover.commit_gpu_rootonly(yo, R))
    p2 = p3.irs_prove(prover, tr_, irs_tables(zk, sf), Y, Yo, (L, iL, iY), li + lk, sf, 1, R, Q, ledger, luq)
    lug = p3.lu_flush(prover, tr_, luq, ledger, R)
    bo = p3.tail_prove(prover, tr_, ledger, R, Q, "fc-bo")
    blob = lambda b: len(b).to_bytes(4, "little") + b
    want = blob(p1) + blob(p2) + len(lug).to_bytes(4, "little") + b"".join(blob(b) for b in lug) \
        + len(bo).to_bytes(4, "little") + b"".join(blob(b) for b in bo)
    assert (run / "proofs" / prefix / "proof.bin").read_bytes() == want
    assert (run / "proofs" / prefix / "roots.bin").read_bytes() == X[1] + Y[1] + Yo[1]
    # the rescaled output the driver hands to the next obligation is the integer result
    yr = np.fromfile(run / "data" / (prefix + ".yr.i32"), dtype=np.int32).reshape(B, OUT)
    acc = x0.astype(np.int64) @ ws[0].astype(np.int64)
    assert (yr == ((acc + (1 << (sf - 1))) >> sf)).all()
    # a tampered proof turns the walk's verdict, through the harness entry point
    pf = run / "proofs" / shapes[1][0] / "proof.bin"
    raw = bytearray(pf.read_bytes())
    raw[len(raw) // 2] ^= 2
    pf.write_bytes(bytes(raw))
    r = subprocess.run(["bash", os.path.join(PKG, "host", "verify.sh"), str(run), str(run / "public.json"), str(out)],
                       capture_output=True, text=True)
    assert r.returncode == 1 and json.loads(out.read_text())["verdict"] == "REJECT"
