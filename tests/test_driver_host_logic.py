"""The driver executable zkob_p3fc (one quantised linear obligation: matmul + rescale on one transcript) and the native
verifier behind its `verify` mode (include/zkh_p3_verify.hpp), on CPU.

Proofs come from the package's host logic (p3.imm_prove / irs_prove / lu_flush / tail_prove) over the oracle-backed
stand-in engine (test infrastructure) -- the same bytes the CUDA engine produces -- and are written in the driver's file
layout.  `verify` needs no GPU: it must accept them, reject every tampered variant with exit code 1, and speak the
orchestrator's driver protocol (exit codes, ACCEPT-conditional in claim mode, the serve loop), checked with the
reference's own unmodified run_driver / DriverPool where the reference tree is present."""
import importlib.util
import os
import subprocess
import sys

import numpy as np
import pytest

from ig_helpers import OracleGadgetEngine
from irs_helpers import irs_tables, lift
from lu_helpers import _Arr

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "zk-hillclimb_b200", "zkob_p3fc")
R, Q = 1, 24


def blob(b):
    return len(b).to_bytes(4, "little") + b


def linear_proof(orc, zk, seed, B, IN, OUT, sf, rng_seed=5):
    """(files, shape args): the composed proof of Yr = round(X W / 2^sf), dimensions padded to powers of two as the driver
    pads them."""
    p3 = zk.p3
    li, lj, lk = (max(n - 1, 0).bit_length() for n in (B, IN, OUT))
    if li + lk < 1:
        li = 1
    g = np.random.default_rng(rng_seed)
    x = np.zeros((1 << li, 1 << lj), dtype=np.int64)
    w = np.zeros((1 << lj, 1 << lk), dtype=np.int64)
    x[:B, :IN] = g.integers(-127, 128, (B, IN))
    w[:IN, :OUT] = g.integers(-127, 128, (IN, OUT))
    y = x @ w
    eng = OracleGadgetEngine(orc)
    com = lambda a: (lambda c: (c, eng.commit_gpu_rootonly(c, R)))(_Arr(lift(a.reshape(-1))))
    X, W, Y = com(x), com(w), com(y)
    tr = zk.Transcript(seed)
    ledger, luq = p3.Ledger(), []
    p1 = p3.imm_prove(eng, tr, X, W, Y, lj, lk, li, R, Q, ledger)
    yo, L, iL, iY = eng.irs_witness(Y[0], sf, 1)
    Yo = (yo, eng.commit_gpu_rootonly(yo, R))
    p2 = p3.irs_prove(eng, tr, irs_tables(zk, sf), Y, Yo, (L, iL, iY), li + lk, sf, 1, R, Q, ledger, luq)
    lug = p3.lu_flush(eng, tr, luq, ledger, R)
    bo = p3.tail_prove(eng, tr, ledger, R, Q, "fc-bo")
    proof = blob(p1) + blob(p2) + len(lug).to_bytes(4, "little") + b"".join(blob(b) for b in lug) \
        + len(bo).to_bytes(4, "little") + b"".join(blob(b) for b in bo)
    nclaims = sum(len(c[2]) for c in ledger.cls)
    return {"roots": X[1] + Y[1] + Yo[1], "root_W": W[1], "proof": proof, "nclaims": nclaims}


def write_ob(tmp, files):
    ob = tmp / "ob"
    ob.mkdir(exist_ok=True)
    (ob / "roots.bin").write_bytes(files["roots"])
    (ob / "proof.bin").write_bytes(files["proof"])
    (tmp / "root_W.bin").write_bytes(files["root_W"])
    return ob


def verify_cmd(ob, tmp, seed, B, IN, OUT, sf):
    return [EXE, "verify", str(ob), seed] + [str(v) for v in (B, IN, OUT, sf, R, Q)] + [str(tmp / "root_W.bin")]


@pytest.fixture(scope="module")
def case(orc, zk):
    B, IN, OUT, sf = 6, 12, 8, 8              # padded to 8 x 16 . 16 x 8
    return (B, IN, OUT, sf), linear_proof(orc, zk, "run0:layer0.mlp.up_proj", B, IN, OUT, sf)


def test_verify_accepts_host_logic_proof_and_rejects_tampering(case, tmp_path):
    (B, IN, OUT, sf), files = case
    ob = write_ob(tmp_path, files)
    seed = "run0:layer0.mlp.up_proj"
    r = subprocess.run(verify_cmd(ob, tmp_path, seed, B, IN, OUT, sf), capture_output=True, text=True)
    assert r.returncode == 0 and r.stdout.strip() == "ACCEPT", r.stdout + r.stderr
    # another seed, other public dimensions, a weight root that is not the registered one
    assert subprocess.run(verify_cmd(ob, tmp_path, "run0:layer0.mlp.gate_proj", B, IN, OUT, sf), capture_output=True).returncode == 1
    assert subprocess.run(verify_cmd(ob, tmp_path, seed, B, IN, OUT, sf + 1), capture_output=True).returncode == 1
    (tmp_path / "root_W.bin").write_bytes(bytes([files["root_W"][0] ^ 1]) + files["root_W"][1:])
    r = subprocess.run(verify_cmd(ob, tmp_path, seed, B, IN, OUT, sf), capture_output=True, text=True)
    assert r.returncode == 1 and "REJECT" in r.stdout
    (tmp_path / "root_W.bin").write_bytes(files["root_W"])
    # a flipped bit anywhere in the proof, in any of the prover-supplied roots, and a truncated proof
    pf = files["proof"]
    rng = np.random.default_rng(11)
    for off in [8, 30, len(pf) // 5, len(pf) // 2, len(pf) - 40] + [int(x) for x in rng.integers(0, len(pf), 24)]:
        bad = bytearray(pf)
        bad[off] ^= 1 << int(rng.integers(0, 8))
        (ob / "proof.bin").write_bytes(bytes(bad))
        r = subprocess.run(verify_cmd(ob, tmp_path, seed, B, IN, OUT, sf), capture_output=True, text=True)
        assert r.returncode == 1 and r.stdout.startswith("REJECT"), (off, r.stdout, r.stderr)
    (ob / "proof.bin").write_bytes(pf[:-64])
    assert subprocess.run(verify_cmd(ob, tmp_path, seed, B, IN, OUT, sf), capture_output=True).returncode == 1
    (ob / "proof.bin").write_bytes(pf)
    for k in range(3):
        bad = bytearray(files["roots"])
        bad[32 * k + 3] ^= 4
        (ob / "roots.bin").write_bytes(bytes(bad))
        assert subprocess.run(verify_cmd(ob, tmp_path, seed, B, IN, OUT, sf), capture_output=True).returncode == 1
    # a missing file is a crash (exit code other than 0 and 1), not a verdict
    os.remove(ob / "roots.bin")
    assert subprocess.run(verify_cmd(ob, tmp_path, seed, B, IN, OUT, sf), capture_output=True).returncode not in (0, 1)


def test_verifier_agrees_with_reference_verifier_on_the_gadget_proofs(orc, ref, zk, tmp_path):
    """The standalone matmul and rescale proofs that the reference's own verifiers accept are the two halves the driver
    composes; here the composed proof of a second shape is accepted while the reference accepts its standalone twins."""
    from imm_helpers import ref_imm_verify
    from irs_helpers import ref_irs_verify
    p3 = zk.p3
    eng = OracleGadgetEngine(orc)
    g = np.random.default_rng(3)
    li, lj, lk, sf = 2, 3, 4, 14
    x, w = g.integers(-127, 128, (1 << li, 1 << lj)), g.integers(-127, 128, (1 << lj, 1 << lk))
    com = lambda a: (lambda c: (c, eng.commit_gpu_rootonly(c, R)))(_Arr(lift(a.reshape(-1))))
    X, W, Y = com(x), com(w), com((x @ w) << 6)
    tr = zk.Transcript("t-imm")
    Ym = com(x @ w)
    pf = p3.imm_prove(eng, tr, X, W, Ym, lj, lk, li, R, Q)
    assert ref_imm_verify(ref, zk.Transcript("t-imm").state, [X[1], W[1], Ym[1]], lj, lk, li, R, Q, pf)[0]
    yo, L, iL, iY = eng.irs_witness(Y[0], sf, 1)
    Yo = (yo, eng.commit_gpu_rootonly(yo, R))
    tr = zk.Transcript("t-irs")
    pf2 = p3.irs_prove(eng, tr, irs_tables(zk, sf), Y, Yo, (L, iL, iY), li + lk, sf, 1, R, Q)
    assert ref_irs_verify(ref, zk.Transcript("t-irs").state, Y[1], Yo[1], li + lk, sf, 1, R, Q, pf2)[0]
    files = linear_proof(orc, zk, "run1:lm_head", 4, 8, 16, 14, rng_seed=9)
    ob = write_ob(tmp_path, files)
    r = subprocess.run(verify_cmd(ob, tmp_path, "run1:lm_head", 4, 8, 16, 14), capture_output=True, text=True)
    assert r.returncode == 0 and "ACCEPT" in r.stdout, r.stdout + r.stderr


def test_claim_mode_and_usage_errors(case, tmp_path):
    (B, IN, OUT, sf), files = case
    ob = write_ob(tmp_path, files)
    acc = tmp_path / "vacc"
    acc.mkdir()
    cmd = verify_cmd(ob, tmp_path, "run0:layer0.mlp.up_proj", B, IN, OUT, sf) + ["--claims", str(acc), "layer0.mlp.up_proj"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0 and "ACCEPT-conditional" in r.stdout
    raw = (acc / "claims.bin").read_bytes()
    assert raw.count(b"layer0.mlp.up_proj") == files["nclaims"]
    assert subprocess.run([EXE, "verify", str(ob)], capture_output=True).returncode not in (0, 1)
    assert subprocess.run([EXE, "frobnicate"], capture_output=True).returncode == 2
    import torch
    if not torch.cuda.is_available():       # proving has no CPU path: it fails loudly
        r = subprocess.run([EXE, "selftest"], capture_output=True, text=True)
        assert r.returncode not in (0, 1) and "cannot create a context" in r.stderr


def _reference_common():
    root = os.environ.get("ZKH_REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference")
    path = os.path.join(root, "orchestrator", "common.py")
    if not os.path.exists(path):
        pytest.skip("reference tree not present")
    spec = importlib.util.spec_from_file_location("zkref_orch_common", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_driven_by_the_reference_orchestrator_helpers(case, tmp_path):
    """run_driver (one-shot) and DriverPool (the serve loop) of the reference's orchestrator/common.py, unmodified, drive
    the executable: accept, reject with expect_reject_ok, crash raised as RuntimeError, several requests on one worker."""
    C = _reference_common()
    C.GPU_LOCK = str(tmp_path / "gpu.lock")
    (B, IN, OUT, sf), files = case
    ob = write_ob(tmp_path, files)
    seed = "run0:layer0.mlp.up_proj"
    quiet = lambda *a, **k: None
    good = verify_cmd(ob, tmp_path, seed, B, IN, OUT, sf)
    ok, _, out = C.run_driver(good, "fc verify", expect_reject_ok=True, log=quiet, cwd=str(tmp_path))
    assert ok and "ACCEPT" in out
    bad = verify_cmd(ob, tmp_path, "run0:other", B, IN, OUT, sf)
    ok, _, out = C.run_driver(bad, "fc verify (wrong seed)", expect_reject_ok=True, log=quiet, cwd=str(tmp_path))
    assert not ok and "REJECT" in out
    with pytest.raises(RuntimeError):
        C.run_driver([EXE, "verify", str(tmp_path / "nowhere"), seed] + good[4:], "fc verify (missing dir)", retries=0, log=quiet,
                     cwd=str(tmp_path))
    pool = C.DriverPool(str(tmp_path), log=quiet)
    try:
        for _ in range(2):
            ok, _, out = pool.run(good, "fc verify (served)", expect_reject_ok=True)
            assert ok and "ACCEPT" in out
            ok, _, out = pool.run(bad, "fc verify (served, wrong seed)", expect_reject_ok=True)
            assert not ok and "REJECT" in out
        with pytest.raises(RuntimeError):          # a crash inside a request comes back as rc 3, the worker stays up
            pool.run([EXE, "verify", str(tmp_path / "nowhere"), seed] + good[4:], "fc verify (served, missing dir)")
        ok, _, _ = pool.run(good, "fc verify (served, after a failed request)", expect_reject_ok=True)
        assert ok
    finally:
        pool.close()


def _walk_run(orc, zk, tmp_path):
    """A two-obligation chain (the second takes the first's rescaled output) laid out as a run directory, proofs from
    the host logic over the oracle engine."""
    import json
    p3 = zk.p3
    eng = OracleGadgetEngine(orc)
    run = tmp_path / "run"
    (run / "registration").mkdir(parents=True)
    obs = [{"prefix": "layer0.mlp.up_proj", "B": 4, "IN": 8, "OUT": 16, "sf": 8, "weight": "registration/w0.i32",
            "weight_root": "registration/w0.root", "input_from": None},
           {"prefix": "layer0.mlp.down_proj", "B": 4, "IN": 16, "OUT": 8, "sf": 8, "weight": "registration/w1.i32",
            "weight_root": "registration/w1.root", "input_from": "layer0.mlp.up_proj"}]
    pub = {"R": R, "Q": Q, "input": "registration/input.i32", "input_root": "registration/input.root", "obligations": obs}
    raw = json.dumps(pub, indent=1).encode()
    (run / "public.json").write_bytes(raw)
    import hashlib
    run_seed = hashlib.sha256(raw).hexdigest()
    g = np.random.default_rng(21)
    x = g.integers(-127, 128, (4, 8))
    com = lambda a: (lambda c: (c, eng.commit_gpu_rootonly(c, R)))(_Arr(lift(np.asarray(a).reshape(-1))))
    prevYo = None
    for k, o in enumerate(obs):
        w = g.integers(-127, 128, (o["IN"], o["OUT"]))
        li, lj, lk = (max(n - 1, 0).bit_length() for n in (o["B"], o["IN"], o["OUT"]))
        X = prevYo if prevYo is not None else com(x)
        if k == 0:
            (run / "registration" / "input.root").write_bytes(X[1])
        W, Y = com(w), com(x @ w)
        (run / "registration" / ("w%d.root" % k)).write_bytes(W[1])
        tr = zk.Transcript("%s:%s" % (run_seed, o["prefix"]))
        ledger, luq = p3.Ledger(), []
        p1 = p3.imm_prove(eng, tr, X, W, Y, lj, lk, li, R, Q, ledger)
        yo, L, iL, iY = eng.irs_witness(Y[0], o["sf"], 1)
        Yo = (yo, eng.commit_gpu_rootonly(yo, R))
        p2 = p3.irs_prove(eng, tr, irs_tables(zk, o["sf"]), Y, Yo, (L, iL, iY), li + lk, o["sf"], 1, R, Q, ledger, luq)
        lug = p3.lu_flush(eng, tr, luq, ledger, R)
        bo = p3.tail_prove(eng, tr, ledger, R, Q, "fc-bo")
        proof = blob(p1) + blob(p2) + len(lug).to_bytes(4, "little") + b"".join(blob(b) for b in lug) \
            + len(bo).to_bytes(4, "little") + b"".join(blob(b) for b in bo)
        ob = run / "proofs" / o["prefix"]
        ob.mkdir(parents=True)
        (ob / "roots.bin").write_bytes(X[1] + Y[1] + Yo[1])
        (ob / "proof.bin").write_bytes(proof)
        sy = yo.a.astype(np.int64)
        sy = np.where(yo.a > np.uint64(0x7FFFFFFF80000000), (yo.a - np.uint64(0xFFFFFFFF00000001)).astype(np.int64), sy)
        x = sy.reshape(x.shape[0], -1)
        prevYo = Yo
    return run, obs


def test_verify_walk_transcript_and_harness_coverage(orc, zk, tmp_path):
    """The walk over a chained two-obligation run: ACCEPT with a transcript that the reference's check_transcript.py finds
    complete against the manifest ids of its linear_obligations(); a swapped proof, a broken chain edge and a wrong
    registered root each turn the verdict to REJECT (exit code 1 from verify.sh)."""
    import json
    import zkh_import
    zkh_import.load()
    from zk_hillclimb_b200 import p3walk
    run, obs = _walk_run(orc, zk, tmp_path)
    quiet = lambda *a, **k: None
    out = tmp_path / "transcript.json"
    tr = p3walk.verify_walk(str(run), None, str(out), log=quiet)
    assert tr["verdict"] == "ACCEPT" and tr["checked"] == p3walk.manifest_ids(json.loads((run / "public.json").read_text()))
    assert tr["edges"] == ["registered input -> layer0.mlp.up_proj", "layer0.mlp.up_proj -> layer0.mlp.down_proj"]
    # the shell entry point of the harness contract
    sh = os.path.join(ROOT, "zk-hillclimb_b200", "host", "verify.sh")
    r = subprocess.run(["bash", sh, str(run), str(run / "public.json"), str(out)], capture_output=True, text=True)
    assert r.returncode == 0 and json.loads(out.read_text())["verdict"] == "ACCEPT", r.stdout + r.stderr
    # coverage against a manifest, with the reference's checker where its tree is present
    manifest = {"obligations": [{"id": i, "waived": None} for i in tr["checked"]] + [{"id": "embedding.lookup", "waived": "not a linear layer"}]}
    (tmp_path / "manifest.json").write_text(json.dumps(manifest))
    root = os.environ.get("ZKH_REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference")
    chk = os.path.join(root, "harness", "check_transcript.py")
    if os.path.exists(chk):
        r = subprocess.run([sys.executable, chk, str(tmp_path / "manifest.json"), str(out)], capture_output=True, text=True)
        assert r.returncode == 0 and "missing: 0  unknown: 0" in r.stdout, r.stdout
        # with the reference's own DriverPool as the transport
        C = _reference_common()
        C.GPU_LOCK = str(tmp_path / "gpu.lock")
        pool = C.DriverPool(str(run), log=quiet)
        try:
            assert p3walk.verify_walk(str(run), None, None, run=pool.run, log=quiet)["verdict"] == "ACCEPT"
        finally:
            pool.close()
    # forgeries
    a, b = (run / "proofs" / o["prefix"] / "proof.bin" for o in obs)
    pa, pb = a.read_bytes(), b.read_bytes()
    a.write_bytes(pb)
    tr = p3walk.verify_walk(str(run), None, str(out), log=quiet)
    assert tr["verdict"] == "REJECT" and "layer0.mlp.up_proj.matmul" not in tr["checked"] and "layer0.mlp.down_proj.matmul" in tr["checked"]
    r = subprocess.run(["bash", sh, str(run), str(run / "public.json"), str(out)], capture_output=True, text=True)
    assert r.returncode == 1
    a.write_bytes(pa)
    rb = run / "proofs" / obs[1]["prefix"] / "roots.bin"
    good = rb.read_bytes()
    rb.write_bytes(bytes([good[0] ^ 1]) + good[1:])
    tr = p3walk.verify_walk(str(run), None, None, log=quiet)
    assert tr["verdict"] == "REJECT" and any("edge" in f for f in tr["failed"])
    rb.write_bytes(good)
    wr = run / "registration" / "w1.root"
    goodw = wr.read_bytes()
    wr.write_bytes(goodw[::-1])
    assert p3walk.verify_walk(str(run), None, None, log=quiet)["verdict"] == "REJECT"
    wr.write_bytes(goodw)
    assert p3walk.verify_walk(str(run), None, None, log=quiet)["verdict"] == "ACCEPT"
    # a statement that changes (another Q) changes the run seed: every proof is rejected
    pub = json.loads((run / "public.json").read_text())
    pub["Q"] = Q + 1
    (run / "public.json").write_text(json.dumps(pub, indent=1))
    assert p3walk.verify_walk(str(run), None, None, log=quiet)["verdict"] == "REJECT"
