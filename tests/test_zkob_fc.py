"""The fully connected driver of the first proof stack (zk-hillclimb_b200/zkob_fc, the reference's zkob_fc command line).
CPU: usage errors, refused flags, and a loud failure without a CUDA device.  GPU: its selftest; every file it writes compared
byte for byte with the files of the reference's own program built from the reference tree (oracle/_ref/zkob_fc_ref) on the same
inputs; its verifier on both programs' output and on changed files; the serve loop."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

import fr_oracle as fo

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "zk-hillclimb_b200", "zkob_fc")
REF_EXE = os.path.join(ROOT, "oracle", "_ref", "zkob_fc_ref")
FILES = ["dims.bin", "com_X.bin", "com_Y.bin", "sumcheck.bin", "ipa_W.bin", "ipa_X.bin", "ipa_Y.bin"]


def run(exe, *args, timeout=900):
    return subprocess.run([exe] + [str(a) for a in args], capture_output=True, text=True, timeout=timeout)


def test_usage_and_refused_flags(tmp_path):
    assert os.path.exists(EXE), "build() makes the driver"
    assert run(EXE).returncode == 2 and run(EXE, "prove", "x").returncode == 2
    r = run(EXE, "prove", tmp_path, "seed", "X", "W", 4, 6, 3, "gi", "go", "q", "--claims", "acc", "id", "comW", "--wpriv", "wacc", "blinds")
    assert r.returncode == 2 and "not built" in r.stderr
    assert run(EXE, "prove", tmp_path, "seed", "X", "W", 4, 6, 3, "gi", "go", "q", "--claims", "acc", "id").returncode == 2   # no registered com_W
    import torch
    if not torch.cuda.is_available():
        (tmp_path / "W.i32").write_bytes(np.zeros(18, dtype=np.int32).tobytes())
        (tmp_path / "go.bin").write_bytes(bytes(4 * 144))
        r = run(EXE, "commit", tmp_path / "W.i32", 6, 3, tmp_path / "go.bin", tmp_path / "com.bin")
        assert r.returncode == 3 and "CUDA" in r.stderr and not (tmp_path / "com.bin").exists()


@pytest.mark.gpu
def test_selftest():
    r = run(EXE, "selftest")
    assert r.returncode == 0 and "ALL PASS" in r.stdout and "FAIL" not in r.stdout, r.stdout + r.stderr


def _inputs(tmp_path, B, IN, OUT, seed):
    if not fo.ReferenceFr.available():
        pytest.skip("oracle/_ref/libfrref.so not built")
    lib = fo.ReferenceFr().lib
    if not lib.refA_gpu_available():
        pytest.skip("no GPU")
    INp, OUTp = 1 << (IN - 1).bit_length(), 1 << (OUT - 1).bit_length()
    for name, n in (("gen_in.bin", INp), ("gen_out.bin", OUTp), ("q.bin", 1)):
        buf = (C.c_uint8 * (n * 144))()
        assert lib.refA_commit_random(C.c_uint32(n), buf) == 0          # the reference's own generator sampling
        (tmp_path / name).write_bytes(bytes(buf))
    g = np.random.default_rng(seed)
    (tmp_path / "X.i32").write_bytes(g.integers(-(1 << 15), 1 << 15, B * IN, dtype=np.int32).tobytes())
    (tmp_path / "W.i32").write_bytes(g.integers(-(1 << 15), 1 << 15, IN * OUT, dtype=np.int32).tobytes())
    return [tmp_path / n for n in ("X.i32", "W.i32", "gen_in.bin", "gen_out.bin", "q.bin")]


@pytest.mark.gpu
@pytest.mark.parametrize("B,IN,OUT", [(4, 6, 3), (16, 12, 5), (128, 768, 768)])
def test_files_equal_the_reference_programs(tmp_path, B, IN, OUT):
    if not os.path.exists(REF_EXE):
        pytest.skip("oracle/_ref/zkob_fc_ref not built")
    X, W, gi, go, q = _inputs(tmp_path, B, IN, OUT, 10 * B + OUT)
    ours, ref = tmp_path / "ours", tmp_path / "ref"
    ours.mkdir()
    ref.mkdir()
    for exe, d in ((EXE, ours), (REF_EXE, ref)):
        r = run(exe, "commit", W, IN, OUT, go, d / "com_W.bin")
        assert r.returncode == 0, r.stdout + r.stderr
        r = run(exe, "prove", d, "run-seed:layer0.fc", X, W, B, IN, OUT, gi, go, q, d / "Y.i64")
        assert r.returncode == 0, r.stdout + r.stderr
    for name in FILES + ["com_W.bin", "Y.i64"]:
        assert (ours / name).read_bytes() == (ref / name).read_bytes(), name
    # this verifier on the reference program's files and on its own; a wrong seed, a wrong registration, a changed file
    for d in (ref, ours):
        assert run(EXE, "verify", d, "run-seed:layer0.fc", B, IN, OUT, d / "com_W.bin", gi, go, q).returncode == 0
    assert run(EXE, "verify", ours, "run-seed:layer1.fc", B, IN, OUT, ours / "com_W.bin", gi, go, q).returncode == 1
    w2 = np.frombuffer(W.read_bytes(), dtype=np.int32).copy()
    w2[0] += 1
    (tmp_path / "W2.i32").write_bytes(w2.tobytes())
    assert run(EXE, "commit", tmp_path / "W2.i32", IN, OUT, go, tmp_path / "com_W2.bin").returncode == 0
    assert run(EXE, "verify", ours, "run-seed:layer0.fc", B, IN, OUT, tmp_path / "com_W2.bin", gi, go, q).returncode == 1
    sc = bytearray((ours / "sumcheck.bin").read_bytes())
    sc[40] ^= 1
    (ours / "sumcheck.bin").write_bytes(bytes(sc))
    r = run(EXE, "verify", ours, "run-seed:layer0.fc", B, IN, OUT, ours / "com_W.bin", gi, go, q)
    assert r.returncode == 1 and "REJECT" in r.stdout


@pytest.mark.gpu
def test_serve_loop_and_changed_opening(tmp_path):
    B, IN, OUT = 8, 8, 8
    X, W, gi, go, q = _inputs(tmp_path, B, IN, OUT, 5)
    ob = tmp_path / "ob"
    ob.mkdir()
    lines = ["commit %s %d %d %s %s" % (W, IN, OUT, go, ob / "com_W.bin"),
             "prove %s seed-a %s %s %d %d %d %s %s %s" % (ob, X, W, B, IN, OUT, gi, go, q),
             "verify %s seed-a %d %d %d %s %s %s %s" % (ob, B, IN, OUT, ob / "com_W.bin", gi, go, q),
             "verify %s seed-b %d %d %d %s %s %s %s" % (ob, B, IN, OUT, ob / "com_W.bin", gi, go, q),
             "prove %s" % ob]
    r = subprocess.run([EXE, "serve"], input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=900)
    out = r.stdout.splitlines()
    assert r.returncode == 0 and out[0] == "ZKW-READY", r.stdout + r.stderr
    assert [l for l in out if l.startswith("ZKW-RC")] == ["ZKW-RC 0", "ZKW-RC 0", "ZKW-RC 0", "ZKW-RC 1", "ZKW-RC 2"]
    ipa = bytearray((ob / "ipa_W.bin").read_bytes())
    ipa[4 + 20] ^= 1                                   # a coordinate of L_0
    (ob / "ipa_W.bin").write_bytes(bytes(ipa))
    r = run(EXE, "verify", ob, "seed-a", B, IN, OUT, ob / "com_W.bin", gi, go, q)
    assert r.returncode == 1 and "claim_W" in r.stdout


@pytest.mark.gpu
@pytest.mark.parametrize("B,IN,OUT", [(4, 6, 3), (16, 12, 5)])
def test_claim_mode_files_equal_the_reference_programs(tmp_path, B, IN, OUT):
    """--claims: claims.bin, drvstates.bin, witrefs.txt and the witness tensors of prove, and the verifier's recomputed claims, against
    the reference's program run at the same paths (the claim records carry the commitment paths)."""
    if not os.path.exists(REF_EXE):
        pytest.skip("oracle/_ref/zkob_fc_ref not built")
    X, W, gi, go, q = _inputs(tmp_path, B, IN, OUT, 3 * B + OUT)
    comW = tmp_path / "registered_com_W.bin"
    assert run(EXE, "commit", W, IN, OUT, go, comW).returncode == 0
    kept = {}
    for tag, exe in (("ref", REF_EXE), ("ours", EXE)):
        ob, acc, vacc = tmp_path / "ob", tmp_path / "acc", tmp_path / "vacc"
        for d in (ob, acc, vacc):
            d.mkdir()
        r = run(exe, "prove", ob, "run-seed:l0.fc", X, W, B, IN, OUT, gi, go, q, "--claims", acc, "l0.fc", comW)
        assert r.returncode == 0 and "claim mode" in r.stdout, r.stdout + r.stderr
        assert not (ob / "ipa_W.bin").exists()
        r = run(exe, "verify", ob, "run-seed:l0.fc", B, IN, OUT, comW, gi, go, q, "--claims", vacc, "l0.fc")
        assert r.returncode == 0 and "ACCEPT-conditional" in r.stdout, r.stdout + r.stderr
        kept[tag] = {p.relative_to(tmp_path).as_posix(): p.read_bytes() for d in (ob, acc, vacc) for p in sorted(d.iterdir())}
        for d in (ob, acc, vacc):
            for p in d.iterdir():
                p.unlink()
            d.rmdir()
    assert kept["ours"].keys() == kept["ref"].keys()
    for name in kept["ref"]:
        assert kept["ours"][name] == kept["ref"][name], name
    assert kept["ours"]["acc/claims.bin"] == kept["ours"]["vacc/claims.bin"]          # what the orchestrator compares
