"""The opening_batch program of the first proof stack (zk-hillclimb_b200/zkob_batchopen, the reference's zkob_batchopen command line).
CPU: usage errors and the modes that are not built.  GPU: a fully connected and a rescaling obligation proved in claim mode into
one accumulator (two generator domains, tensors of different sizes), the batch proved by this program and by the reference's own
program built from its tree (oracle/_ref/zkob_batchopen_ref) at the same paths, every batch file compared byte for byte; this
verifier on both, and on changed files with the reference's locus names."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

import fr_oracle as fo

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "zk-hillclimb_b200")
REFD = os.path.join(ROOT, "oracle", "_ref")
OURS = {"fc": os.path.join(PKG, "zkob_fc"), "rs": os.path.join(PKG, "zkob_rescale"), "bo": os.path.join(PKG, "zkob_batchopen")}
REF = {"fc": os.path.join(REFD, "zkob_fc_ref"), "rs": os.path.join(REFD, "zkob_rescale_ref"), "bo": os.path.join(REFD, "zkob_batchopen_ref")}
BATCH_FILES = ["batch_sumcheck.bin", "batch_vfin.bin", "ipa_batch_4.bin", "ipa_batch_8.bin"]


def run(exe, *args, timeout=900, env=None):
    return subprocess.run([exe] + [str(a) for a in args], capture_output=True, text=True, timeout=timeout, env=env)


def test_usage_and_modes_not_built(tmp_path):
    bo = OURS["bo"]
    assert os.path.exists(bo), "build() makes the program"
    assert run(bo).returncode == 2 and run(bo, "prove", "acc").returncode == 2
    r = run(bo, "wprove", "wacc", "seed", "q", "4=g")
    assert r.returncode == 2 and "not built" in r.stderr
    # a verifier-side list without claims is refused before any device work
    (tmp_path / "v").mkdir()
    (tmp_path / "p").mkdir()
    (tmp_path / "v" / "claims.bin").write_bytes(b"ZKCL" + (1).to_bytes(4, "little") + (0).to_bytes(4, "little"))
    r = run(bo, "verify", tmp_path / "p", tmp_path / "v", "seed", "q", "4=g")
    assert r.returncode == 1 and "REJECT[opening_batch.empty]" in r.stdout


def _setup(tmp_path):
    if not fo.ReferenceFr.available():
        pytest.skip("oracle/_ref/libfrref.so not built")
    lib = fo.ReferenceFr().lib
    if not lib.refA_gpu_available():
        pytest.skip("no GPU")
    for name, n in (("g4", 4), ("g8", 8), ("q", 1)):
        buf = (C.c_uint8 * (n * 144))()
        assert lib.refA_commit_random(C.c_uint32(n), buf) == 0
        (tmp_path / name).write_bytes(bytes(buf))
    g = np.random.default_rng(11)
    (tmp_path / "X.i32").write_bytes(g.integers(-1000, 1000, 4 * 6, dtype=np.int32).tobytes())
    (tmp_path / "W.i32").write_bytes(g.integers(-1000, 1000, 6 * 3, dtype=np.int32).tobytes())
    (tmp_path / "Z.i64").write_bytes(g.integers(-(1 << 20), 1 << 20, 8 * 4, dtype=np.int64).tobytes())
    assert run(OURS["fc"], "commit", tmp_path / "W.i32", 6, 3, tmp_path / "g4", tmp_path / "comW.bin").returncode == 0


def _walk(tmp_path, progs):
    """One prove walk (claim mode) + the verifier's recomputed claims + the batch proof; returns the directory names."""
    t = tmp_path
    for d in ("obfc", "obrs", "acc", "vacc"):
        (t / d).mkdir()
    r = run(progs["fc"], "prove", t / "obfc", "rs:l0.fc", t / "X.i32", t / "W.i32", 4, 6, 3, t / "g8", t / "g4", t / "q", "--claims", t / "acc", "l0.fc", t / "comW.bin")
    assert r.returncode == 0, r.stdout + r.stderr
    r = run(progs["rs"], "prove", t / "obrs", "rs:l0.rs", t / "Z.i64", 8, 4, 4, t / "g4", t / "q", "--claims", t / "acc", "l0.rs")
    assert r.returncode == 0, r.stdout + r.stderr
    assert run(OURS["fc"], "verify", t / "obfc", "rs:l0.fc", 4, 6, 3, t / "comW.bin", t / "g8", t / "g4", t / "q", "--claims", t / "vacc", "l0.fc").returncode == 0
    assert run(OURS["rs"], "verify", t / "obrs", "rs:l0.rs", 8, 4, 4, t / "g4", t / "q", "--claims", t / "vacc", "l0.rs").returncode == 0
    r = run(progs["bo"], "prove", t / "acc", "rs", t / "q", "4=%s" % (t / "g4"), "8=%s" % (t / "g8"))
    assert r.returncode == 0 and "PROVED opening_batch" in r.stdout, r.stdout + r.stderr


def _verify(tmp_path, *extra_env):
    t = tmp_path
    return run(OURS["bo"], "verify", t / "acc", t / "vacc", "rs", t / "q", "4=%s" % (t / "g4"), "8=%s" % (t / "g8"))


def _clear(tmp_path):
    for d in ("obfc", "obrs", "acc", "vacc"):
        for p in (tmp_path / d).iterdir():
            p.unlink()
        (tmp_path / d).rmdir()


@pytest.mark.gpu
def test_batch_files_equal_the_reference_programs_and_verify(tmp_path):
    for p in REF.values():
        if not os.path.exists(p):
            pytest.skip("reference programs not built under oracle/_ref")
    _setup(tmp_path)
    _walk(tmp_path, REF)
    ref_files = {n: (tmp_path / "acc" / n).read_bytes() for n in BATCH_FILES}
    r = _verify(tmp_path)
    assert r.returncode == 0 and "opening_batch ACCEPT (6 claims, 6 tensors, 2 domains)" in r.stdout, r.stdout + r.stderr
    _clear(tmp_path)
    _walk(tmp_path, OURS)
    for n in BATCH_FILES:
        assert (tmp_path / "acc" / n).read_bytes() == ref_files[n], n
    r = _verify(tmp_path)
    assert r.returncode == 0 and "opening_batch ACCEPT" in r.stdout, r.stdout + r.stderr
    # changed artefacts, each refused at the reference's locus
    acc = tmp_path / "acc"

    def flipped(name, off, locus):
        raw = bytearray((acc / name).read_bytes())
        raw[off] ^= 1
        (acc / name).write_bytes(bytes(raw))
        r = _verify(tmp_path)
        assert r.returncode == 1 and "REJECT[opening_batch.%s]" % locus in r.stdout, (name, r.stdout)
        raw[off] ^= 1
        (acc / name).write_bytes(bytes(raw))

    flipped("batch_sumcheck.bin", 16 + 5, "round0")
    flipped("batch_sumcheck.bin", 8, "xcheck")
    flipped("batch_vfin.bin", 8 + 3, "terminal")
    flipped("ipa_batch_8.bin", -5, "ipa8")
    flipped("ipa_batch_4.bin", 4 + 30, "ipa4")
    flipped("claims.bin", -7, "claims_match")
    os.rename(acc / "ipa_batch_4.bin", acc / "kept")
    r = _verify(tmp_path)
    assert r.returncode == 1 and "group_missing" in r.stdout
    os.rename(acc / "kept", acc / "ipa_batch_4.bin")
    com = tmp_path / "obrs" / "com_A.bin"
    raw = com.read_bytes()
    com.write_bytes(raw + raw[:144])                     # a trailing commitment row
    r = _verify(tmp_path)
    assert r.returncode == 1 and "REJECT[opening_batch.shape]" in r.stdout
    com.write_bytes(raw)
    assert _verify(tmp_path).returncode == 0
