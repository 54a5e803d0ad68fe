"""The skip-connection driver of the first proof stack (zk-hillclimb_b200/zkob_skip, the reference's zkob_skip command line): the
homomorphic sum of two commitment files byte for byte against the reference's own program (oracle/_ref/zkob_skip_ref) and against
the commitment of the summed tensors, and the verifier on honest and forged sums."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

import fr_oracle as fo

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "zk-hillclimb_b200", "zkob_skip")
FC = os.path.join(ROOT, "zk-hillclimb_b200", "zkob_fc")
REF_EXE = os.path.join(ROOT, "oracle", "_ref", "zkob_skip_ref")


def run(exe, *args, timeout=600):
    return subprocess.run([exe] + [str(a) for a in args], capture_output=True, text=True, timeout=timeout)


def test_usage(tmp_path):
    assert os.path.exists(EXE), "build() makes the driver"
    assert run(EXE).returncode == 2 and run(EXE, "add", "a", "b").returncode == 2
    assert run(EXE, "add", "a", "b", "z", "--wpriv", "x").returncode == 2
    (tmp_path / "a").write_bytes(bytes(2 * 144))
    (tmp_path / "b").write_bytes(bytes(3 * 144))
    (tmp_path / "z").write_bytes(bytes(2 * 144))
    r = run(EXE, "verify", tmp_path / "a", tmp_path / "b", tmp_path / "z")
    assert r.returncode == 1 and "row counts" in r.stdout             # refused before any device work


@pytest.mark.gpu
def test_sums_equal_the_reference_program_and_the_commitment_of_the_sum(tmp_path):
    if not fo.ReferenceFr.available():
        pytest.skip("oracle/_ref/libfrref.so not built")
    lib = fo.ReferenceFr().lib
    if not lib.refA_gpu_available():
        pytest.skip("no GPU")
    IN, OUT = 16, 8                                   # commitments of IN rows over OUT generators (the fc driver's commit mode)
    buf = (C.c_uint8 * (OUT * 144))()
    assert lib.refA_commit_random(C.c_uint32(OUT), buf) == 0
    (tmp_path / "gen").write_bytes(bytes(buf))
    g = np.random.default_rng(3)
    a, b = g.integers(-1000, 1000, IN * OUT, dtype=np.int32), g.integers(-1000, 1000, IN * OUT, dtype=np.int32)
    for name, m in (("A", a), ("B", b), ("S", a + b), ("Sbad", a + b + (np.arange(IN * OUT) == 9))):
        (tmp_path / (name + ".i32")).write_bytes(m.astype(np.int32).tobytes())
        assert run(FC, "commit", tmp_path / (name + ".i32"), IN, OUT, tmp_path / "gen", tmp_path / ("com_" + name)).returncode == 0
    r = run(EXE, "add", tmp_path / "com_A", tmp_path / "com_B", tmp_path / "Z", "--claims", tmp_path, "l0.skip")
    assert r.returncode == 0 and "0 claims emitted" in r.stdout, r.stdout + r.stderr
    if os.path.exists(REF_EXE):
        assert run(REF_EXE, "add", tmp_path / "com_A", tmp_path / "com_B", tmp_path / "Zref").returncode == 0
        assert (tmp_path / "Z").read_bytes() == (tmp_path / "Zref").read_bytes()
    # the homomorphic sum and the commitment of the summed tensor are the same points (other Jacobian triples): both verify
    assert (tmp_path / "Z").read_bytes() != (tmp_path / "com_S").read_bytes()
    for z in ("Z", "com_S"):
        r = run(EXE, "verify", tmp_path / "com_A", tmp_path / "com_B", tmp_path / z)
        assert r.returncode == 0 and "ACCEPT" in r.stdout, r.stdout + r.stderr
    r = run(EXE, "verify", tmp_path / "com_A", tmp_path / "com_B", tmp_path / "com_Sbad")
    assert r.returncode == 1 and "REJECT" in r.stdout and "1 rows" in r.stdout
