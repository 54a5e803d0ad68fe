"""The rescaling driver of the first proof stack (zk-hillclimb_b200/zkob_rescale, the reference's zkob_rescale command line).
CPU: usage errors, the refused flag, a loud failure without a CUDA device.  GPU: its selftest; every file it writes compared byte
for byte with the files of the reference's own program built from the reference tree (oracle/_ref/zkob_rescale_ref) on the same
inputs; its verifier on both programs' output, on changed files and on a remainder moved out of range."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

import fr_oracle as fo

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "zk-hillclimb_b200", "zkob_rescale")
REF_EXE = os.path.join(ROOT, "oracle", "_ref", "zkob_rescale_ref")
FILES = ["dims.bin", "com_X.bin", "com_Xr.bin", "com_rem.bin", "com_m.bin", "com_A.bin", "lookup.bin", "ipa_A.bin", "ipa_rem.bin", "ipa_m.bin"]


def run(exe, *args, timeout=900):
    return subprocess.run([exe] + [str(a) for a in args], capture_output=True, text=True, timeout=timeout)


def test_usage_and_refused_flag(tmp_path):
    assert os.path.exists(EXE), "build() makes the driver"
    assert run(EXE).returncode == 2 and run(EXE, "verify", "x").returncode == 2
    r = run(EXE, "prove", tmp_path, "seed", "X", 8, 4, 4, "gen", "q", "--wpriv", "acc", "id")
    assert r.returncode == 2 and "not built" in r.stderr
    assert run(EXE, "prove", tmp_path, "seed", "X", 8, 4, 4, "gen", "q", "--claims", "acc").returncode == 2
    import torch
    if not torch.cuda.is_available():
        (tmp_path / "X.i64").write_bytes(np.zeros(32, dtype=np.int64).tobytes())
        (tmp_path / "gen.bin").write_bytes(bytes(4 * 144))
        (tmp_path / "q.bin").write_bytes(bytes(144))
        r = run(EXE, "prove", tmp_path, "seed", tmp_path / "X.i64", 8, 4, 4, tmp_path / "gen.bin", tmp_path / "q.bin")
        assert r.returncode == 3 and "CUDA" in r.stderr and not (tmp_path / "com_X.bin").exists()
    # a layout the argument does not cover (table larger than the witness) is refused before any device work
    (tmp_path / "X.i64").write_bytes(np.zeros(4, dtype=np.int64).tobytes())
    (tmp_path / "gen.bin").write_bytes(bytes(2 * 144))
    (tmp_path / "q.bin").write_bytes(bytes(144))
    r = run(EXE, "prove", tmp_path, "seed", tmp_path / "X.i64", 2, 2, 8, tmp_path / "gen.bin", tmp_path / "q.bin")
    assert r.returncode == 3 and "layout" in r.stderr


@pytest.mark.gpu
def test_selftest():
    r = run(EXE, "selftest")
    assert r.returncode == 0 and "ALL PASS" in r.stdout and "FAIL" not in r.stdout, r.stdout + r.stderr


def _inputs(tmp_path, B, Cc, log_sf, seed):
    if not fo.ReferenceFr.available():
        pytest.skip("oracle/_ref/libfrref.so not built")
    lib = fo.ReferenceFr().lib
    if not lib.refA_gpu_available():
        pytest.skip("no GPU")
    Cp = 1 << (Cc - 1).bit_length()
    for name, n in (("gen.bin", Cp), ("q.bin", 1)):
        buf = (C.c_uint8 * (n * 144))()
        assert lib.refA_commit_random(C.c_uint32(n), buf) == 0
        (tmp_path / name).write_bytes(bytes(buf))
    g = np.random.default_rng(seed)
    # pre-rescale products of a matmul: beyond 32 bits
    lim = 1 << (log_sf + 24)                          # the quotient still fits the int32 output file
    (tmp_path / "X.i64").write_bytes(g.integers(-lim, lim, B * Cc, dtype=np.int64).tobytes())
    return tmp_path / "X.i64", tmp_path / "gen.bin", tmp_path / "q.bin"


@pytest.mark.gpu
@pytest.mark.parametrize("B,Cc,log_sf", [(8, 4, 4), (4, 16, 4), (8, 6, 6), (128, 768, 16)])
def test_files_equal_the_reference_programs(tmp_path, B, Cc, log_sf):
    if not os.path.exists(REF_EXE):
        pytest.skip("oracle/_ref/zkob_rescale_ref not built")
    X, gen, q = _inputs(tmp_path, B, Cc, log_sf, 100 * B + Cc)
    ours, ref = tmp_path / "ours", tmp_path / "ref"
    ours.mkdir()
    ref.mkdir()
    for exe, d in ((EXE, ours), (REF_EXE, ref)):
        r = run(exe, "prove", d, "run-seed:layer0.rescale", X, B, Cc, log_sf, gen, q, d / "Xr.i32")
        assert r.returncode == 0, r.stdout + r.stderr
    for name in FILES + ["Xr.i32"]:
        assert (ours / name).read_bytes() == (ref / name).read_bytes(), name
    for d in (ref, ours):
        r = run(EXE, "verify", d, "run-seed:layer0.rescale", B, Cc, log_sf, gen, q)
        assert r.returncode == 0 and "ACCEPT" in r.stdout, r.stdout + r.stderr
    assert run(EXE, "verify", ours, "run-seed:layer1.rescale", B, Cc, log_sf, gen, q).returncode == 1
    for name, off in (("lookup.bin", 4 + 32), ("com_rem.bin", 24), ("ipa_m.bin", -16)):
        raw = bytearray((ours / name).read_bytes())
        raw[off] ^= 1
        (ours / name).write_bytes(bytes(raw))
        r = run(EXE, "verify", ours, "run-seed:layer0.rescale", B, Cc, log_sf, gen, q)
        assert r.returncode == 1 and "REJECT" in r.stdout, name
        raw[off] ^= 1
        (ours / name).write_bytes(bytes(raw))
    assert run(EXE, "verify", ours, "run-seed:layer0.rescale", B, Cc, log_sf, gen, q).returncode == 0


@pytest.mark.gpu
@pytest.mark.parametrize("B,Cc,log_sf", [(8, 4, 4), (8, 6, 6)])
def test_claim_mode_files_equal_the_reference_programs(tmp_path, B, Cc, log_sf):
    if not os.path.exists(REF_EXE):
        pytest.skip("oracle/_ref/zkob_rescale_ref not built")
    X, gen, q = _inputs(tmp_path, B, Cc, log_sf, 7 * B + Cc)
    kept = {}
    for tag, exe in (("ref", REF_EXE), ("ours", EXE)):
        ob, acc, vacc = tmp_path / "ob", tmp_path / "acc", tmp_path / "vacc"
        for d in (ob, acc, vacc):
            d.mkdir()
        r = run(exe, "prove", ob, "run-seed:l0.rs", X, B, Cc, log_sf, gen, q, "--claims", acc, "l0.rs")
        assert r.returncode == 0 and "claim mode" in r.stdout, r.stdout + r.stderr
        r = run(EXE, "verify", ob, "run-seed:l0.rs", B, Cc, log_sf, gen, q, "--claims", vacc, "l0.rs")
        assert r.returncode == 0 and "ACCEPT-conditional" in r.stdout, r.stdout + r.stderr
        kept[tag] = {p.relative_to(tmp_path).as_posix(): p.read_bytes() for d in (ob, acc, vacc) for p in sorted(d.iterdir())}
        for d in (ob, acc, vacc):
            for p in d.iterdir():
                p.unlink()
            d.rmdir()
    assert kept["ours"].keys() == kept["ref"].keys()
    for name in kept["ref"]:
        assert kept["ours"][name] == kept["ref"][name], name
    assert kept["ours"]["acc/claims.bin"] == kept["ours"]["vacc/claims.bin"]
