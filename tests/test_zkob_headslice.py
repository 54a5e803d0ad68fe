"""The per-head slicing driver of the first proof stack (zk-hillclimb_b200/zkob_headslice, the reference's zkob_headslice command
line): every file byte for byte against the reference's own program (oracle/_ref/zkob_headslice_ref) in the plain and the claim
mode, the per-head operand files, this verifier on both programs' output and on changed files, the claims through the batch."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

import fr_oracle as fo

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "zk-hillclimb_b200")
EXE = os.path.join(PKG, "zkob_headslice")
BATCH = os.path.join(PKG, "zkob_batchopen")
REF_EXE = os.path.join(ROOT, "oracle", "_ref", "zkob_headslice_ref")


def run(exe, *args, timeout=900):
    return subprocess.run([exe] + [str(a) for a in args], capture_output=True, text=True, timeout=timeout)


def test_usage_and_layout_rules(tmp_path):
    assert os.path.exists(EXE), "build() makes the driver"
    assert run(EXE).returncode == 2 and run(EXE, "prove", "x").returncode == 2
    for name, n in (("Q", 8 * 12), ("K", 8 * 12), ("V", 8 * 12)):
        (tmp_path / name).write_bytes(np.zeros(n, dtype=np.int32).tobytes())
    (tmp_path / "gb").write_bytes(bytes(16 * 144))
    (tmp_path / "gs").write_bytes(bytes(4 * 144))
    (tmp_path / "q").write_bytes(bytes(144))
    # no generator set of size B = 8 for the transposed key slices
    r = run(EXE, "prove", tmp_path, "s", tmp_path / "Q", tmp_path / "K", tmp_path / "V", 8, 12, 4, tmp_path / "gb", tmp_path / "gs", tmp_path / "q")
    assert r.returncode == 3 and "size B" in r.stderr
    r = run(EXE, "verify", tmp_path, "s", 8, 12, 4, tmp_path / "gb", tmp_path / "gs", tmp_path / "q")
    assert r.returncode == 1 and "bad layout params" in r.stdout


def _inputs(tmp_path, B, Cc, HD, seed):
    if not fo.ReferenceFr.available():
        pytest.skip("oracle/_ref/libfrref.so not built")
    lib = fo.ReferenceFr().lib
    if not lib.refA_gpu_available():
        pytest.skip("no GPU")
    Cp = 1 << (Cc - 1).bit_length()
    for name, k in (("gb", Cp), ("gs", HD), ("q", 1)):
        buf = (C.c_uint8 * (k * 144))()
        assert lib.refA_commit_random(C.c_uint32(k), buf) == 0
        (tmp_path / name).write_bytes(bytes(buf))
    g = np.random.default_rng(seed)
    for name in ("Q", "K", "V"):
        (tmp_path / name).write_bytes(g.integers(-(1 << 15), 1 << 15, B * Cc, dtype=np.int32).tobytes())
    return [tmp_path / k for k in ("Q", "K", "V", "gb", "gs", "q")]


@pytest.mark.gpu
@pytest.mark.parametrize("B,Cc,HD", [(4, 8, 4), (16, 12, 4), (8, 32, 8)])
def test_files_equal_the_reference_programs(tmp_path, B, Cc, HD):
    if not os.path.exists(REF_EXE):
        pytest.skip("oracle/_ref/zkob_headslice_ref not built")
    Q, K, V, gb, gs, q = _inputs(tmp_path, B, Cc, HD, 9 * B + Cc)
    dirs = {}
    for tag, exe in (("ours", EXE), ("ref", REF_EXE)):
        d, sl = tmp_path / tag, tmp_path / (tag + "_slices")
        d.mkdir()
        sl.mkdir()
        r = run(exe, "prove", d, "rs:l0.slice", Q, K, V, B, Cc, HD, gb, gs, q, sl)
        assert r.returncode == 0, r.stdout + r.stderr
        dirs[tag] = (d, sl)
    for k in (0, 1):
        names = sorted(p.name for p in dirs["ref"][k].iterdir())
        assert names == sorted(p.name for p in dirs["ours"][k].iterdir()) and len(names) >= 3 * (Cc // HD)
        for n in names:
            assert (dirs["ours"][k] / n).read_bytes() == (dirs["ref"][k] / n).read_bytes(), n
    ours = dirs["ours"][0]
    for d in (dirs["ref"][0], ours):
        r = run(EXE, "verify", d, "rs:l0.slice", B, Cc, HD, gb, gs, q)
        assert r.returncode == 0 and "ACCEPT" in r.stdout, r.stdout + r.stderr
    assert run(EXE, "verify", ours, "rs:l1.slice", B, Cc, HD, gb, gs, q).returncode == 1
    for name, off, what in (("evals.bin", 32 + 3, "eK00"), ("com_Vh01.bin", 30, "eQ00"), ("ipa_Kf01.bin", -9, "eK01 vs com_K (head-selector point)")):
        raw = bytearray((ours / name).read_bytes())
        raw[off] ^= 1
        (ours / name).write_bytes(bytes(raw))
        r = run(EXE, "verify", ours, "rs:l0.slice", B, Cc, HD, gb, gs, q)
        assert r.returncode == 1 and "REJECT" in r.stdout and what in r.stdout, (name, r.stdout)
        raw[off] ^= 1
        (ours / name).write_bytes(bytes(raw))


@pytest.mark.gpu
def test_claim_mode_files_equal_the_reference_and_the_batch_accepts(tmp_path):
    if not os.path.exists(REF_EXE):
        pytest.skip("oracle/_ref/zkob_headslice_ref not built")
    B, Cc, HD = 8, 16, 8                             # the transposed key slices share the 8-generator set with Qh / Vh
    Q, K, V, gb, gs, q = _inputs(tmp_path, B, Cc, HD, 31)
    kept = {}
    for tag, exe in (("ref", REF_EXE), ("ours", EXE)):
        ob, acc, vacc = tmp_path / "ob", tmp_path / "acc", tmp_path / "vacc"
        for d in (ob, acc, vacc):
            d.mkdir()
        r = run(exe, "prove", ob, "rs:l0.slice", Q, K, V, B, Cc, HD, gb, gs, q, "--claims", acc, "l0.slice")
        assert r.returncode == 0 and "12 claims emitted" in r.stdout, r.stdout + r.stderr
        r = run(exe, "verify", ob, "rs:l0.slice", B, Cc, HD, gb, gs, q, "--claims", vacc, "l0.slice")
        assert r.returncode == 0 and "ACCEPT-conditional (12 claims" in r.stdout, r.stdout + r.stderr
        kept[tag] = {p.relative_to(tmp_path).as_posix(): p.read_bytes() for d in (ob, acc, vacc) for p in sorted(d.iterdir())}
        if tag == "ours":
            assert run(BATCH, "prove", acc, "rs", q, "16=%s" % gb, "8=%s" % gs).returncode == 0
            r = run(BATCH, "verify", acc, vacc, "rs", q, "16=%s" % gb, "8=%s" % gs)
            assert r.returncode == 0 and "opening_batch ACCEPT (12 claims, 9 tensors, 2 domains)" in r.stdout, r.stdout + r.stderr
        for d in (ob, acc, vacc):
            for p in d.iterdir():
                p.unlink()
            d.rmdir()
    assert kept["ours"].keys() == kept["ref"].keys()
    for name in kept["ref"]:
        assert kept["ours"][name] == kept["ref"][name], name
    assert kept["ours"]["acc/claims.bin"] == kept["ours"]["vacc/claims.bin"]
