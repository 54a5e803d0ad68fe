"""The gated-activation driver of the first proof stack (zk-hillclimb_b200/zkob_glu, the reference's zkob_glu command line): a
mapping lookup on G + r S against the public table and a Hadamard sumcheck for H = S .* U.  GPU: every file byte for byte against
the reference's own program (oracle/_ref/zkob_glu_ref) in the plain and the claim mode, this verifier on both programs' output and
on changed files, and the claim lists through the batch program."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

import fr_oracle as fo

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "zk-hillclimb_b200")
EXE = os.path.join(PKG, "zkob_glu")
BATCH = os.path.join(PKG, "zkob_batchopen")
REF_EXE = os.path.join(ROOT, "oracle", "_ref", "zkob_glu_ref")
FILES = ["dims.bin", "com_G.bin", "com_S.bin", "com_U.bin", "com_H.bin", "com_m.bin", "com_A.bin", "lookup.bin", "hp.bin",
         "ipa_A.bin", "ipa_comb.bin", "ipa_m.bin", "ipa_H.bin", "ipa_S.bin", "ipa_U.bin"]


def run(exe, *args, timeout=900):
    return subprocess.run([exe] + [str(a) for a in args], capture_output=True, text=True, timeout=timeout)


def test_usage_and_layout_rules(tmp_path):
    assert os.path.exists(EXE), "build() makes the driver"
    assert run(EXE).returncode == 2 and run(EXE, "prove", "x").returncode == 2
    assert run(EXE, "verify", "ob", "s", 8, 4, -8, 16, "m", "g", "q", "--wpriv", "w").returncode == 2
    # a table without the row (0, 0) is refused before any device work
    (tmp_path / "G").write_bytes(np.zeros(32, dtype=np.int32).tobytes())
    (tmp_path / "U").write_bytes(np.zeros(32, dtype=np.int32).tobytes())
    (tmp_path / "map").write_bytes(np.ones(16, dtype=np.int32).tobytes())
    (tmp_path / "gen").write_bytes(bytes(4 * 144))
    (tmp_path / "q").write_bytes(bytes(144))
    r = run(EXE, "prove", tmp_path, "s", tmp_path / "G", tmp_path / "U", 8, 4, -8, 16, tmp_path / "map", tmp_path / "gen", tmp_path / "q")
    assert r.returncode == 3 and "mapped(0)" in r.stderr


def _inputs(tmp_path, B, Cc, low, n, seed):
    if not fo.ReferenceFr.available():
        pytest.skip("oracle/_ref/libfrref.so not built")
    lib = fo.ReferenceFr().lib
    if not lib.refA_gpu_available():
        pytest.skip("no GPU")
    Cp = 1 << (Cc - 1).bit_length()
    for name, k in (("gen", Cp), ("q", 1)):
        buf = (C.c_uint8 * (k * 144))()
        assert lib.refA_commit_random(C.c_uint32(k), buf) == 0
        (tmp_path / name).write_bytes(bytes(buf))
    g = np.random.default_rng(seed)
    xs = np.arange(low, low + n, dtype=np.int64)
    (tmp_path / "map").write_bytes((xs * xs - 3 * xs).astype(np.int32).tobytes())        # f(0) = 0
    (tmp_path / "G").write_bytes(g.integers(low, low + n, B * Cc, dtype=np.int32).tobytes())
    (tmp_path / "U").write_bytes(g.integers(-(1 << 12), 1 << 12, B * Cc, dtype=np.int32).tobytes())
    return [tmp_path / k for k in ("G", "U", "map", "gen", "q")]


@pytest.mark.gpu
@pytest.mark.parametrize("B,Cc,low,n", [(8, 4, -8, 16), (4, 16, -8, 16), (8, 6, -32, 64), (32, 40, -512, 1024)])
def test_files_equal_the_reference_programs(tmp_path, B, Cc, low, n):
    if not os.path.exists(REF_EXE):
        pytest.skip("oracle/_ref/zkob_glu_ref not built")
    G, U, mp, gen, q = _inputs(tmp_path, B, Cc, low, n, 5 * B + Cc)
    ours, ref = tmp_path / "ours", tmp_path / "ref"
    ours.mkdir()
    ref.mkdir()
    for exe, d in ((EXE, ours), (REF_EXE, ref)):
        r = run(exe, "prove", d, "rs:l0.glu", G, U, B, Cc, low, n, mp, gen, q, d / "H.i64")
        assert r.returncode == 0, r.stdout + r.stderr
    for name in FILES + ["H.i64"]:
        assert (ours / name).read_bytes() == (ref / name).read_bytes(), name
    for d in (ref, ours):
        r = run(EXE, "verify", d, "rs:l0.glu", B, Cc, low, n, mp, gen, q)
        assert r.returncode == 0 and "ACCEPT" in r.stdout, r.stdout + r.stderr
    assert run(EXE, "verify", ours, "rs:l1.glu", B, Cc, low, n, mp, gen, q).returncode == 1
    for name, off in (("lookup.bin", 4 + 32), ("hp.bin", 32 + 4 + 40), ("hp.bin", -20), ("com_S.bin", 24), ("ipa_comb.bin", -16), ("ipa_U.bin", 4 + 9)):
        raw = bytearray((ours / name).read_bytes())
        raw[off] ^= 1
        (ours / name).write_bytes(bytes(raw))
        r = run(EXE, "verify", ours, "rs:l0.glu", B, Cc, low, n, mp, gen, q)
        assert r.returncode == 1 and "REJECT" in r.stdout, (name, off)
        raw[off] ^= 1
        (ours / name).write_bytes(bytes(raw))
    assert run(EXE, "verify", ours, "rs:l0.glu", B, Cc, low, n, mp, gen, q).returncode == 0


@pytest.mark.gpu
def test_claim_mode_files_equal_the_reference_and_the_batch_accepts(tmp_path):
    if not os.path.exists(REF_EXE):
        pytest.skip("oracle/_ref/zkob_glu_ref not built")
    B, Cc, low, n = 8, 6, -32, 64
    G, U, mp, gen, q = _inputs(tmp_path, B, Cc, low, n, 77)
    kept = {}
    for tag, exe in (("ref", REF_EXE), ("ours", EXE)):
        ob, acc, vacc = tmp_path / "ob", tmp_path / "acc", tmp_path / "vacc"
        for d in (ob, acc, vacc):
            d.mkdir()
        r = run(exe, "prove", ob, "rs:l0.glu", G, U, B, Cc, low, n, mp, gen, q, "--claims", acc, "l0.glu")
        assert r.returncode == 0 and "6 claims emitted" in r.stdout, r.stdout + r.stderr
        r = run(EXE, "verify", ob, "rs:l0.glu", B, Cc, low, n, mp, gen, q, "--claims", vacc, "l0.glu")
        assert r.returncode == 0 and "ACCEPT-conditional" in r.stdout, r.stdout + r.stderr
        kept[tag] = {p.relative_to(tmp_path).as_posix(): p.read_bytes() for d in (ob, acc, vacc) for p in sorted(d.iterdir())}
        if tag == "ours":
            # the six claims (the combined witness against com_comb.bin among them) through the batch program
            assert run(BATCH, "prove", acc, "rs", q, "8=%s" % gen).returncode == 0
            r = run(BATCH, "verify", acc, vacc, "rs", q, "8=%s" % gen)
            assert r.returncode == 0 and "opening_batch ACCEPT (6 claims, 6 tensors, 1 domains)" in r.stdout, r.stdout + r.stderr
            # a com_comb.bin that is not com_G + r com_S is refused by the driver's verifier
            raw = bytearray((ob / "com_comb.bin").read_bytes())
            raw[144 + 7] ^= 1
            (ob / "com_comb.bin").write_bytes(bytes(raw))
            (tmp_path / "vacc2").mkdir()
            r = run(EXE, "verify", ob, "rs:l0.glu", B, Cc, low, n, mp, gen, q, "--claims", tmp_path / "vacc2", "l0.glu")
            assert r.returncode == 1 and "com_comb.bin" in r.stdout and not (tmp_path / "vacc2" / "claims.bin").exists()
        for d in (ob, acc, vacc):
            for p in d.iterdir():
                p.unlink()
            d.rmdir()
    assert kept["ours"].keys() == kept["ref"].keys()
    for name in kept["ref"]:
        assert kept["ours"][name] == kept["ref"][name], name
    assert kept["ours"]["acc/claims.bin"] == kept["ours"]["vacc/claims.bin"]
