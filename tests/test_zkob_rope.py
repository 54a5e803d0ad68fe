"""The rotary-embedding driver of the first proof stack (zk-hillclimb_b200/zkob_rope, the reference's zkob_rope command line): every
file byte for byte against the reference's own program (oracle/_ref/zkob_rope_ref) in the plain and the claim mode, the Y64 chain
file against a numpy statement of the integer relation, this verifier on both programs' output, on changed files and on other
tables, the claims (two of them on one tensor) through the batch."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

import fr_oracle as fo

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "zk-hillclimb_b200")
EXE = os.path.join(PKG, "zkob_rope")
BATCH = os.path.join(PKG, "zkob_batchopen")
REF_EXE = os.path.join(ROOT, "oracle", "_ref", "zkob_rope_ref")


def run(exe, *args, timeout=900):
    return subprocess.run([exe] + [str(a) for a in args], capture_output=True, text=True, timeout=timeout)


def test_usage_and_layout_rules(tmp_path):
    assert os.path.exists(EXE), "build() makes the driver"
    assert run(EXE).returncode == 2 and run(EXE, "prove", "x").returncode == 2
    (tmp_path / "T").write_bytes(np.zeros(8 * 12, dtype=np.int32).tobytes())
    (tmp_path / "cos").write_bytes(np.zeros(8 * 4, dtype=np.int32).tobytes())
    (tmp_path / "sin").write_bytes(np.zeros(8 * 4 + 1, dtype=np.int32).tobytes())
    (tmp_path / "g").write_bytes(bytes(8 * 144))
    (tmp_path / "q").write_bytes(bytes(144))
    t = tmp_path
    r = run(EXE, "prove", t, "s", t / "T", 8, 12, 4, t / "cos", t / "sin", t / "g", t / "q")
    assert r.returncode == 3 and "table file size" in r.stderr
    (tmp_path / "sin").write_bytes(np.zeros(8 * 4, dtype=np.int32).tobytes())
    r = run(EXE, "prove", t, "s", t / "T", 8, 12, 4, t / "cos", t / "sin", t / "g", t / "q")
    assert r.returncode == 3 and "generator size != C_pad" in r.stderr
    r = run(EXE, "verify", t, "s", 8, 12, 4, t / "cos", t / "sin", t / "g", t / "q")
    assert r.returncode == 1 and "bad layout params" in r.stdout


def _inputs(tmp_path, B, Cc, HD, seed):
    if not fo.ReferenceFr.available():
        pytest.skip("oracle/_ref/libfrref.so not built")
    lib = fo.ReferenceFr().lib
    if not lib.refA_gpu_available():
        pytest.skip("no GPU")
    Cp = 1 << (Cc - 1).bit_length()
    for name, k in (("g", Cp), ("q", 1)):
        buf = (C.c_uint8 * (k * 144))()
        assert lib.refA_commit_random(C.c_uint32(k), buf) == 0
        (tmp_path / name).write_bytes(bytes(buf))
    g = np.random.default_rng(seed)
    T = g.integers(-(1 << 15), 1 << 15, (B, Cc), dtype=np.int32)
    ang = g.uniform(0, 2 * np.pi, (B, HD))
    cos = np.rint(np.cos(ang) * 65536).astype(np.int32)
    sin = np.rint(np.sin(ang) * 65536).astype(np.int32)
    for name, a in (("T", T), ("cos", cos), ("sin", sin)):
        (tmp_path / name).write_bytes(a.tobytes())
    return T, cos, sin, [tmp_path / k for k in ("T", "cos", "sin", "g", "q")]


def _y64(T, cos, sin, HD):
    B, Cc = T.shape
    e = np.arange(Cc)
    sign = np.where(e & (HD // 2), 1, -1).astype(np.int64)
    Cp = 1 << (Cc - 1).bit_length()
    Tp = np.zeros((B, Cp), dtype=np.int64)
    Tp[:, :Cc] = T
    return T.astype(np.int64) * cos[:, e % HD] + Tp[:, e ^ (HD // 2)] * (sign * sin[:, e % HD])


@pytest.mark.gpu
@pytest.mark.parametrize("B,Cc,HD", [(8, 6, 2), (4, 8, 4), (16, 12, 4), (8, 32, 8)])
def test_files_equal_the_reference_programs(tmp_path, B, Cc, HD):
    if not os.path.exists(REF_EXE):
        pytest.skip("oracle/_ref/zkob_rope_ref not built")
    T, cos, sin, (Tp, cp, sp, g, q) = _inputs(tmp_path, B, Cc, HD, 3 * B + Cc)
    dirs = {}
    for tag, exe in (("ours", EXE), ("ref", REF_EXE)):
        d = tmp_path / tag
        d.mkdir()
        r = run(exe, "prove", d, "rs:l0.rope.q", Tp, B, Cc, HD, cp, sp, g, q, tmp_path / (tag + "_Y.bin"))
        assert r.returncode == 0, r.stdout + r.stderr
        dirs[tag] = d
    names = sorted(p.name for p in dirs["ref"].iterdir())
    assert names == sorted(p.name for p in dirs["ours"].iterdir()) and len(names) == 9
    for n in names:
        assert (dirs["ours"] / n).read_bytes() == (dirs["ref"] / n).read_bytes(), n
    chain = (tmp_path / "ours_Y.bin").read_bytes()
    assert chain == (tmp_path / "ref_Y.bin").read_bytes()
    assert np.array_equal(np.frombuffer(chain, dtype=np.int64).reshape(B, Cc), _y64(T, cos, sin, HD))
    ours = dirs["ours"]
    for d in (dirs["ref"], ours):
        r = run(EXE, "verify", d, "rs:l0.rope.q", B, Cc, HD, cp, sp, g, q)
        assert r.returncode == 0 and "ACCEPT" in r.stdout, r.stdout + r.stderr
    assert run(EXE, "verify", ours, "rs:l0.rope.k", B, Cc, HD, cp, sp, g, q).returncode == 1
    # a verifier holding other tables rebuilds other weights
    for name, a, what in (("cos2", cos, "h1 weight terminal"), ("sin2", sin, "h2 weight terminal")):
        b = a.copy()
        b[1, 0] += 1
        (tmp_path / name).write_bytes(b.tobytes())
        args = (tmp_path / "cos2", sp) if name == "cos2" else (cp, tmp_path / "sin2")
        r = run(EXE, "verify", ours, "rs:l0.rope.q", B, Cc, HD, *args, g, q)
        assert r.returncode == 1 and what in r.stdout, r.stdout
    if B != 8:                                                      # the changed-file loop on the 8-row shapes only
        return
    for name, off, what in (("hp1.bin", 36, "h1 round 0 p(0)+p(1) != claim"), ("hp1.bin", -32, "h1 U_f2 != 1"), ("hp2.bin", -32, "h2 U_f2 != 1"),
                            ("hp2.bin", -64, "h2 weight terminal"), ("ev.bin", 4, "h1 round 1"), ("com_Y64.bin", 30, "h1 round 1"),
                            ("ipa_T1.bin", -9, "IPA opening of h1 terminal vs com_T"),
                            ("ipa_T2.bin", -9, "IPA opening of h2 terminal vs com_T at the flipped point"), ("ipa_Y.bin", -9, "IPA opening of ev vs com_Y64")):
        raw = bytearray((ours / name).read_bytes())
        raw[off] ^= 1
        (ours / name).write_bytes(bytes(raw))
        r = run(EXE, "verify", ours, "rs:l0.rope.q", B, Cc, HD, cp, sp, g, q)
        assert r.returncode == 1 and "REJECT" in r.stdout and what in r.stdout, (name, r.stdout)
        raw[off] ^= 1
        (ours / name).write_bytes(bytes(raw))


@pytest.mark.gpu
def test_claim_mode_files_equal_the_reference_and_the_batch_accepts(tmp_path):
    if not os.path.exists(REF_EXE):
        pytest.skip("oracle/_ref/zkob_rope_ref not built")
    B, Cc, HD = 16, 12, 4
    _, _, _, (Tp, cp, sp, g, q) = _inputs(tmp_path, B, Cc, HD, 77)
    kept = {}
    for tag, exe in (("ref", REF_EXE), ("ours", EXE)):
        ob, acc, vacc = tmp_path / "ob", tmp_path / "acc", tmp_path / "vacc"
        for d in (ob, acc, vacc):
            d.mkdir()
        r = run(exe, "prove", ob, "rs:l0.rope.q", Tp, B, Cc, HD, cp, sp, g, q, "--claims", acc, "l0.rope.q")
        assert r.returncode == 0 and "3 claims emitted" in r.stdout, r.stdout + r.stderr
        r = run(exe, "verify", ob, "rs:l0.rope.q", B, Cc, HD, cp, sp, g, q, "--claims", vacc, "l0.rope.q")
        assert r.returncode == 0 and "ACCEPT-conditional (3 claims" in r.stdout, r.stdout + r.stderr
        kept[tag] = {p.relative_to(tmp_path).as_posix(): p.read_bytes() for d in (ob, acc, vacc) for p in sorted(d.iterdir())}
        if tag == "ours":
            assert run(BATCH, "prove", acc, "rs", q, "16=%s" % g).returncode == 0
            r = run(BATCH, "verify", acc, vacc, "rs", q, "16=%s" % g)
            assert r.returncode == 0 and "opening_batch ACCEPT (3 claims, 2 tensors, 1 domains)" in r.stdout, r.stdout + r.stderr
        for d in (ob, acc, vacc):
            for p in d.iterdir():
                p.unlink()
            d.rmdir()
    assert kept["ours"].keys() == kept["ref"].keys()
    for name in kept["ref"]:
        assert kept["ours"][name] == kept["ref"][name], name
    assert kept["ours"]["acc/claims.bin"] == kept["ours"]["vacc/claims.bin"]
