"""The head-merge driver of the first proof stack (zk-hillclimb_b200/zkob_headmerge, the reference's zkob_headmerge command line):
every file byte for byte against the reference's own program (oracle/_ref/zkob_headmerge_ref) in the plain and the claim mode for
both permutations, the merged-tensor chain file, this verifier on both programs' output and on changed files, the claims through
the batch."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

import fr_oracle as fo

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "zk-hillclimb_b200")
EXE = os.path.join(PKG, "zkob_headmerge")
BATCH = os.path.join(PKG, "zkob_batchopen")
REF_EXE = os.path.join(ROOT, "oracle", "_ref", "zkob_headmerge_ref")


def run(exe, *args, timeout=900):
    return subprocess.run([exe] + [str(a) for a in args], capture_output=True, text=True, timeout=timeout)


def test_usage_and_layout_rules(tmp_path):
    assert os.path.exists(EXE), "build() makes the driver"
    assert run(EXE).returncode == 2 and run(EXE, "prove", "x").returncode == 2
    for h in range(3):
        (tmp_path / ("O%02d.i32.bin" % h)).write_bytes(np.zeros(8 * 4, dtype=np.int32).tobytes())
    (tmp_path / "gb").write_bytes(bytes(16 * 144))
    (tmp_path / "gs").write_bytes(bytes(8 * 144))
    (tmp_path / "q").write_bytes(bytes(144))
    pre = str(tmp_path / "O")
    # the small generator set must hold HD = 4 points
    r = run(EXE, "prove", tmp_path, "s", pre, 8, 12, 4, "pi157", tmp_path / "gb", tmp_path / "gs", tmp_path / "q")
    assert r.returncode == 3 and "gen_small size" in r.stderr
    r = run(EXE, "prove", tmp_path, "s", pre, 8, 12, 4, "rot", tmp_path / "gb", tmp_path / "gs", tmp_path / "q")
    assert r.returncode == 3 and "perm" in r.stderr
    r = run(EXE, "verify", tmp_path, "s", 8, 12, 4, "concat", tmp_path / "gb", tmp_path / "gs", tmp_path / "q")
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
    heads = []
    for h in range(Cc // HD):
        o = g.integers(-(1 << 15), 1 << 15, B * HD, dtype=np.int32)
        (tmp_path / ("O%02d.i32.bin" % h)).write_bytes(o.tobytes())
        heads.append(o.reshape(B, HD))
    return str(tmp_path / "O"), heads, tmp_path / "gb", tmp_path / "gs", tmp_path / "q"


def _merged(heads, B, Cc, perm):
    M = np.concatenate(heads, axis=1)                              # B x C head concatenation
    if perm == "concat":
        return M
    m = np.arange(B * Cc)                                          # flat index of O2[i, j]; O2.flat[m] = M[m mod B, m div B]
    return M[m % B, m // B].reshape(B, Cc)


@pytest.mark.gpu
@pytest.mark.parametrize("B,Cc,HD,perm", [(8, 6, 2, "pi157"), (4, 4, 2, "pi157"), (16, 12, 4, "pi157"), (16, 6, 2, "concat"), (8, 32, 8, "concat")])
def test_files_equal_the_reference_programs(tmp_path, B, Cc, HD, perm):
    if not os.path.exists(REF_EXE):
        pytest.skip("oracle/_ref/zkob_headmerge_ref not built")
    pre, heads, gb, gs, q = _inputs(tmp_path, B, Cc, HD, 7 * B + Cc)
    dirs = {}
    for tag, exe in (("ours", EXE), ("ref", REF_EXE)):
        d = tmp_path / tag
        d.mkdir()
        r = run(exe, "prove", d, "rs:l0.merge", pre, B, Cc, HD, perm, gb, gs, q, tmp_path / (tag + "_O2.bin"))
        assert r.returncode == 0, r.stdout + r.stderr
        dirs[tag] = d
    names = sorted(p.name for p in dirs["ref"].iterdir())
    NH = Cc // HD
    assert names == sorted(p.name for p in dirs["ours"].iterdir()) and len(names) == 4 + 3 * NH
    for n in names:
        assert (dirs["ours"] / n).read_bytes() == (dirs["ref"] / n).read_bytes(), n
    chain = (tmp_path / "ours_O2.bin").read_bytes()
    assert chain == (tmp_path / "ref_O2.bin").read_bytes()
    assert np.array_equal(np.frombuffer(chain, dtype=np.int32).reshape(B, Cc), _merged(heads, B, Cc, perm))
    ours = dirs["ours"]
    for d in (dirs["ref"], ours):
        r = run(EXE, "verify", d, "rs:l0.merge", B, Cc, HD, perm, gb, gs, q)
        assert r.returncode == 0 and "ACCEPT" in r.stdout, r.stdout + r.stderr
    assert run(EXE, "verify", ours, "rs:l1.merge", B, Cc, HD, perm, gb, gs, q).returncode == 1
    other = "concat" if perm == "pi157" else "pi157"
    r = run(EXE, "verify", ours, "rs:l0.merge", B, Cc, HD, other, gb, gs, q)
    assert r.returncode == 1 and "dims.bin mismatch" in r.stdout
    if B != 8:                                                      # the changed-file loop on the 8-row shapes only
        return
    for name, off, what in (("hp00.bin", 36, "merge hadamard 00 round 0 p(0)+p(1) != claim"), ("hp01.bin", -32, "merge hadamard 01 U_f2 != 1"),
                            ("hp01.bin", -64, "merge hadamard 01 terminal"), ("ev.bin", 4, "merge hadamard 00 round 1"),
                            ("com_O01.bin", 30, "merge hadamard 00"), ("ipa_O00.bin", -9, "IPA opening of head 00 terminal vs com_O00"),
                            ("ipa_O2.bin", -9, "IPA opening of ev vs com_O2")):
        raw = bytearray((ours / name).read_bytes())
        raw[off] ^= 1
        (ours / name).write_bytes(bytes(raw))
        r = run(EXE, "verify", ours, "rs:l0.merge", B, Cc, HD, perm, gb, gs, q)
        assert r.returncode == 1 and "REJECT" in r.stdout and what in r.stdout, (name, r.stdout)
        raw[off] ^= 1
        (ours / name).write_bytes(bytes(raw))


@pytest.mark.gpu
def test_a_merged_tensor_in_the_other_layout_is_refused(tmp_path):
    """Head claims that sum to another tensor's evaluation: the proof of a concat merge does not verify as a pi157 merge even with
    dims.bin rewritten (the verifier rebuilds its own weights from the permutation it is given)."""
    B, Cc, HD = 8, 16, 4
    pre, _, gb, gs, q = _inputs(tmp_path, B, Cc, HD, 5)
    ob = tmp_path / "ob"
    ob.mkdir()
    assert run(EXE, "prove", ob, "s", pre, B, Cc, HD, "concat", gb, gs, q).returncode == 0
    (ob / "dims.bin").write_bytes(np.array([B, Cc, HD, 0], dtype=np.uint32).tobytes())
    r = run(EXE, "verify", ob, "s", B, Cc, HD, "pi157", gb, gs, q)
    assert r.returncode == 1 and "REJECT" in r.stdout


@pytest.mark.gpu
@pytest.mark.parametrize("perm", ["pi157", "concat"])
def test_claim_mode_files_equal_the_reference_and_the_batch_accepts(tmp_path, perm):
    if not os.path.exists(REF_EXE):
        pytest.skip("oracle/_ref/zkob_headmerge_ref not built")
    B, Cc, HD = 8, 16, 8
    pre, _, gb, gs, q = _inputs(tmp_path, B, Cc, HD, 31)
    kept = {}
    for tag, exe in (("ref", REF_EXE), ("ours", EXE)):
        ob, acc, vacc = tmp_path / "ob", tmp_path / "acc", tmp_path / "vacc"
        for d in (ob, acc, vacc):
            d.mkdir()
        r = run(exe, "prove", ob, "rs:l0.merge", pre, B, Cc, HD, perm, gb, gs, q, "--claims", acc, "l0.merge")
        assert r.returncode == 0 and "3 claims emitted" in r.stdout, r.stdout + r.stderr
        r = run(exe, "verify", ob, "rs:l0.merge", B, Cc, HD, perm, gb, gs, q, "--claims", vacc, "l0.merge")
        assert r.returncode == 0 and "ACCEPT-conditional (3 claims" in r.stdout, r.stdout + r.stderr
        kept[tag] = {p.relative_to(tmp_path).as_posix(): p.read_bytes() for d in (ob, acc, vacc) for p in sorted(d.iterdir())}
        if tag == "ours":
            assert run(BATCH, "prove", acc, "rs", q, "16=%s" % gb, "8=%s" % gs).returncode == 0
            r = run(BATCH, "verify", acc, vacc, "rs", q, "16=%s" % gb, "8=%s" % gs)
            assert r.returncode == 0 and "opening_batch ACCEPT (3 claims, 3 tensors, 2 domains)" in r.stdout, r.stdout + r.stderr
        for d in (ob, acc, vacc):
            for p in d.iterdir():
                p.unlink()
            d.rmdir()
    assert kept["ours"].keys() == kept["ref"].keys()
    for name in kept["ref"]:
        assert kept["ours"][name] == kept["ref"][name], name
    assert kept["ours"]["acc/claims.bin"] == kept["ours"]["vacc/claims.bin"]
