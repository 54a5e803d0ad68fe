"""The causal softmax driver of the first proof stack (zk-hillclimb_b200/zkob_softmax, the reference's zkob_softmax command line):
every file byte for byte against the reference's own program (oracle/_ref/zkob_softmax_ref) in the plain and the claim mode, the
P chain file against a numpy statement of the rounding rule, this verifier on both programs' output, on changed files and on another
exp table, the sixteen claims through the batch."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

import fr_oracle as fo

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "zk-hillclimb_b200")
EXE = os.path.join(PKG, "zkob_softmax")
BATCH = os.path.join(PKG, "zkob_batchopen")
REF_EXE = os.path.join(ROOT, "oracle", "_ref", "zkob_softmax_ref")


def run(exe, *args, timeout=900):
    return subprocess.run([exe] + [str(a) for a in args], capture_output=True, text=True, timeout=timeout)


def test_usage_and_layout_rules(tmp_path):
    assert os.path.exists(EXE), "build() makes the driver"
    assert run(EXE).returncode == 2 and run(EXE, "prove", "x").returncode == 2
    t = tmp_path
    (t / "z").write_bytes(np.zeros(8 * 8, dtype=np.int32).tobytes())
    (t / "map").write_bytes(np.ones(16, dtype=np.int32).tobytes())
    (t / "g").write_bytes(bytes(8 * 144))
    (t / "q").write_bytes(bytes(144))
    r = run(EXE, "prove", t, "s", t / "z", 8, 8, -8, 16, t / "map", 4, t / "g", t / "q")       # LEN_R below NCOL
    assert r.returncode == 3 and "limb lookup layout" in r.stderr
    r = run(EXE, "prove", t, "s", t / "z", 8, 8, -8, 12, t / "map", 32, t / "g", t / "q")
    assert r.returncode == 3 and "pow2" in r.stderr
    r = run(EXE, "prove", t, "s", t / "z", 8, 8, 1, 16, t / "map", 32, t / "g", t / "q")        # z = 0 lies below LOW_E = 1
    assert r.returncode == 3 and "out of table domain" in r.stderr
    r = run(EXE, "verify", t, "s", 8, 4, -8, 16, t / "map", 32, t / "g", t / "q")
    assert r.returncode == 1 and "bad layout params" in r.stdout


def _inputs(tmp_path, B, low, len_e, len_r, seed, top):
    if not fo.ReferenceFr.available():
        pytest.skip("oracle/_ref/libfrref.so not built")
    lib = fo.ReferenceFr().lib
    if not lib.refA_gpu_available():
        pytest.skip("no GPU")
    for name, k in (("g", B), ("q", 1)):
        buf = (C.c_uint8 * (k * 144))()
        assert lib.refA_commit_random(C.c_uint32(k), buf) == 0
        (tmp_path / name).write_bytes(bytes(buf))
    g = np.random.default_rng(seed)
    z = g.integers(low, low + len_e, (B, B), dtype=np.int32)
    x = np.arange(low, low + len_e)
    emap = np.maximum(1, np.rint(top * np.exp((x - x.max()) * (8.0 / len_e)))).astype(np.int32)
    assert 2 * B * int(emap.max()) <= len_r * len_r                  # both bracket residuals fit two limbs
    (tmp_path / "z").write_bytes(z.tobytes())
    (tmp_path / "map").write_bytes(emap.tobytes())
    return z, emap, [tmp_path / k for k in ("z", "map", "g", "q")]


def _probabilities(z, emap, low):
    B = z.shape[0]
    mask = np.tril(np.ones((B, B), dtype=np.int64))
    E = emap[z - low].astype(np.int64)
    S = (E * mask).sum(axis=1, keepdims=True)
    return ((mask * E << 17) + S) // (2 * S)


CASES = [(8, -8, 16, 32, 60), (4, -8, 16, 32, 100), (16, -32, 64, 64, 120), (64, -1023, 1024, 4096, 65536)]


@pytest.mark.gpu
@pytest.mark.parametrize("B,low,len_e,len_r,top", CASES)
def test_files_equal_the_reference_programs(tmp_path, B, low, len_e, len_r, top):
    if not os.path.exists(REF_EXE):
        pytest.skip("oracle/_ref/zkob_softmax_ref not built")
    z, emap, (zp, mp, g, q) = _inputs(tmp_path, B, low, len_e, len_r, 5 * B + len_e, top)
    dirs = {}
    for tag, exe in (("ours", EXE), ("ref", REF_EXE)):
        d = tmp_path / tag
        d.mkdir()
        r = run(exe, "prove", d, "rs:l0.softmax.h00", zp, B, B, low, len_e, mp, len_r, g, q, tmp_path / (tag + "_P.bin"))
        assert r.returncode == 0, r.stdout + r.stderr
        dirs[tag] = d
    names = sorted(p.name for p in dirs["ref"].iterdir())
    assert names == sorted(p.name for p in dirs["ours"].iterdir()) and len(names) == 10 + 2 + 3 + 1 + 16
    for n in names:
        assert (dirs["ours"] / n).read_bytes() == (dirs["ref"] / n).read_bytes(), n
    chain = (tmp_path / "ours_P.bin").read_bytes()
    assert chain == (tmp_path / "ref_P.bin").read_bytes()
    assert np.array_equal(np.frombuffer(chain, dtype=np.int32).reshape(B, B), _probabilities(z, emap, low))
    ours = dirs["ours"]
    args = (B, B, low, len_e, mp, len_r, g, q)
    for d in (dirs["ref"], ours):
        r = run(EXE, "verify", d, "rs:l0.softmax.h00", *args)
        assert r.returncode == 0 and "ACCEPT" in r.stdout, r.stdout + r.stderr
    assert run(EXE, "verify", ours, "rs:l0.softmax.h01", *args).returncode == 1
    other = emap.copy()
    other[3] += 1
    (tmp_path / "map2").write_bytes(other.tobytes())
    r = run(EXE, "verify", ours, "rs:l0.softmax.h00", B, B, low, len_e, tmp_path / "map2", len_r, g, q)
    assert r.returncode == 1 and "exp lookup terminal identity" in r.stdout, r.stdout
    if B != 8:                                                      # the changed-file loop on the 8-row shapes only
        return
    for name, off, what in (("lookup_E.bin", 7, "exp lookup round 0"), ("lookup_L.bin", 4, "limb lookup round 0"), ("lookup_L.bin", -9, "limb lookup terminal identity"),
                            ("hp_rs.bin", 36, "row-sum round 0"), ("hp_rs.bin", -32, "row-sum U_f2 != 1"), ("hp_v1.bin", -64, "V1 terminal identity"),
                            ("hp_v2.bin", -32, "V2 terminal identity"), ("com_P.bin", 30, "exp lookup round 0"),
                            ("lvals.bin", 0, "IPA opening of L00 vs com_L"), ("lvals.bin", 4 * 32, "IPA opening of S_id vs com_S"),
                            ("ipa_comb.bin", -9, "IPA opening of S_f vs com_z + r*com_E"), ("ipa_S_v2.bin", -9, "IPA opening of V2 U_f2 vs com_S"),
                            ("ipa_L11.bin", -9, "IPA opening of L11 vs com_L")):
        raw = bytearray((ours / name).read_bytes())
        raw[off] ^= 1
        (ours / name).write_bytes(bytes(raw))
        r = run(EXE, "verify", ours, "rs:l0.softmax.h00", *args)
        assert r.returncode == 1 and "REJECT" in r.stdout and what in r.stdout, (name, r.stdout)
        raw[off] ^= 1
        (ours / name).write_bytes(bytes(raw))


@pytest.mark.gpu
def test_claim_mode_files_equal_the_reference_and_the_batch_accepts(tmp_path):
    if not os.path.exists(REF_EXE):
        pytest.skip("oracle/_ref/zkob_softmax_ref not built")
    B, low, len_e, len_r, top = CASES[2]
    _, _, (zp, mp, g, q) = _inputs(tmp_path, B, low, len_e, len_r, 77, top)
    kept = {}
    for tag, exe in (("ref", REF_EXE), ("ours", EXE)):
        ob, acc, vacc = tmp_path / "ob", tmp_path / "acc", tmp_path / "vacc"
        for d in (ob, acc, vacc):
            d.mkdir()
        r = run(exe, "prove", ob, "rs:l0.softmax.h00", zp, B, B, low, len_e, mp, len_r, g, q, "--claims", acc, "l0.softmax.h00")
        assert r.returncode == 0 and "16 claims emitted" in r.stdout, r.stdout + r.stderr
        # this verifier on both provers' output: the reference program's own claim-mode verifier compares com_comb.bin through its
        # point negation, which this toolchain builds as the identity, and so refuses its own prover's file
        r = run(EXE, "verify", ob, "rs:l0.softmax.h00", B, B, low, len_e, mp, len_r, g, q, "--claims", vacc, "l0.softmax.h00")
        assert r.returncode == 0 and "ACCEPT-conditional (16 claims" in r.stdout, r.stdout + r.stderr
        kept[tag] = {p.relative_to(tmp_path).as_posix(): p.read_bytes() for d in (ob, acc, vacc) for p in sorted(d.iterdir())}
        if tag == "ours":
            assert run(BATCH, "prove", acc, "rs", q, "%d=%s" % (B, g)).returncode == 0
            r = run(BATCH, "verify", acc, vacc, "rs", q, "%d=%s" % (B, g))
            assert r.returncode == 0 and "opening_batch ACCEPT (16 claims, 9 tensors, 1 domains)" in r.stdout, r.stdout + r.stderr
            # a changed combination file is refused before any claim is written
            raw = bytearray((ob / "com_comb.bin").read_bytes())
            raw[30] ^= 1
            (ob / "com_comb.bin").write_bytes(bytes(raw))
            r = run(EXE, "verify", ob, "rs:l0.softmax.h00", B, B, low, len_e, mp, len_r, g, q, "--claims", tmp_path, "x")
            assert r.returncode == 1 and "com_comb.bin != com_z + r*com_E" in r.stdout, r.stdout
        for d in (ob, acc, vacc):
            for p in d.iterdir():
                p.unlink()
            d.rmdir()
    assert kept["ours"].keys() == kept["ref"].keys()
    for name in kept["ref"]:
        assert kept["ours"][name] == kept["ref"][name], name
    assert kept["ours"]["acc/claims.bin"] == kept["ours"]["vacc/claims.bin"]
