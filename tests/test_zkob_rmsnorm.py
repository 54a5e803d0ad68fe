"""The RMS-norm driver of the first proof stack (zk-hillclimb_b200/zkob_rmsnorm, the reference's zkob_rmsnorm command line): every
file byte for byte against the reference's own program (oracle/_ref/zkob_rmsnorm_ref) in the plain and the claim mode, the W and Y
chain files against a numpy statement, this verifier on both programs' output and on changed files, an advice value two away from
the exact one refused by the prover, the seventeen claims (two domains) through the batch."""
import ctypes as C
import math
import os
import subprocess

import numpy as np
import pytest

import fr_oracle as fo

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "zk-hillclimb_b200")
EXE = os.path.join(PKG, "zkob_rmsnorm")
BATCH = os.path.join(PKG, "zkob_batchopen")
REF_EXE = os.path.join(ROOT, "oracle", "_ref", "zkob_rmsnorm_ref")
C_EPS = round(1e-5 * (1 << 32))                                     # per column; multiplied by C below


def run(exe, *args, timeout=900):
    return subprocess.run([exe] + [str(a) for a in args], capture_output=True, text=True, timeout=timeout)


def _advice(X, c_eps):
    """R with (R-1)^2 M <= 2^64 C <= (R+1)^2 M for every row, M = sum X^2 + c_eps (Python integers)."""
    B, Cc = X.shape
    out = []
    for s in range(B):
        M = sum(int(v) * int(v) for v in X[s]) + c_eps
        r = math.isqrt((Cc << 64) // M)
        while (r + 1) * (r + 1) * M < (Cc << 64):
            r += 1
        assert (r - 1) * (r - 1) * M <= (Cc << 64) <= (r + 1) * (r + 1) * M
        out.append(r)
    return np.array(out, dtype=np.int32)


def _write_inputs(tmp_path, B, Cc, seed):
    g = np.random.default_rng(seed)
    X = g.integers(-(1 << 15), 1 << 15, (B, Cc), dtype=np.int32)
    gain = g.integers(1 << 15, 1 << 17, Cc, dtype=np.int32)
    c_eps = C_EPS * Cc
    R = _advice(X, c_eps)
    for name, a in (("X", X), ("R", R), ("g", gain)):
        (tmp_path / name).write_bytes(a.tobytes())
    return X, R, gain, c_eps


def test_usage_layout_rules_and_the_bracket(tmp_path):
    assert os.path.exists(EXE), "build() makes the driver"
    assert run(EXE).returncode == 2 and run(EXE, "prove", "x").returncode == 2
    t = tmp_path
    X, R, gain, c_eps = _write_inputs(t, 8, 5, 1)
    (t / "gC").write_bytes(bytes(8 * 144))
    (t / "gB").write_bytes(bytes(8 * 144))
    (t / "gB4").write_bytes(bytes(4 * 144))
    (t / "q").write_bytes(bytes(144))
    r = run(EXE, "prove", t, "s", t / "X", t / "R", t / "g", 8, 5, c_eps, t / "gC", t / "gB4", t / "q")
    assert r.returncode == 3 and "gen_B size" in r.stderr
    r = run(EXE, "prove", t, "s", t / "X", t / "R", t / "g", 8, 5, c_eps, t / "gC", t / "gB", t / "q", "--wpriv", t, t / "b")
    assert r.returncode == 2 and "not built" in r.stderr
    R2 = R.copy()
    R2[3] += 2                                                      # outside the +-1 tolerance: the honest prover stops
    (t / "R2").write_bytes(R2.tobytes())
    r = run(EXE, "prove", t, "s", t / "X", t / "R2", t / "g", 8, 5, c_eps, t / "gC", t / "gB", t / "q")
    assert r.returncode == 3 and "bracket violated" in r.stderr
    r = run(EXE, "verify", t, "s", 6, 5, c_eps, t / "cg", t / "gC", t / "gB", t / "q")
    assert r.returncode == 1 and "bad layout params" in r.stdout


def _inputs(tmp_path, B, Cc, seed):
    if not fo.ReferenceFr.available():
        pytest.skip("oracle/_ref/libfrref.so not built")
    lib = fo.ReferenceFr().lib
    if not lib.refA_gpu_available():
        pytest.skip("no GPU")
    Cp = 1 << (Cc - 1).bit_length()
    for name, k in (("gC", Cp), ("gB", B), ("q", 1)):
        buf = (C.c_uint8 * (k * 144))()
        assert lib.refA_commit_random(C.c_uint32(k), buf) == 0
        (tmp_path / name).write_bytes(bytes(buf))
    if Cp == B:                                                     # one shared domain: one generator set
        (tmp_path / "gB").write_bytes((tmp_path / "gC").read_bytes())
    X, R, gain, c_eps = _write_inputs(tmp_path, B, Cc, seed)
    return X, R, gain, c_eps, [tmp_path / k for k in ("X", "R", "g", "gC", "gB", "q")]


@pytest.mark.gpu
@pytest.mark.parametrize("B,Cc", [(8, 5), (16, 5), (4, 8), (64, 48)])
def test_files_equal_the_reference_programs(tmp_path, B, Cc):
    if not os.path.exists(REF_EXE):
        pytest.skip("oracle/_ref/zkob_rmsnorm_ref not built")
    X, R, gain, c_eps, (Xp, Rp, gp, gC, gB, q) = _inputs(tmp_path, B, Cc, 11 * B + Cc)
    dirs = {}
    for tag, exe in (("ours", EXE), ("ref", REF_EXE)):
        d = tmp_path / tag
        d.mkdir()
        r = run(exe, "prove", d, "rs:l0.norm1", Xp, Rp, gp, B, Cc, c_eps, gC, gB, q, tmp_path / (tag + "_W.bin"), tmp_path / (tag + "_Y.bin"))
        assert r.returncode == 0, r.stdout + r.stderr
        dirs[tag] = d
    names = sorted(p.name for p in dirs["ref"].iterdir())
    assert names == sorted(p.name for p in dirs["ours"].iterdir()) and len(names) == 1 + 12 + 6 + 17
    for n in names:
        assert (dirs["ours"] / n).read_bytes() == (dirs["ref"] / n).read_bytes(), n
    W = R.astype(np.int64)[:, None] * gain.astype(np.int64)[None, :]
    Wr = (W + (1 << 15)) >> 16                                      # remainder in [-2^15, 2^15)
    for name, want in (("W", W), ("Y", Wr * X)):
        chain = (tmp_path / ("ours_%s.bin" % name)).read_bytes()
        assert chain == (tmp_path / ("ref_%s.bin" % name)).read_bytes()
        assert np.array_equal(np.frombuffer(chain, dtype=np.int64).reshape(B, Cc), want), name
    ours = dirs["ours"]
    args = (B, Cc, c_eps, ours / "com_g.bin", gC, gB, q)
    for d in (dirs["ref"], ours):
        r = run(EXE, "verify", d, "rs:l0.norm1", B, Cc, c_eps, d / "com_g.bin", gC, gB, q)
        assert r.returncode == 0 and "ACCEPT" in r.stdout, r.stdout + r.stderr
    assert run(EXE, "verify", ours, "rs:l0.norm2", *args).returncode == 1
    r = run(EXE, "verify", ours, "rs:l0.norm1", B, Cc, c_eps + 1, ours / "com_g.bin", gC, gB, q)
    assert r.returncode == 1 and "dims.bin mismatch" in r.stdout
    if B != 8:                                                      # the changed-file loop on the 8-row shapes only
        return
    for name, off, what in (("com_P1.bin", 30, "affine link P1"), ("com_L.bin", 5 * 144 + 30, "affine link P2"), ("lookup.bin", 7, "limb lookup round 0"),
                            ("hpss.bin", 36, "SS round 0"), ("hpss.bin", -32, "SS S_f2 != U_f2"), ("qp1.bin", 36, "q1 round 0"), ("qp2.bin", -96, "q2 A_f != B_f"),
                            ("qp2.bin", -32, "q2 terminal identity"), ("outer.bin", 32, "outer product check"), ("hp.bin", -64, "hadamard terminal identity"),
                            ("ipa_R_q1.bin", -9, "IPA opening of R@pt1 (expect q1.A_f + 1) vs com_R"), ("ipa_g.bin", -9, "IPA opening of val_g vs registered com_g"),
                            ("ipa_X_h.bin", -9, "IPA opening of X (hadamard) vs com_X")):
        raw = bytearray((ours / name).read_bytes())
        raw[off] ^= 1
        (ours / name).write_bytes(bytes(raw))
        r = run(EXE, "verify", ours, "rs:l0.norm1", *args)
        assert r.returncode == 1 and "REJECT" in r.stdout and what in r.stdout, (name, r.stdout)
        raw[off] ^= 1
        (ours / name).write_bytes(bytes(raw))


@pytest.mark.gpu
@pytest.mark.parametrize("B,Cc,domains", [(8, 5, 1), (16, 5, 2)])
def test_claim_mode_files_equal_the_reference_and_the_batch_accepts(tmp_path, B, Cc, domains):
    if not os.path.exists(REF_EXE):
        pytest.skip("oracle/_ref/zkob_rmsnorm_ref not built")
    _, _, _, c_eps, (Xp, Rp, gp, gC, gB, q) = _inputs(tmp_path, B, Cc, 77)
    reg = tmp_path / "registered_com_g.bin"                         # the registered commitment of g: the prover's own row commitment
    (tmp_path / "plain").mkdir()
    assert run(EXE, "prove", tmp_path / "plain", "x", Xp, Rp, gp, B, Cc, c_eps, gC, gB, q).returncode == 0
    reg.write_bytes((tmp_path / "plain" / "com_g.bin").read_bytes())
    kept = {}
    for tag, exe in (("ref", REF_EXE), ("ours", EXE)):
        ob, acc, vacc = tmp_path / "ob", tmp_path / "acc", tmp_path / "vacc"
        for d in (ob, acc, vacc):
            d.mkdir()
        r = run(exe, "prove", ob, "rs:l0.norm1", Xp, Rp, gp, B, Cc, c_eps, gC, gB, q, "--claims", acc, "l0.norm1", reg)
        assert r.returncode == 0 and "17 claims" in r.stdout, r.stdout + r.stderr
        # this verifier on both provers' output: the reference program's own verifier compares its affine limb links through its point
        # negation, which this toolchain builds as the identity, and so refuses its own prover's commitments
        r = run(EXE, "verify", ob, "rs:l0.norm1", B, Cc, c_eps, reg, gC, gB, q, "--claims", vacc, "l0.norm1")
        assert r.returncode == 0 and "ACCEPT-conditional (17 claims" in r.stdout, r.stdout + r.stderr
        kept[tag] = {p.relative_to(tmp_path).as_posix(): p.read_bytes() for d in (ob, acc, vacc) for p in sorted(d.iterdir())}
        if tag == "ours":
            Cp = 1 << (Cc - 1).bit_length()
            gens = ["%d=%s" % (B, gB)] + (["%d=%s" % (Cp, gC)] if Cp != B else [])
            assert run(BATCH, "prove", acc, "rs", q, *gens).returncode == 0
            r = run(BATCH, "verify", acc, vacc, "rs", q, *gens)
            assert r.returncode == 0 and "opening_batch ACCEPT (17 claims, 12 tensors, %d domains)" % domains in r.stdout, r.stdout + r.stderr
        for d in (ob, acc, vacc):
            for p in d.iterdir():
                p.unlink()
            d.rmdir()
    assert kept["ours"].keys() == kept["ref"].keys()
    for name in kept["ref"]:
        assert kept["ours"][name] == kept["ref"][name], name
    assert kept["ours"]["acc/claims.bin"] == kept["ours"]["vacc/claims.bin"]
