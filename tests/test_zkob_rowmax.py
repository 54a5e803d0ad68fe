"""The row-maximum driver of the first proof stack (zk-hillclimb_b200/zkob_rowmax, the reference's zkob_rowmax command line): every
file byte for byte against the reference's own program (oracle/_ref/zkob_rowmax_ref) in the causal and the padded-vocabulary mode
(one and two limb planes, with and without target columns), in the plain and the claim mode; the mx chain file against numpy; this
verifier on both programs' output, on changed files and on other target columns; the claims through the batch."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

import fr_oracle as fo

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "zk-hillclimb_b200")
EXE = os.path.join(PKG, "zkob_rowmax")
BATCH = os.path.join(PKG, "zkob_batchopen")
REF_EXE = os.path.join(ROOT, "oracle", "_ref", "zkob_rowmax_ref")


def run(exe, *args, timeout=900):
    return subprocess.run([exe] + [str(a) for a in args], capture_output=True, text=True, timeout=timeout)


def test_usage_and_layout_rules(tmp_path):
    assert os.path.exists(EXE), "build() makes the driver"
    assert run(EXE).returncode == 2 and run(EXE, "prove", "x").returncode == 2
    t = tmp_path
    (t / "z").write_bytes(np.zeros(8 * 8, dtype=np.int32).tobytes())
    (t / "zbig").write_bytes(np.full(8 * 8, 100, dtype=np.int32).tobytes())
    (t / "g").write_bytes(bytes(8 * 144))
    (t / "q").write_bytes(bytes(144))
    (t / "ts").write_bytes(np.zeros(8, dtype=np.int32).tobytes())
    r = run(EXE, "prove", t, "s", t / "z", 8, 8, "causal", 3, 32, 1, t / "g", t / "g", t / "q")
    assert r.returncode == 3 and "causal requires V == 0" in r.stderr
    r = run(EXE, "prove", t, "s", t / "z", 8, 8, "rows", 0, 32, 1, t / "g", t / "g", t / "q")
    assert r.returncode == 3 and "MODE must be" in r.stderr
    r = run(EXE, "prove", t, "s", t / "z", 8, 8, "causal", 0, 32, 3, t / "g", t / "g", t / "q")
    assert r.returncode == 3 and "NPL must be 1 or 2" in r.stderr
    r = run(EXE, "prove", t, "s", t / "z", 8, 8, "causal", 0, 32, 1, t / "g", t / "g", t / "q", "-", t / "ts")
    assert r.returncode == 3 and "t* supplied in causal mode" in r.stderr
    r = run(EXE, "verify", t, "s", 8, 8, "vpad", 9, 32, 1, t / "g", t / "g", t / "q")
    assert r.returncode == 1 and "bad layout params" in r.stdout
    r = run(EXE, "verify", t, "s", 8, 8, "vpad", 5, 32, 1, t / "g", t / "g", t / "q", t / "zbig")        # a file of 64 values as t*: only B are read
    assert r.returncode == 1 and "t* token out of [0, V)" in r.stdout


def _inputs(tmp_path, B, NCOL, mode, V, LEN_R, NPL, tstar, seed):
    if not fo.ReferenceFr.available():
        pytest.skip("oracle/_ref/libfrref.so not built")
    lib = fo.ReferenceFr().lib
    if not lib.refA_gpu_available():
        pytest.skip("no GPU")
    for name, k in (("g", NCOL), ("gmx", B), ("q", 1)):
        buf = (C.c_uint8 * (k * 144))()
        assert lib.refA_commit_random(C.c_uint32(k), buf) == 0
        (tmp_path / name).write_bytes(bytes(buf))
    if NCOL == B:                                                   # one shared domain: one generator set
        (tmp_path / "gmx").write_bytes((tmp_path / "g").read_bytes())
    g = np.random.default_rng(seed)
    cols = V if mode == "vpad" else NCOL
    span = LEN_R ** NPL                                             # every allowed difference mx - z below LEN_R^NPL
    z = g.integers(-(span // 2) + 1, span // 2, (B, cols), dtype=np.int32)
    (tmp_path / "z").write_bytes(z.tobytes())
    extra = []
    if tstar:
        ts = np.array([int(np.argmax(z[i])) for i in range(B)], dtype=np.int32)      # the lowest attaining column
        (tmp_path / "ts").write_bytes(ts.tobytes())
        extra = [tmp_path / "ts"]
    return z, extra, [tmp_path / k for k in ("z", "g", "gmx", "q")]


def _row_max(z, mode):
    if mode == "vpad":
        return z.max(axis=1).astype(np.int32)
    return np.array([z[i, :i + 1].max() for i in range(z.shape[0])], dtype=np.int32)


CASES = [(8, 8, "causal", 0, 32, 1, False), (8, 16, "vpad", 11, 32, 2, True), (16, 16, "causal", 0, 64, 1, False), (4, 8, "vpad", 8, 32, 2, False),
         (64, 64, "causal", 0, 1024, 2, False)]


@pytest.mark.gpu
@pytest.mark.parametrize("B,NCOL,mode,V,LEN_R,NPL,tstar", CASES)
def test_files_equal_the_reference_programs(tmp_path, B, NCOL, mode, V, LEN_R, NPL, tstar):
    if not os.path.exists(REF_EXE):
        pytest.skip("oracle/_ref/zkob_rowmax_ref not built")
    z, extra, (zp, g, gmx, q) = _inputs(tmp_path, B, NCOL, mode, V, LEN_R, NPL, tstar, 13 * B + NCOL + NPL)
    dirs = {}
    for tag, exe in (("ours", EXE), ("ref", REF_EXE)):
        d = tmp_path / tag
        d.mkdir()
        r = run(exe, "prove", d, "rs:l0.rowmax.h00", zp, B, NCOL, mode, V, LEN_R, NPL, g, gmx, q, tmp_path / (tag + "_mx.bin"), *extra)
        assert r.returncode == 0, r.stdout + r.stderr
        dirs[tag] = d
    names = sorted(p.name for p in dirs["ref"].iterdir())
    assert names == sorted(p.name for p in dirs["ours"].iterdir()) and len(names) == 1 + 6 + 1 + 6 + 1 + 11 + NPL + 2 * tstar
    for n in names:
        assert (dirs["ours"] / n).read_bytes() == (dirs["ref"] / n).read_bytes(), n
    chain = (tmp_path / "ours_mx.bin").read_bytes()
    assert chain == (tmp_path / "ref_mx.bin").read_bytes()
    assert np.array_equal(np.frombuffer(chain, dtype=np.int32), _row_max(z, mode))
    ours = dirs["ours"]
    args = (B, NCOL, mode, V, LEN_R, NPL, g, gmx, q, *extra)
    for d in (dirs["ref"], ours):
        r = run(EXE, "verify", d, "rs:l0.rowmax.h00", *args)
        assert r.returncode == 0 and "ACCEPT" in r.stdout, r.stdout + r.stderr
    assert run(EXE, "verify", ours, "rs:l0.rowmax.h01", *args).returncode == 1
    if tstar:                                                       # other target columns: another transcript and other weights
        ts = np.frombuffer((tmp_path / "ts").read_bytes(), dtype=np.int32).copy()
        ts[2] = (ts[2] + 1) % V
        (tmp_path / "ts2").write_bytes(ts.tobytes())
        r = run(EXE, "verify", ours, "rs:l0.rowmax.h00", B, NCOL, mode, V, LEN_R, NPL, g, gmx, q, tmp_path / "ts2")
        assert r.returncode == 1 and "REJECT" in r.stdout
    if B != 8:                                                      # the changed-file loop on the 8-row shapes only
        return
    loci = [("lookup_L.bin", 7, "limb lookup round 0"), ("hp_bin.bin", 3, "BIN claim_H != protocol constant 0"), ("hp_sum.bin", 3, "SUM claim_H != protocol constant 1"),
            ("hp_bin.bin", -32, "BIN U_f2 != S_f2 - 1"), ("hp_sum.bin", -64, "SUM terminal identity"), ("hp_mask.bin", -32, "MASK U_f2 != 1"),
            ("hp_att.bin", -64, "ATT terminal identity"), ("hp_c1.bin", 36, "c1 round 0"), ("hp_c2.bin", -64, "c2 terminal identity"),
            ("lvals.bin", 3, "IPA opening of L plane 0 vs com_L"), ("ipa_mx_att.bin", -9, "IPA opening of ev_mx vs com_mx"),
            ("ipa_mx_c2.bin", -9, "IPA opening of c2 terminal vs com_mx"), ("ipa_S_mask.bin", -9, "IPA opening of S (MASK) vs com_S")]
    if tstar:
        loci += [("hp_tbind.bin", 3, "T-BIND claim_H != protocol constant 1"), ("ipa_S_tbind.bin", -9, "IPA opening of S (T-BIND) vs com_S")]
    for name, off, what in loci:
        raw = bytearray((ours / name).read_bytes())
        raw[off] ^= 1
        (ours / name).write_bytes(bytes(raw))
        r = run(EXE, "verify", ours, "rs:l0.rowmax.h00", *args)
        assert r.returncode == 1 and "REJECT" in r.stdout and what in r.stdout, (name, r.stdout)
        raw[off] ^= 1
        (ours / name).write_bytes(bytes(raw))


@pytest.mark.gpu
@pytest.mark.parametrize("case,claims,tensors,domains", [(0, 12, 6, 1), (1, 14, 6, 2)])
def test_claim_mode_files_equal_the_reference_and_the_batch_accepts(tmp_path, case, claims, tensors, domains):
    if not os.path.exists(REF_EXE):
        pytest.skip("oracle/_ref/zkob_rowmax_ref not built")
    B, NCOL, mode, V, LEN_R, NPL, tstar = CASES[case]
    _, extra, (zp, g, gmx, q) = _inputs(tmp_path, B, NCOL, mode, V, LEN_R, NPL, tstar, 77)
    kept = {}
    for tag, exe in (("ref", REF_EXE), ("ours", EXE)):
        ob, acc, vacc = tmp_path / "ob", tmp_path / "acc", tmp_path / "vacc"
        for d in (ob, acc, vacc):
            d.mkdir()
        r = run(exe, "prove", ob, "rs:l0.rowmax.h00", zp, B, NCOL, mode, V, LEN_R, NPL, g, gmx, q, "-", *extra, "--claims", acc, "l0.rowmax.h00")
        assert r.returncode == 0 and "claim mode" in r.stdout, r.stdout + r.stderr
        r = run(EXE, "verify", ob, "rs:l0.rowmax.h00", B, NCOL, mode, V, LEN_R, NPL, g, gmx, q, *extra, "--claims", vacc, "l0.rowmax.h00")
        assert r.returncode == 0 and "ACCEPT-conditional" in r.stdout, r.stdout + r.stderr
        kept[tag] = {p.relative_to(tmp_path).as_posix(): p.read_bytes() for d in (ob, acc, vacc) for p in sorted(d.iterdir())}
        if tag == "ours":
            gens = ["%d=%s" % (NCOL, g)] + (["%d=%s" % (B, gmx)] if B != NCOL else [])
            assert run(BATCH, "prove", acc, "rs", q, *gens).returncode == 0
            r = run(BATCH, "verify", acc, vacc, "rs", q, *gens)
            assert r.returncode == 0 and "opening_batch ACCEPT (%d claims, %d tensors, %d domains)" % (claims, tensors, domains) in r.stdout, r.stdout + r.stderr
        for d in (ob, acc, vacc):
            for p in d.iterdir():
                p.unlink()
            d.rmdir()
    assert kept["ours"].keys() == kept["ref"].keys()
    for name in kept["ref"]:
        assert kept["ours"][name] == kept["ref"][name], name
    assert kept["ours"]["acc/claims.bin"] == kept["ours"]["vacc/claims.bin"]
