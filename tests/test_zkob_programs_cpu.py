"""What every driver program of the first proof stack must do before it touches a GPU: print its usage with exit code 2, refuse the
weight-privacy flags with exit code 2, and keep the serve protocol (ZKW-READY, one "ZKW-RC <rc>" per request line, a failed request
does not end the loop).  No GPU."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "zk-hillclimb_b200")
PROGRAMS = ["zkob_fc", "zkob_rescale", "zkob_rmsnorm", "zkob_rope", "zkob_headslice", "zkob_rowmax", "zkob_softmax", "zkob_softmax8", "zkob_headmerge",
            "zkob_glu", "zkob_skip", "zkob_batchopen"]


@pytest.mark.parametrize("prog", PROGRAMS)
def test_usage_flags_and_serve_protocol(prog, tmp_path):
    exe = os.path.join(PKG, prog)
    assert os.path.exists(exe), "build() makes the program"
    r = subprocess.run([exe], capture_output=True, text=True, timeout=60)
    assert r.returncode == 2 and "usage" in r.stderr.lower()
    r = subprocess.run([exe, "frobnicate", "x"], capture_output=True, text=True, timeout=60)
    assert r.returncode == 2
    if prog not in ("zkob_skip", "zkob_batchopen"):
        for flag in ("--wpriv", "--apriv", "--hiding"):
            r = subprocess.run([exe, "prove", tmp_path, "s", flag, "x"], capture_output=True, text=True, timeout=60)
            assert r.returncode == 2 and "not built" in r.stderr, (flag, r.stderr)
    r = subprocess.run([exe, "serve"], input="frobnicate x\n\nverify %s/none s\nfrobnicate y\n" % tmp_path, capture_output=True, text=True, timeout=60)
    assert r.returncode == 0
    lines = [l for l in r.stdout.splitlines() if l.startswith("ZKW-")]
    assert lines[0] == "ZKW-READY" and len(lines) == 4 and lines[1] == "ZKW-RC 2" and lines[3] == "ZKW-RC 2"
    assert lines[2] in ("ZKW-RC 2", "ZKW-RC 3")                      # a malformed or unreadable request fails alone


def _claims(items):
    """claims.bin: "ZKCL", version 1, count; per claim id and comref (length-prefixed), domain, n_rows, the point (count-prefixed
    32-byte scalars), tag 0, the evaluation."""
    out = b"ZKCL" + (1).to_bytes(4, "little") + len(items).to_bytes(4, "little")
    for cid, comref, domain, n_rows, point, ev in items:
        out += len(cid).to_bytes(4, "little") + cid.encode() + len(str(comref)).to_bytes(4, "little") + str(comref).encode()
        out += domain.to_bytes(4, "little") + n_rows.to_bytes(4, "little") + len(point).to_bytes(4, "little")
        out += b"".join(p.to_bytes(32, "little") for p in point) + b"\x00" + ev.to_bytes(32, "little")
    return out


def test_batch_verifier_refuses_malformed_accumulators_before_any_device_work(tmp_path):
    """The reference's refusal loci of the batch verifier that need no group arithmetic (zkllm-src/zkob_claims.cuh:1063-1150)."""
    bo = os.path.join(PKG, "zkob_batchopen")
    p, v = tmp_path / "p", tmp_path / "v"
    p.mkdir()
    v.mkdir()
    com, gen, q = tmp_path / "com.bin", tmp_path / "g4", tmp_path / "q"
    q.write_bytes(bytes(144))

    def verdict(items, prover_items=None, gens=("4=%s" % gen,)):
        (v / "claims.bin").write_bytes(_claims(items))
        (p / "claims.bin").write_bytes(_claims(items if prover_items is None else prover_items))
        r = subprocess.run([bo, "verify", p, v, "seed", q, *gens], capture_output=True, text=True, timeout=60)
        assert r.returncode == 1, r.stdout + r.stderr
        return r.stdout

    good = [("ob:T", com, 4, 2, [1, 2, 3], 5)]                       # 2 rows of 4 scalars: 3 variables
    assert "REJECT[opening_batch.claims_match]" in verdict(good, [("ob:T", com, 4, 2, [1, 2, 3], 6)])
    assert "REJECT[opening_batch.shape]" in verdict([("ob:T", com, 4, 4, [1, 2, 3], 5)])             # n_rows != 2^(variables - log2 domain)
    out = verdict([("ob:T", com, 4, 2, [1, 2, 3], 5), ("ob:T2", com, 4, 1, [1, 2], 5)])             # one commitment file, two shapes
    assert "REJECT[opening_batch.shape]" in out
    out = verdict(good)
    assert "REJECT[opening_batch.shape]" in out and "commitment file missing" in out
    com.write_bytes(bytes(3 * 144))
    out = verdict(good)
    assert "REJECT[opening_batch.shape]" in out and "commitment row count 3 != n_rows 2" in out
    com.write_bytes(bytes(2 * 144))
    out = verdict(good, gens=("8=%s" % gen,))
    assert "REJECT[opening_batch.shape]" in out and "no generator file mapped for domain 4" in out
    gen.write_bytes(bytes(3 * 144))
    out = verdict(good)
    assert "REJECT[opening_batch.shape]" in out and "generator file size != domain 4" in out
    gen.write_bytes(bytes(4 * 144))
    assert "REJECT[opening_batch.xcheck]" in verdict(good)           # no batch_sumcheck.bin
    (p / "batch_sumcheck.bin").write_bytes(b"ZKBX" + bytes(12))
    out = verdict(good)
    assert "REJECT[opening_batch.xcheck]" in out and "header" in out
    (v / "claims.bin").write_bytes(_claims(good)[:-1] + b"\x01" + b"\x00")       # trailing byte
    r = subprocess.run([bo, "verify", p, v, "seed", q, "4=%s" % gen], capture_output=True, text=True, timeout=60)
    assert r.returncode not in (0, 1) and "trailing" in r.stderr


def _batch_sumcheck_oracle(run_seed, items, wits, comfiles):
    """The sumcheck half of the batch opening in Python integers (zkllm-src/zkob_claims.cuh:832-960: the first absorbs, the powers of
    rho, M_j = sum_i rho^i eq(point_i), the rounds from the top variable down with the smaller tensors carried by (1 - x)^2 factors,
    the terminal values): the round evaluations and the terminals a prover writes to batch_sumcheck.bin and batch_vfin.bin."""
    import hashlib
    import sys
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import fr_oracle as fo
    P = fo.P
    tensors, key = [], {}
    for i, (cid, comref, domain, n_rows, point, ev) in enumerate(items):
        k = str(comref)
        if k not in key:
            key[k] = len(tensors)
            tensors.append({"comref": k, "vars": len(point), "idx": []})
        tensors[key[k]]["idx"].append(i)
    tr = fo.Transcript(run_seed + ":opening_batch")
    tr.absorb("n_claims", len(items).to_bytes(4, "little"))
    for it in items:
        tr.absorb("claim", _claims([it])[12:])                       # the claim's record without the file header
    for t in tensors:
        tr.absorb("comref", len(t["comref"]).to_bytes(4, "little") + t["comref"].encode() + hashlib.sha256(comfiles[t["comref"]]).digest())
    rho = tr.challenge_fr()
    rp = [pow(rho, i, P) for i in range(len(items))]
    m_max = max(t["vars"] for t in tensors)
    M, Pw, S, c2 = [], [], [], []
    for t in tensors:
        n = 1 << t["vars"]
        m = [0] * n
        for i in t["idx"]:
            e = fo.eq_build(items[i][4])
            m = [(a + rp[i] * b) % P for a, b in zip(m, e)]
        M.append(m)
        Pw.append(list(wits[t["comref"]]))
        S.append(sum(a * b for a, b in zip(m, Pw[-1])) % P)
        c2.append(1)
    cur = sum(rp[i] * items[i][5] for i in range(len(items))) % P
    evs, r = [], [0] * m_max
    for rnd in range(m_max):
        v = m_max - 1 - rnd
        p = [0, 0, 0]
        for j, t in enumerate(tensors):
            if t["vars"] <= v:
                p[0] = (p[0] + c2[j] * S[j]) % P
                p[2] = (p[2] + c2[j] * S[j]) % P
            else:
                h = len(M[j]) // 2
                for T in range(3):
                    p[T] = (p[T] + c2[j] * sum((M[j][i] + T * (M[j][i + h] - M[j][i])) * (Pw[j][i] + T * (Pw[j][i + h] - Pw[j][i])) for i in range(h))) % P
        assert cur == (p[0] + p[1]) % P
        for lab, val in zip(("bp0", "bp1", "bp2"), p):
            tr.absorb_fr(lab, val)
        x = tr.challenge_fr()
        r[v] = x
        evs += p
        cur = fo.lagrange(p, x)
        for j, t in enumerate(tensors):
            if t["vars"] <= v:
                c2[j] = c2[j] * (1 - x) * (1 - x) % P
            else:
                h = len(M[j]) // 2
                M[j] = [(M[j][i] + x * (M[j][i + h] - M[j][i])) % P for i in range(h)]
                Pw[j] = [(Pw[j][i] + x * (Pw[j][i + h] - Pw[j][i])) % P for i in range(h)]
    return evs, [pw[0] for pw in Pw], m_max, len(tensors)


def test_batch_verifier_replays_a_python_provers_sumcheck(tmp_path):
    """Two tensors of different sizes, three claims (two on one tensor): the round evaluations and terminals of a Python-integer
    prover pass every host-side check of the batch verifier (which then stops only at the group arithmetic, where it needs the GPU or
    the missing argument file); changed rounds, terminals and evaluations are refused at the reference's loci."""
    import random
    import sys
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import fr_oracle as fo
    P = fo.P
    rng = random.Random(21)
    bo = os.path.join(PKG, "zkob_batchopen")
    p, v = tmp_path / "p", tmp_path / "v"
    p.mkdir()
    v.mkdir()
    gen, q = tmp_path / "g4", tmp_path / "q"
    gen.write_bytes(bytes(4 * 144))
    q.write_bytes(bytes(144))
    comA, comB = tmp_path / "comA.bin", tmp_path / "comB.bin"
    comA.write_bytes(bytes(range(144)) * 4)                          # 4 rows of 4: 4 variables
    comB.write_bytes(bytes(range(1, 145)))                           # 1 row of 4: 2 variables
    wA, wB = [rng.randrange(P) for _ in range(16)], [rng.randrange(P) for _ in range(4)]
    pts = [[rng.randrange(P) for _ in range(4)], [rng.randrange(P) for _ in range(2)], [rng.randrange(P) for _ in range(4)]]
    items = [("a:T", comA, 4, 4, pts[0], fo.mle_eval(wA, pts[0])), ("b:S", comB, 4, 1, pts[1], fo.mle_eval(wB, pts[1])),
             ("c:T2", comA, 4, 4, pts[2], fo.mle_eval(wA, pts[2]))]
    wits = {str(comA): wA, str(comB): wB}
    comfiles = {str(comA): comA.read_bytes(), str(comB): comB.read_bytes()}
    evs, vfin, m_max, nT = _batch_sumcheck_oracle("seed", items, wits, comfiles)

    def verdict(evs_, vfin_, items_=items):
        (v / "claims.bin").write_bytes(_claims(items_))
        (p / "claims.bin").write_bytes(_claims(items_))
        (p / "batch_sumcheck.bin").write_bytes(b"ZKBS" + len(items_).to_bytes(4, "little") + m_max.to_bytes(4, "little") + len(evs_).to_bytes(4, "little")
                                               + b"".join(e.to_bytes(32, "little") for e in evs_))
        (p / "batch_vfin.bin").write_bytes(b"ZKBV" + nT.to_bytes(4, "little") + b"".join(e.to_bytes(32, "little") for e in vfin_))
        return subprocess.run([bo, "verify", p, v, "seed", q, "4=%s" % gen], capture_output=True, text=True, timeout=120)

    r = verdict(evs, vfin)
    host_rejects = ("claims_match", "shape", "xcheck", "round", "vfin_count", "terminal")
    assert not any("REJECT[opening_batch." + k in r.stdout for k in host_rejects), r.stdout
    assert r.returncode != 0                                         # no argument file (and on this machine no GPU): never an ACCEPT
    assert "no CUDA device" in r.stderr or "REJECT[opening_batch.group_missing]" in r.stdout, r.stdout + r.stderr
    bad = list(evs)
    bad[4] = (bad[4] + 1) % P
    assert "REJECT[opening_batch.round1]" in verdict(bad, vfin).stdout
    bad = list(evs)
    bad[2] = (bad[2] + 1) % P                                        # p(2) of round 0 moves the next running claim
    assert "REJECT[opening_batch.round1]" in verdict(bad, vfin).stdout
    assert "REJECT[opening_batch.terminal]" in verdict(evs, [vfin[0], (vfin[1] + 1) % P]).stdout
    wrong = [items[0], (items[1][0], items[1][1], 4, 1, pts[1], (items[1][5] + 1) % P), items[2]]
    assert "REJECT[opening_batch.round0]" in verdict(evs, vfin, wrong).stdout


def test_honest_prover_guards_stop_before_the_device(tmp_path):
    """The range and layout guards of the provers (the reference's honest-prover throws) fire on the host: exit code 3 with the
    reference's message, no device needed."""
    import numpy as np
    t = tmp_path

    def f(name, a, dtype=np.int32):
        (t / name).write_bytes(np.asarray(a).astype(dtype).tobytes())
        return t / name

    for name, k in (("g16", 16), ("g8", 8), ("q", 1)):
        (t / name).write_bytes(bytes(k * 144))
    g16, g8, q = t / "g16", t / "g8", t / "q"

    def stopped(prog, message, *args):
        r = subprocess.run([os.path.join(PKG, prog), "prove", t, "s"] + [str(a) for a in args], capture_output=True, text=True, timeout=120)
        assert r.returncode == 3 and message in r.stderr, (prog, message, r.returncode, r.stderr[-300:])

    z = np.zeros((8, 8), dtype=np.int32)
    z[5, 2] = -40                                                    # row maximum 0, difference 40
    stopped("zkob_rowmax", "allowed Df >= LEN_R^NPL", f("z", z), 8, 8, "causal", 0, 32, 1, g8, g8, q)
    stopped("zkob_rowmax", "vpad |z| >= 2^25", f("zb", np.full((8, 5), 1 << 25)), 8, 8, "vpad", 5, 32, 1, g8, g8, q)
    emap8 = np.ones(16, dtype=np.int32)
    emap8[-1] = 0
    z2 = np.zeros((8, 8), dtype=np.int32)
    z2[3, 1] = -20                                                   # below LOW8 = -14
    stopped("zkob_softmax8", "allowed diff below LOW8", f("z2", z2), f("mx", np.zeros(8)), 8, 8, -14, 16, f("m8", emap8), 32, g8, q)
    z3 = np.zeros((8, 8), dtype=np.int32)
    z3[0, 0] = 1 << 19
    stopped("zkob_softmax8", "z_ outside the +-2^19 envelope", f("z3", z3), t / "mx", 8, 8, -14, 16, t / "m8", 32, g8, q)
    stopped("zkob_softmax", "bracket residual >= LEN_R^2", f("z0", np.zeros((8, 8))), 8, 8, -8, 16, f("mbig", np.full(16, 1 << 20)), 32, g8, q)
    stopped("zkob_softmax", "S[i] < 1", t / "z0", 8, 8, -8, 16, f("mzero", np.zeros(16)), 32, g8, q)
    big = np.full((8, 16), (1 << 31) - 1, dtype=np.int32)
    stopped("zkob_rope", "|Y64| >= 2^47", f("T", big), 8, 16, 8, f("cos", np.full((8, 8), 1 << 16)), f("sin", np.full((8, 8), 1 << 16)), g16, q)
    stopped("zkob_rope", "NH = C/HD must be >= 2", t / "T", 8, 16, 16, f("cos16", np.zeros((8, 16))), t / "cos16", g16, q)
    G = np.zeros((8, 16), dtype=np.int32)
    G[2, 3] = 64                                                     # the table covers [-64, 64)
    stopped("zkob_glu", "outside the table", f("G", G), f("U", np.ones((8, 16))), 8, 16, -64, 128, f("mg", np.zeros(128)), g16, q)
    stopped("zkob_glu", "mapped(0) == 0", t / "G", t / "U", 8, 16, -64, 128, f("mg1", np.ones(128)), g16, q)
    f("o00.i32.bin", np.zeros((8, 8)))
    f("o01.i32.bin", np.zeros((8, 7)))
    stopped("zkob_headmerge", "file size != expected int32 count", t / "o", 8, 16, 8, "concat", g16, g8, q)
    stopped("zkob_headslice", "HD must divide C", f("Q", np.zeros((8, 12))), t / "Q", t / "Q", 8, 12, 8, g16, g8, q)
    stopped("zkob_rescale", "layout needs C_pad <= N <= D", f("X64", np.zeros((8, 16)), np.int64), 8, 16, 16, g16, q)
    X = np.full((8, 16), 100, dtype=np.int32)
    stopped("zkob_rmsnorm", "bracket violated", f("X", X), f("R", np.full(8, 5)), f("gain", np.ones(16)), 8, 16, 7, g16, g8, q)
    stopped("zkob_rmsnorm", "gen_C size != C_pad", t / "X", t / "R", t / "gain", 8, 16, 7, g8, g8, q)
