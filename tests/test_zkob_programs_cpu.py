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
