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
