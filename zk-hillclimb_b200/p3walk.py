#!/usr/bin/env python
"""Prove and verify walks over the quantised linear obligations of a run, with the zkob_p3fc driver.

The reference's orchestrator walks a plan of obligations, runs one driver invocation per obligation under the driver
protocol (orchestrator/common.py:144-184 run_driver, :231-276 DriverPool; prove_walk.py:162-191; verify_walk.py:280-345)
and its harness checks that the verifier's transcript names every obligation of the manifest
(harness/check_transcript.py:16-36, harness/manifest.py:40-57 linear_obligations).  This module is that walk for the
Goldilocks / Basefold stack: same run layout, same seeds, same verdict rules, new file contents.

Run layout (the reference's, ORCHESTRATOR_DESIGN):
    <run>/public.json            the statement; run_seed = sha256 of its bytes
    <run>/registration/          input activations, weights (prover only) and their registered commitment roots
    <run>/data/                  prover-only chain files (the rescaled outputs that feed the next obligation)
    <run>/proofs/<prefix>/       one directory per linear obligation, made here, filled by the driver

public.json: {"R": 1, "Q": 24, "input": "registration/input.i32", "input_root": "registration/input.root",
              "obligations": [{"prefix": "layer0.mlp.up_proj", "B": 8, "IN": 16, "OUT": 32, "sf": 8,
                               "weight": "registration/w0.i32", "weight_root": "registration/w0.root",
                               "input_from": null}, ...]}
An obligation with "input_from": "<prefix>" takes the rescaled output of that obligation as its X; the verifier then
requires its X commitment to equal the producer's Yr commitment (a chain edge), and the first X to equal the
registered input root.  One linear obligation discharges three manifest ids: <prefix>.matmul, <prefix>.rescaling and
<prefix>.commitment_opening (the weight claim is opened against the REGISTERED root inside the proof's batched openings).

    p3walk.py prove  <run_dir>
    p3walk.py verify <run_dir> <public.json> <transcript-out>       exit 0 = ACCEPT, 1 = REJECT

Standard library only: it can be run as a script beside the driver executable.
"""
import hashlib
import json
import os
import subprocess
import sys
import threading
import time

HERE = os.path.dirname(os.path.abspath(__file__))
DRIVER = os.path.join(HERE, "zkob_p3fc")
DRIVER_TIMEOUT_S = 900
MANIFEST_KINDS = ("matmul", "rescaling", "commitment_opening")


def run_seed_of_bytes(pub_bytes):
    return hashlib.sha256(pub_bytes).hexdigest()


def run_driver(cmd, label, expect_reject_ok=False, retries=1, log=print, timeout=DRIVER_TIMEOUT_S, cwd=None):
    """One driver invocation: (accepted, seconds, output).  Exit 0 = success / ACCEPT; exit 1 = REJECT (returned when
    expect_reject_ok, never retried); any other exit code is a crash, retried `retries` times, then RuntimeError; a
    timeout is a RuntimeError at once."""
    attempt = 0
    while True:
        attempt += 1
        t0 = time.time()
        try:
            r = subprocess.run(cmd, cwd=cwd, capture_output=True, text=True, timeout=timeout)
        except subprocess.TimeoutExpired:
            raise RuntimeError("driver TIMEOUT after %ss: %s" % (timeout, " ".join(cmd)))
        dt = time.time() - t0
        out = (r.stdout or "") + (r.stderr or "")
        if r.returncode == 0:
            log("  [%7.2fs] %s" % (dt, label))
            return True, dt, out
        if r.returncode == 1 and expect_reject_ok:
            log("  [%7.2fs] %s -> REJECT" % (dt, label))
            return False, dt, out
        if attempt <= retries:
            log("  RETRY (%d) %s: %s" % (r.returncode, label, out[-300:]))
            continue
        raise RuntimeError("driver failed rc=%d: %s\n%s" % (r.returncode, " ".join(cmd), out[-2000:]))


class ServePool:
    """One persistent `serve` worker per driver binary: requests go down its stdin one line each, the answer ends with
    "ZKW-RC <rc>".  Same contract as run_driver, no retry (a dead worker is respawned for the next request)."""

    def __init__(self, cwd, log=print):
        self.cwd, self.log, self.procs = cwd, log, {}

    def _get(self, binpath):
        p = self.procs.get(binpath)
        if p is not None and p.poll() is None:
            return p
        p = subprocess.Popen([binpath, "serve"], cwd=self.cwd, stdin=subprocess.PIPE, stdout=subprocess.PIPE,
                             stderr=subprocess.STDOUT, text=True, bufsize=1)
        line = p.stdout.readline()
        if "ZKW-READY" not in line:
            raise RuntimeError("serve worker failed to start: %s (%r)" % (binpath, line))
        self.procs[binpath] = p
        return p

    def run(self, cmd, label, expect_reject_ok=False, timeout=DRIVER_TIMEOUT_S):
        binpath, args = cmd[0], [str(c) for c in cmd[1:]]
        if any(ch.isspace() for a in args for ch in a):
            raise ValueError("whitespace in a driver argument")
        t0 = time.time()
        p = self._get(binpath)
        try:
            p.stdin.write(" ".join(args) + "\n")
            p.stdin.flush()
        except (BrokenPipeError, OSError):
            raise RuntimeError("serve worker died before the request: " + label)
        lines, rc, timed_out = [], None, []
        watchdog = threading.Timer(timeout, lambda: (timed_out.append(1), p.kill()))
        watchdog.start()
        try:
            while True:
                line = p.stdout.readline()
                if line == "":
                    raise RuntimeError("serve request %s: %s" % ("TIMEOUT" if timed_out else "worker died", label))
                if line.startswith("ZKW-RC "):
                    rc = int(line.split()[1])
                    break
                lines.append(line)
        finally:
            watchdog.cancel()
        dt, out = time.time() - t0, "".join(lines)
        if rc == 0:
            self.log("  [%7.2fs] %s" % (dt, label))
            return True, dt, out
        if rc == 1 and expect_reject_ok:
            self.log("  [%7.2fs] %s -> REJECT" % (dt, label))
            return False, dt, out
        raise RuntimeError("serve request failed rc=%s: %s\n%s" % (rc, " ".join([binpath] + args), out[-2000:]))

    def close(self):
        for p in self.procs.values():
            try:
                p.stdin.close()
                p.wait(timeout=10)
            except (OSError, subprocess.TimeoutExpired):
                p.kill()
        self.procs.clear()


def load_public(path):
    with open(path, "rb") as f:
        raw = f.read()
    pub = json.loads(raw)
    prefixes = [o["prefix"] for o in pub["obligations"]]
    if len(set(prefixes)) != len(prefixes):
        raise ValueError("duplicate obligation prefix")
    for o in pub["obligations"]:
        src = o.get("input_from")
        if src is not None and src not in prefixes[:prefixes.index(o["prefix"])]:
            raise ValueError("%s: input_from names no earlier obligation" % o["prefix"])
        if any(ch.isspace() or ch == "/" for ch in o["prefix"]):
            raise ValueError("bad obligation prefix")
    return pub, run_seed_of_bytes(raw)


def manifest_ids(pub):
    return ["%s.%s" % (o["prefix"], k) for o in pub["obligations"] for k in MANIFEST_KINDS]


def _shape(pub, o):
    return [str(o[k]) for k in ("B", "IN", "OUT", "sf")] + [str(pub["R"]), str(pub["Q"])]


def prove_walk(run_dir, driver=DRIVER, run=None, log=print):
    """Every obligation of <run_dir>/public.json in plan order; makes the obligation directories (drivers never do).
    Returns the seconds spent per obligation."""
    pub, run_seed = load_public(os.path.join(run_dir, "public.json"))
    pool = None
    if run is None:
        pool = ServePool(run_dir, log)
        run = pool.run
    os.makedirs(os.path.join(run_dir, "data"), exist_ok=True)
    secs = {}
    try:
        for o in pub["obligations"]:
            ob = os.path.join("proofs", o["prefix"])
            os.makedirs(os.path.join(run_dir, ob), exist_ok=True)
            x = pub["input"] if o.get("input_from") is None else os.path.join("data", o["input_from"] + ".yr.i32")
            cmd = [driver, "prove", ob, "%s:%s" % (run_seed, o["prefix"]), x, o["weight"]] + _shape(pub, o) + \
                  [os.path.join("data", o["prefix"] + ".yr.i32")]
            _, secs[o["prefix"]], _ = run(cmd, "prove " + o["prefix"])
    finally:
        if pool is not None:
            pool.close()
    return secs


def verify_walk(run_dir, public_path=None, transcript_out=None, driver=DRIVER, run=None, log=print):
    """Verifies every obligation and every chain edge; never reads <run_dir>/data.  Writes the transcript
    {"checked": [manifest ids], "verdict": "ACCEPT" | "REJECT", ...} and returns it.  Fail-closed: a driver crash or a
    malformed statement is a REJECT."""
    checked, failed, edges = [], [], []
    try:
        pub, run_seed = load_public(public_path or os.path.join(run_dir, "public.json"))
    except Exception as e:                        # noqa: BLE001 -- any malformed statement rejects
        tr = {"checked": [], "verdict": "REJECT", "failed": ["public.json: %r" % (e,)]}
        if transcript_out:
            with open(transcript_out, "w") as f:
                json.dump(tr, f, indent=1)
        return tr
    pool = None
    if run is None:
        pool = ServePool(run_dir, log)
        run = pool.run

    def roots_of(prefix):
        with open(os.path.join(run_dir, "proofs", prefix, "roots.bin"), "rb") as f:
            b = f.read()
        if len(b) != 96:
            raise ValueError("roots.bin of %s is malformed" % prefix)
        return b[:32], b[32:64], b[64:]

    try:
        for o in pub["obligations"]:
            why = []
            try:
                cmd = [driver, "verify", os.path.join("proofs", o["prefix"]), "%s:%s" % (run_seed, o["prefix"])] + \
                      _shape(pub, o) + [o["weight_root"]]
                ok, _, out = run(cmd, "verify " + o["prefix"], expect_reject_ok=True)
                if not (ok and "ACCEPT" in out):
                    why.append("%s: %s" % (o["prefix"], (out.strip().splitlines() or ["REJECT"])[-1]))
                # chain edge: this obligation's X is the producer's rescaled output, or the registered input
                rx = roots_of(o["prefix"])[0]
                if o.get("input_from") is None:
                    with open(os.path.join(run_dir, pub["input_root"]), "rb") as f:
                        want = f.read()
                    edge = "registered input -> " + o["prefix"]
                else:
                    want = roots_of(o["input_from"])[2]
                    edge = "%s -> %s" % (o["input_from"], o["prefix"])
                if rx != want:
                    why.append("edge " + edge)
                else:
                    edges.append(edge)
            except Exception as e:                # noqa: BLE001 -- crash, timeout, missing file: fail closed
                why.append("%s: %s" % (o["prefix"], str(e).splitlines()[0] if str(e) else repr(e)))
            if why:
                failed += why
            else:
                checked += ["%s.%s" % (o["prefix"], k) for k in MANIFEST_KINDS]
    finally:
        if pool is not None:
            pool.close()
    tr = {"checked": checked, "verdict": "ACCEPT" if not failed else "REJECT", "failed": failed, "edges": edges,
          "run_seed": run_seed, "stack": "p3 (Goldilocks, Basefold)"}
    if transcript_out:
        with open(transcript_out, "w") as f:
            json.dump(tr, f, indent=1)
    return tr


def main(argv):
    if len(argv) == 3 and argv[1] == "prove":
        prove_walk(argv[2])
        return 0
    if len(argv) == 5 and argv[1] == "verify":
        tr = verify_walk(argv[2], argv[3], argv[4])
        print(tr["verdict"])
        return 0 if tr["verdict"] == "ACCEPT" else 1
    sys.stderr.write(__doc__)
    return 2


if __name__ == "__main__":
    sys.exit(main(sys.argv))
