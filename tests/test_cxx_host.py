"""The C++ host side over the C ABI (include/zkh_p3.hpp): a proving flow written in C++ the way a gadget of the
reference is written (commit, absorb roots, p3sg::sc_prove_gpu, p3bf::prove_eval_dev, p3gkr::prove_dev,
p3bo::prove_class) gives the bytes the CPU checker gives for the same inputs, and the reference's verifiers accept."""
import os
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "zk-hillclimb_b200")
EXE = os.path.join(PKG, "zkh_p3_selftest")


def test_cxx_header_compiles_and_program_fails_loudly_without_a_gpu(zk, tmp_path):
    """g++ -Wall -Werror on a translation unit that only includes the header; the built program exits non-zero with the
    library's message where there is no CUDA device (no CPU fallback behind the C++ side either)."""
    tu = tmp_path / "tu.cpp"
    tu.write_text('#include "zkh_p3.hpp"\nint main() { zkh_p3::Transcript t("x"); return (int)(t.chal() & 0); }\n')
    out = tmp_path / "tu"
    subprocess.check_call(["g++", "-std=c++17", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), str(tu), "-o", str(out),
                           "-L", PKG, "-lzkh", "-Wl,-rpath," + PKG])
    assert subprocess.run([str(out)]).returncode == 0
    assert os.path.exists(EXE) and os.path.exists(os.path.join(PKG, "zkh_p3_gadgets_selftest")), "build() makes the selftest programs"
    import torch
    if not torch.cuda.is_available():
        r = subprocess.run([EXE], capture_output=True, text=True)
        assert r.returncode != 0 and "cannot create a context" in r.stderr


def run_selftest(v, R, Q):
    r = subprocess.run([EXE, str(v), str(R), str(Q)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    out = {}
    for line in r.stdout.splitlines():
        k, val = line.split(" ", 1)
        out[k] = val
    return out


@pytest.mark.gpu
@pytest.mark.parametrize("v,R,Q", [(10, 1, 24), (5, 2, 20), (14, 1, 24)])
def test_cxx_flow_matches_checker(orc, ref_or_none, v, R, Q):
    got = run_selftest(v, R, Q)
    a, s = orc.lcg(1 << v, 0xC0FFEE)
    b, s = orc.lcg(1 << v, s)
    ra, rb = orc.merkle_root(orc.rs_encode(a, R)), orc.merkle_root(orc.rs_encode(b, R))
    assert got["root_a"] == ra.hex() and got["root_b"] == rb.hex()
    st = orc.tr_init("cxx-selftest")
    st = orc.tr_absorb(st, "root", ra)
    st = orc.tr_absorb(st, "root", rb)
    from oracle import F_PROD2
    st, m, r, f = orc.sumcheck(st, "sc", F_PROD2, 3, [a, b])
    assert got["sc_msgs"] == np.asarray(m, dtype=np.uint64).tobytes().hex()
    assert got["sc_chals"] == np.asarray(r, dtype=np.uint64).tobytes().hex()
    assert got["sc_finals"] == np.asarray(f, dtype=np.uint64).tobytes().hex()
    ya = orc.mle_eval(a, r)
    want_ev = orc.bf_prove_eval(a, r, ya, R, Q, orc.rs_encode(a, R))
    assert got["eval_proof"] == want_ev.hex()
    st, gp, rfin, cpq = orc.gkr_prove(st, "gkr", a, b, True)
    assert got["gkr_proof"] == gp.hex()
    assert got["gkr_rfin"] == np.asarray(rfin, dtype=np.uint64).tobytes().hex()
    assert got["gkr_cpq"] == np.asarray(cpq, dtype=np.uint64).tobytes().hex()
    pts = np.stack([np.asarray(r, dtype=np.uint64), np.asarray(rfin, dtype=np.uint64)])
    st0 = st
    want_bo, st = orc.bo_prove_class(st0, pts, [a, b, a], [ra, rb, ra], [0, 1, 1], R, Q, "cxx-bo")
    assert got["batch_proof"] == want_bo.hex()
    assert got["state"] == st.hex()
    assert got["bad_call_throws"] == "1"
    if ref_or_none:
        assert ref_or_none.bf_verify_eval(bytes.fromhex(got["eval_proof"]))
        y = [ya, orc.mle_eval(b, rfin), orc.mle_eval(a, rfin)]
        ok, st2 = ref_or_none.bo_verify_class(st0, pts, [ra, rb, ra], [0, 1, 1], y, R, Q, "cxx-bo",
                                              bytes.fromhex(got["batch_proof"]))
        assert ok and st2 == st


GEXE = os.path.join(PKG, "zkh_p3_gadgets_selftest")


def _i8_stream(n, s):
    out = np.empty(n, dtype=np.int64)
    for i in range(n):
        s = (s * 6364136223846793005 + 1442695040888963407) % (1 << 64)
        out[i] = ((s >> 33) % 255) - 127
    return out, s


@pytest.mark.gpu
@pytest.mark.parametrize("li,lj,lk,sf", [(4, 6, 5, 16), (3, 5, 7, 14), (5, 7, 6, 20)])
def test_cxx_gadgets_match_python_host_logic(zk, prover, li, lj, lk, sf):
    """Quantised matmul proof + rescale with range lookups, standalone and composed, driven from C++: the same bytes as the
    Python host logic (which is pinned to the reference's provers and verifiers in the imm / irs tests)."""
    from irs_helpers import irs_tables, lift
    R, Q = 1, 24
    r = subprocess.run([GEXE] + [str(v) for v in (li, lj, lk, sf, R, Q)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    got = dict(line.split(" ", 1) for line in r.stdout.splitlines())
    I, J, K = 1 << li, 1 << lj, 1 << lk
    x, s = _i8_stream(I * J, 0x5EED)
    w, s = _i8_stream(J * K, s)
    y = (x.reshape(I, J) @ w.reshape(J, K)).reshape(-1)
    p3 = zk.p3
    com = lambda a: (lambda d: (d, prover.commit_gpu_rootonly(d, R)))(p3.to_device(lift(a)))
    X, W, Y = com(x), com(w), com(y)
    assert got["root_Y"] == Y[1].hex()
    tr = zk.Transcript("cxx-imm")
    assert got["imm_proof"] == p3.imm_prove(prover, tr, X, W, Y, lj, lk, li, R, Q).hex() and got["imm_state"] == tr.state.hex()
    T = irs_tables(zk, sf)
    yo, L, iL, iY = prover.irs_witness(Y[0], sf, 1)
    Yo = (yo, prover.commit_gpu_rootonly(yo, R))
    tr = zk.Transcript("cxx-irs")
    assert got["irs_proof"] == p3.irs_prove(prover, tr, T, Y, Yo, (L, iL, iY), li + lk, sf, 1, R, Q).hex()
    assert got["irs_state"] == tr.state.hex() and got["irs_rootY"] == Yo[1].hex()
    tr = zk.Transcript("cxx-c0")
    ledger, luq = p3.Ledger(), []
    p1 = p3.imm_prove(prover, tr, X, W, Y, lj, lk, li, R, Q, ledger)
    p2 = p3.irs_prove(prover, tr, T, Y, Yo, (L, iL, iY), li + lk, sf, 1, R, Q, ledger, luq)
    lug = p3.lu_flush(prover, tr, luq, ledger, R)
    bo = p3.tail_prove(prover, tr, ledger, R, Q, "c0-bo")
    blob = lambda bs: b"".join(len(b).to_bytes(4, "little") + b for b in bs)
    assert got["c0_imm"] == p1.hex() and got["c0_irs"] == p2.hex() and got["c0_lug"] == blob(lug).hex()
    assert got["c0_batches"] == blob(bo).hex() and got["c0_state"] == tr.state.hex()
