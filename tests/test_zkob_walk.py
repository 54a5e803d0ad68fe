"""One attention block and one gate of the first proof stack walked through ALL twelve driver programs in claim mode, every program
reading the chain file the previous one wrote: RMS norm, rescale, three fully connected layers, rotary embedding, per-head slicing, per
head the score product, the row maximum with the temperature-8 softmax (head 0) or the plain causal softmax (head 1), the value
product, the head merge, the output projection, the skip connection and a gated activation; then ONE batch opening of every claim of
the walk (two generator domains) and its verifier.  Every chain file is compared with a numpy statement of the same integer chain."""
import ctypes as C
import math
import os
import subprocess

import numpy as np
import pytest

import fr_oracle as fo

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "zk-hillclimb_b200")
B, CC, HD, NH = 8, 16, 8, 2
RS_FC, RS_ROPE, RS_SC, RS_O = 4, 6, 3, 5                            # the rescaling exponents of the walk (tables of 2^k rows must fit the tiny grids)


def rescale(x, log_sf):
    """rescaling_kernel: the remainder in [-sf/2, sf/2)."""
    return (x.astype(np.int64) + (1 << (log_sf - 1))) >> log_sf


def rope(T, cos, sin):
    e = np.arange(T.shape[1])
    sign = np.where(e & (HD // 2), 1, -1).astype(np.int64)
    return T.astype(np.int64) * cos[:, e % HD] + T[:, e ^ (HD // 2)].astype(np.int64) * (sign * sin[:, e % HD])


def softmax_rows(E, mask):
    S = (E * mask).sum(axis=1, keepdims=True)
    return ((mask * E << 17) + S) // (2 * S)


def chain(seed):
    """The integer chain of the walk in numpy: a dict of every tensor a program reads or writes."""
    g = np.random.default_rng(seed)
    t = {}
    t["X"] = g.integers(-128, 128, (B, CC)).astype(np.int32)
    t["gain"] = g.integers(1, 4, CC).astype(np.int32)
    t["c_eps"] = 7 * CC
    R = []
    for s in range(B):
        M = int((t["X"][s].astype(np.int64) ** 2).sum()) + t["c_eps"]
        R.append(math.isqrt((CC << 64) // M))
    t["R"] = np.array(R, dtype=np.int32)
    W = t["R"].astype(np.int64)[:, None] * t["gain"].astype(np.int64)[None, :]
    t["normY"] = rescale(W, 16) * t["X"]                             # zkob_rmsnorm's Y chain file (int64)
    t["n1"] = rescale(t["normY"], 7)
    t["Xn"] = rescale(t["n1"], 5).astype(np.int32)
    for k in "qkvo":
        t["W" + k] = g.integers(-2, 3, (CC, CC)).astype(np.int32)
    ang = g.uniform(0, 2 * np.pi, (B, HD))
    t["cos"], t["sin"] = np.rint(np.cos(ang) * 16).astype(np.int32), np.rint(np.sin(ang) * 16).astype(np.int32)
    for k in "qkv":
        t["Y" + k] = t["Xn"].astype(np.int64) @ t["W" + k].astype(np.int64)
        t[k + "0"] = rescale(t["Y" + k], RS_FC).astype(np.int32)
    for k in "qk":
        t["rope" + k] = rope(t[k + "0"], t["cos"], t["sin"])
        t[k + "r"] = rescale(t["rope" + k], RS_ROPE).astype(np.int32)
    mask = np.tril(np.ones((B, B), dtype=np.int64))
    x8 = np.arange(-62, 2)
    t["map8"] = np.maximum(1, np.rint(4096 * np.exp(x8 / 8.0))).astype(np.int32)
    t["map8"][-1] = 0
    t["map"] = np.maximum(1, np.rint(4096 * np.exp((np.arange(-32, 32) - 31) / 8.0))).astype(np.int32)
    for h in range(NH):
        sl = slice(h * HD, (h + 1) * HD)
        Qh, Kh, Vh = t["qr"][:, sl], t["kr"][:, sl], t["v0"][:, sl]
        t["sc%d" % h] = Qh.astype(np.int64) @ Kh.astype(np.int64).T
        z = rescale(t["sc%d" % h], RS_SC).astype(np.int32)
        t["z%d" % h] = z
        if h == 0:
            mx = np.array([z[i, :i + 1].max() for i in range(B)], dtype=np.int32)
            t["mx0"] = mx
            Dm = np.where(mask == 1, z - mx[:, None], 1)
            assert Dm.min() >= -62
            E = t["map8"][Dm + 62].astype(np.int64)
            t["P0"] = softmax_rows(E, np.ones_like(mask)).astype(np.int32)
        else:
            assert z.min() >= -32 and z.max() < 32
            t["P1"] = softmax_rows(t["map"][z + 32].astype(np.int64), mask).astype(np.int32)
        assert np.abs(z).max() <= 31                                 # the row-maximum limbs: differences below 64
        t["pv%d" % h] = t["P%d" % h].astype(np.int64) @ Vh.astype(np.int64)
        t["o%da" % h] = rescale(t["pv%d" % h], 6)
        t["o%db" % h] = rescale(t["o%da" % h], 6)
        t["o%d" % h] = rescale(t["o%db" % h], 4).astype(np.int32)
    t["O2"] = np.concatenate([t["o0"], t["o1"]], axis=1).astype(np.int32)
    t["Yo"] = t["O2"].astype(np.int64) @ t["Wo"].astype(np.int64)
    t["attn"] = rescale(t["Yo"], RS_O).astype(np.int32)
    assert t["attn"].min() >= -64 and t["attn"].max() < 64           # the gate's table covers [-64, 64)
    xg = np.arange(-64, 64)
    t["mapg"] = np.rint(xg / (1 + np.exp(-xg / 8.0))).astype(np.int32)
    assert t["mapg"][64] == 0
    t["H"] = t["mapg"][t["attn"] + 64].astype(np.int64) * t["Xn"]
    return t


def test_the_numpy_chain_stays_inside_every_table():
    t = chain(3)
    assert t["P0"].shape == (B, B) and (np.triu(t["P0"], 1) == 0).all() and abs(int(t["P0"][B - 1].sum()) - 65536) <= B
    assert (np.triu(t["P1"], 1) == 0).all() and abs(int(t["P1"][B - 1].sum()) - 65536) <= B


def run(exe, *args):
    r = subprocess.run([os.path.join(PKG, exe)] + [str(a) for a in args], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, (exe, args[:3], r.stdout[-400:], r.stderr[-400:])
    return r.stdout


@pytest.mark.gpu
def test_an_attention_block_and_a_gate_through_all_twelve_programs(tmp_path):
    if not fo.ReferenceFr.available():
        pytest.skip("oracle/_ref/libfrref.so not built")
    lib = fo.ReferenceFr().lib
    if not lib.refA_gpu_available():
        pytest.skip("no GPU")
    d = tmp_path
    for name, k in (("g16", 16), ("g8", 8), ("q", 1)):
        buf = (C.c_uint8 * (k * 144))()
        assert lib.refA_commit_random(C.c_uint32(k), buf) == 0
        (d / name).write_bytes(bytes(buf))
    g16, g8, q = d / "g16", d / "g8", d / "q"
    t = chain(3)
    for name in ("X", "R", "gain", "Wq", "Wk", "Wv", "Wo", "cos", "sin", "map8", "map", "mapg"):
        (d / name).write_bytes(t[name].tobytes())
    acc, vacc = d / "acc", d / "vacc"
    acc.mkdir()
    vacc.mkdir()
    verifies = []                                                    # (program, arguments after "verify") replayed once the provers are done

    def ob(name):
        (d / name).mkdir()
        return d / name

    def as64(src, dst, shape):
        (d / dst).write_bytes(np.frombuffer((d / src).read_bytes(), dtype=np.int32).astype(np.int64).tobytes())

    def same(path, want, dtype):
        got = np.frombuffer((d / path).read_bytes(), dtype=dtype)
        assert np.array_equal(got, np.asarray(want).astype(dtype).ravel()), path

    def rs(tag, src, dst, rows, cols, log_sf, gen, want):
        o = ob("ob_" + tag)
        run("zkob_rescale", "prove", o, "w:" + tag, d / src, rows, cols, log_sf, gen, q, d / dst, "--claims", acc, tag)
        verifies.append(("zkob_rescale", [o, "w:" + tag, rows, cols, log_sf, gen, q, "--claims", vacc, tag]))
        same(dst, want, np.int32)

    def fc(tag, xsrc, wsrc, rows, n_in, n_out, gen_in, gen_out, dst, want):
        o = ob("ob_" + tag)
        run("zkob_fc", "commit", d / wsrc, n_in, n_out, gen_out, d / ("cw_" + tag))
        run("zkob_fc", "prove", o, "w:" + tag, d / xsrc, d / wsrc, rows, n_in, n_out, gen_in, gen_out, q, d / dst, "--claims", acc, tag, d / ("cw_" + tag))
        verifies.append(("zkob_fc", [o, "w:" + tag, rows, n_in, n_out, d / ("cw_" + tag), gen_in, gen_out, q, "--claims", vacc, tag]))
        same(dst, want, np.int64)

    # RMS norm, then two rescalings down to the activation scale
    o = ob("ob_norm")
    reg = d / "registered_com_g.bin"
    run("zkob_rmsnorm", "prove", ob("ob_norm_plain"), "x", d / "X", d / "R", d / "gain", B, CC, t["c_eps"], g16, g8, q)
    reg.write_bytes((d / "ob_norm_plain" / "com_g.bin").read_bytes())
    run("zkob_rmsnorm", "prove", o, "w:norm", d / "X", d / "R", d / "gain", B, CC, t["c_eps"], g16, g8, q, d / "normW.i64", d / "normY.i64",
        "--claims", acc, "norm", reg)
    verifies.append(("zkob_rmsnorm", [o, "w:norm", B, CC, t["c_eps"], reg, g16, g8, q, "--claims", vacc, "norm"]))
    same("normY.i64", t["normY"], np.int64)
    rs("norm.rs1", "normY.i64", "n1.i32", B, CC, 7, g16, t["n1"])
    as64("n1.i32", "n1.i64", (B, CC))
    rs("norm.rs2", "n1.i64", "Xn.i32", B, CC, 5, g16, t["Xn"])
    # the three projections, rotary embedding on Q and K
    for k in "qkv":
        fc("fc" + k, "Xn.i32", "W" + k, B, CC, CC, g16, g16, "Y%s.i64" % k, t["Y" + k])
        rs("fc%s.rs" % k, "Y%s.i64" % k, "%s0.i32" % k, B, CC, RS_FC, g16, t[k + "0"])
    for k in "qk":
        o = ob("ob_rope" + k)
        run("zkob_rope", "prove", o, "w:rope" + k, d / ("%s0.i32" % k), B, CC, HD, d / "cos", d / "sin", g16, q, d / ("rope%s.i64" % k), "--claims", acc, "rope" + k)
        verifies.append(("zkob_rope", [o, "w:rope" + k, B, CC, HD, d / "cos", d / "sin", g16, q, "--claims", vacc, "rope" + k]))
        same("rope%s.i64" % k, t["rope" + k], np.int64)
        rs("rope%s.rs" % k, "rope%s.i64" % k, "%sr.i32" % k, B, CC, RS_ROPE, g16, t[k + "r"])
    # per-head operands
    o, sl = ob("ob_slice"), ob("slices")
    run("zkob_headslice", "prove", o, "w:slice", d / "qr.i32", d / "kr.i32", d / "v0.i32", B, CC, HD, g16, g8, q, sl, "--claims", acc, "slice")
    verifies.append(("zkob_headslice", [o, "w:slice", B, CC, HD, g16, g8, q, "--claims", vacc, "slice"]))
    for h in range(NH):
        hh = "%02d" % h
        same("slices/KhT%s.i32.bin" % hh, t["kr"][:, h * HD:(h + 1) * HD].T, np.int32)
        fc("sc" + hh, "slices/Qh%s.i32.bin" % hh, "slices/KhT%s.i32.bin" % hh, B, HD, B, g8, g8, "sc%s.i64" % hh, t["sc%d" % h])
        rs("sc%s.rs" % hh, "sc%s.i64" % hh, "z%s.i32" % hh, B, B, RS_SC, g8, t["z%d" % h])
        if h == 0:                                                   # the faithful chain: row maximum, then the temperature-8 softmax
            o = ob("ob_rowmax")
            run("zkob_rowmax", "prove", o, "w:rowmax", d / "z00.i32", B, B, "causal", 0, 64, 1, g8, g8, q, d / "mx00.i32", "--claims", acc, "rowmax")
            verifies.append(("zkob_rowmax", [o, "w:rowmax", B, B, "causal", 0, 64, 1, g8, g8, q, "--claims", vacc, "rowmax"]))
            same("mx00.i32", t["mx0"], np.int32)
            o = ob("ob_sm8")
            run("zkob_softmax8", "prove", o, "w:sm8", d / "z00.i32", d / "mx00.i32", B, B, -62, 64, d / "map8", 256, g8, q, d / "P00.i32", "--claims", acc, "sm8")
            verifies.append(("zkob_softmax8", [o, "w:sm8", B, B, -62, 64, d / "map8", 256, g8, q, "--claims", vacc, "sm8"]))
        else:
            o = ob("ob_sm")
            run("zkob_softmax", "prove", o, "w:sm", d / "z01.i32", B, B, -32, 64, d / "map", 256, g8, q, d / "P01.i32", "--claims", acc, "sm")
            verifies.append(("zkob_softmax", [o, "w:sm", B, B, -32, 64, d / "map", 256, g8, q, "--claims", vacc, "sm"]))
        same("P%s.i32" % hh, t["P%d" % h], np.int32)
        fc("pv" + hh, "P%s.i32" % hh, "slices/Vh%s.i32.bin" % hh, B, B, HD, g8, g8, "pv%s.i64" % hh, t["pv%d" % h])
        rs("pv%s.rs1" % hh, "pv%s.i64" % hh, "o%sa.i32" % hh, B, HD, 6, g8, t["o%da" % h])
        as64("o%sa.i32" % hh, "o%sa.i64" % hh, (B, HD))
        rs("pv%s.rs2" % hh, "o%sa.i64" % hh, "o%sb.i32" % hh, B, HD, 6, g8, t["o%db" % h])
        as64("o%sb.i32" % hh, "o%sb.i64" % hh, (B, HD))
        rs("pv%s.rs3" % hh, "o%sb.i64" % hh, "out%s.i32.bin" % hh, B, HD, 4, g8, t["o%d" % h])
    # merge, output projection, skip connection, gate
    o = ob("ob_merge")
    run("zkob_headmerge", "prove", o, "w:merge", d / "out", B, CC, HD, "concat", g16, g8, q, d / "O2.i32", "--claims", acc, "merge")
    verifies.append(("zkob_headmerge", [o, "w:merge", B, CC, HD, "concat", g16, g8, q, "--claims", vacc, "merge"]))
    same("O2.i32", t["O2"], np.int32)
    fc("fco", "O2.i32", "Wo", B, CC, CC, g16, g16, "Yo.i64", t["Yo"])
    rs("fco.rs", "Yo.i64", "attn.i32", B, CC, RS_O, g16, t["attn"])
    run("zkob_skip", "add", d / "ob_norm" / "com_X.bin", d / "ob_fco.rs" / "com_Xr.bin", d / "com_resid.bin")
    assert "ACCEPT" in run("zkob_skip", "verify", d / "ob_norm" / "com_X.bin", d / "ob_fco.rs" / "com_Xr.bin", d / "com_resid.bin")
    o = ob("ob_glu")
    run("zkob_glu", "prove", o, "w:glu", d / "attn.i32", d / "Xn.i32", B, CC, -64, 128, d / "mapg", g16, q, d / "H.i64", "--claims", acc, "glu")
    verifies.append(("zkob_glu", [o, "w:glu", B, CC, -64, 128, d / "mapg", g16, q, "--claims", vacc, "glu"]))
    same("H.i64", t["H"], np.int64)
    # every verifier, then ONE batch opening over the whole walk
    for prog, args in verifies:
        assert "ACCEPT-conditional" in run(prog, "verify", *args), prog
    assert (acc / "claims.bin").read_bytes() == (vacc / "claims.bin").read_bytes()
    run("zkob_batchopen", "prove", acc, "w", q, "16=%s" % g16, "8=%s" % g8)
    out = run("zkob_batchopen", "verify", acc, vacc, "w", q, "16=%s" % g16, "8=%s" % g8)
    assert "opening_batch ACCEPT" in out and "2 domains" in out, out
    # a claim list from another walk seed is refused
    (vacc / "claims.bin").write_bytes((acc / "claims.bin").read_bytes()[:-1] + b"\x01")
    r = subprocess.run([os.path.join(PKG, "zkob_batchopen"), "verify", acc, vacc, "w", q, "16=%s" % g16, "8=%s" % g8], capture_output=True, text=True, timeout=600)
    assert r.returncode == 1 and "REJECT" in r.stdout


def test_every_chain_file_without_a_gpu(tmp_path):
    """Every program writes its chain file (the integer tensor the next program reads) before it touches the device: each program of
    the walk is started on the numpy chain's inputs and its chain file compared with the numpy statement.  Without a GPU the run then
    stops at the device context; with one it goes on to prove."""
    d = tmp_path
    t = chain(3)
    for name, k in (("g16", 16), ("g8", 8), ("q", 1)):
        (d / name).write_bytes(bytes(k * 144))                       # sizes only: the layout rules are checked, the points are not read
    g16, g8, q = d / "g16", d / "g8", d / "q"

    def put(name, a, dtype):
        (d / name).write_bytes(np.asarray(a).astype(dtype).tobytes())
        return d / name

    def start(prog, *args):
        (d / "ob").mkdir(exist_ok=True)
        r = subprocess.run([os.path.join(PKG, prog), "prove", d / "ob", "s"] + [str(a) for a in args], capture_output=True, text=True, timeout=600)
        assert r.returncode == 0 or "no CUDA device" in r.stderr, (prog, r.stdout[-300:], r.stderr[-300:])

    def same(path, want, dtype):
        assert np.array_equal(np.frombuffer((d / path).read_bytes(), dtype=dtype), np.asarray(want).astype(dtype).ravel()), path

    start("zkob_rmsnorm", put("X", t["X"], np.int32), put("R", t["R"], np.int32), put("gain", t["gain"], np.int32), B, CC, t["c_eps"], g16, g8, q, d / "W.i64", d / "Y.i64")
    same("Y.i64", t["normY"], np.int64)
    same("W.i64", t["R"].astype(np.int64)[:, None] * t["gain"].astype(np.int64)[None, :], np.int64)
    start("zkob_rescale", put("normY", t["normY"], np.int64), B, CC, 7, g16, q, d / "n1.i32")
    same("n1.i32", t["n1"], np.int32)
    start("zkob_fc", put("Xn", t["Xn"], np.int32), put("Wq", t["Wq"], np.int32), B, CC, CC, g16, g16, q, d / "Yq.i64")
    same("Yq.i64", t["Yq"], np.int64)
    start("zkob_rope", put("q0", t["q0"], np.int32), B, CC, HD, put("cos", t["cos"], np.int32), put("sin", t["sin"], np.int32), g16, q, d / "rope.i64")
    same("rope.i64", t["ropeq"], np.int64)
    (d / "sl").mkdir()
    start("zkob_headslice", put("qr", t["qr"], np.int32), put("kr", t["kr"], np.int32), put("v0", t["v0"], np.int32), B, CC, HD, g16, g8, q, d / "sl")
    for h in range(NH):
        sl = slice(h * HD, (h + 1) * HD)
        same("sl/Qh%02d.i32.bin" % h, t["qr"][:, sl], np.int32)
        same("sl/KhT%02d.i32.bin" % h, t["kr"][:, sl].T, np.int32)
        same("sl/Vh%02d.i32.bin" % h, t["v0"][:, sl], np.int32)
    start("zkob_rowmax", put("z0", t["z0"], np.int32), B, B, "causal", 0, 64, 1, g8, g8, q, d / "mx.i32")
    same("mx.i32", t["mx0"], np.int32)
    start("zkob_softmax8", d / "z0", put("mx0", t["mx0"], np.int32), B, B, -62, 64, put("map8", t["map8"], np.int32), 256, g8, q, d / "P0.i32")
    same("P0.i32", t["P0"], np.int32)
    start("zkob_softmax", put("z1", t["z1"], np.int32), B, B, -32, 64, put("map", t["map"], np.int32), 256, g8, q, d / "P1.i32")
    same("P1.i32", t["P1"], np.int32)
    for h in range(NH):
        put("out%02d.i32.bin" % h, t["o%d" % h], np.int32)
    start("zkob_headmerge", d / "out", B, CC, HD, "concat", g16, g8, q, d / "O2.i32")
    same("O2.i32", t["O2"], np.int32)
    start("zkob_headmerge", d / "out", B, CC, HD, "pi157", g16, g8, q, d / "O2p.i32")
    m = np.arange(B * CC)
    same("O2p.i32", t["O2"][m % B, m // B], np.int32)
    start("zkob_glu", put("attn", t["attn"], np.int32), d / "Xn", B, CC, -64, 128, put("mapg", t["mapg"], np.int32), g16, q, d / "H.i64")
    same("H.i64", t["H"], np.int64)
    # a vocabulary-padded row maximum: 11 real columns of 16, two limb planes
    zv = np.random.default_rng(4).integers(-500, 500, (B, 11)).astype(np.int32)
    start("zkob_rowmax", put("zv", zv, np.int32), B, 16, "vpad", 11, 32, 2, g16, g8, q, d / "mxv.i32")
    same("mxv.i32", zv.max(axis=1), np.int32)
