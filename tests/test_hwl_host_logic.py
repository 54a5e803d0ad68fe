"""The fp8 (Hawkeye) matmul gadget (p3hwl, non-zk) through the host logic in zk_hillclimb_b200.hwl on CPU: tables and
witness equal the reference's, and the proof is accepted by the reference's own host-only verifier."""
import numpy as np
import pytest

from hwl_helpers import OracleHwlEngine, host_col, layer_inputs, ref_hwl_verify, ref_witness_column


def test_tables_equal_reference(ref, zk):
    import ctypes as C
    hwl = zk.hwl
    T = hwl.build_tables()
    u64p = C.POINTER(C.c_uint64)
    for i, name in enumerate(hwl.TAB_ORDER):
        rows, tid = C.c_uint32(0), (C.c_uint8 * 32)()
        nc = ref.lib.ref_hwl_table(i, None, C.byref(rows), tid)
        cols = [np.zeros(rows.value, dtype=np.uint64) for _ in range(nc)]
        ref.lib.ref_hwl_table(i, (u64p * nc)(*[c.ctypes.data_as(u64p) for c in cols]), None, None)
        assert bytes(tid) == T[name]["id"] and len(T[name]["cols"]) == nc
        assert all((a == b).all() for a, b in zip(cols, T[name]["cols"]))


@pytest.mark.parametrize("dims", [(2, 32, 2), (3, 70, 5), (4, 64, 8), (1, 31, 1)])
def test_witness_equals_reference_replay(ref, zk, dims):
    """Every column, every lookup index and the bf16 output equal p3hwl::gen_witness (which also cross-checks the output
    stage against a float replay)."""
    hwl = zk.hwl
    inp = layer_inputs(*dims, seed=sum(dims))
    wt = hwl.gen_witness(*dims, *inp)
    for dom, name, ncol in ((0, "dp", hwl.NDP), (1, "dg", hwl.NDG), (2, "dob", hwl.NDO), (3, "db", hwl.NDS), (4, "dn", hwl.NDS)):
        for c in range(ncol):
            mine = wt[name][c].numpy().view(np.uint64)
            assert (ref_witness_column(ref, dims, inp, dom, c, len(mine)) == mine).all(), (name, c)
    for i in range(hwl.NLU):
        mine = wt["lidx"][i].numpy().view(np.uint32)
        assert (ref_witness_column(ref, dims, inp, 5, i, len(mine), idx=True) == mine).all(), i
    import ctypes as C
    Y = np.zeros(dims[0] * dims[2], dtype=np.uint16)
    f = ref.lib.ref_hwl_witness
    f.restype = C.c_size_t
    vp = lambda a: a.ctypes.data_as(C.c_void_p)
    assert f(*[C.c_uint32(v) for v in dims], vp(inp[0]), vp(inp[1]), vp(inp[2]), vp(inp[3]), 6, 0, None, vp(Y)) == len(Y)
    assert (Y == wt["Y"]).all()


def test_unsupported_scale_raises(zk):
    hwl = zk.hwl
    x, w, xs, ws = layer_inputs(2, 32, 2, seed=3)
    xs = xs.copy()
    xs[0] = 0x7F800000                                   # +inf scale
    with pytest.raises(hwl.WitnessError, match="inf/nan x-scale"):
        hwl.gen_witness(2, 32, 2, x, w, xs, ws)


@pytest.mark.parametrize("dims", [(2, 32, 2), (3, 40, 4)])
def test_proof_accepted_by_reference_verifier(orc, ref, zk, dims):
    R, Q = 1, 24
    hwl = zk.hwl
    T = hwl.build_tables()
    inp = layer_inputs(*dims, seed=7)
    wt = hwl.gen_witness(*dims, *inp)
    eng = OracleHwlEngine(orc, ref)
    ops = hwl.commit_operands(eng, wt, R, host_col)
    tr = zk.Transcript("hwl-layer")
    pf = hwl.prove(eng, tr, wt, T, ops, R, Q, host_col)
    roots4 = [ops[k][1] for k in ("X", "W", "XS", "WS")]
    st0 = zk.Transcript("hwl-layer").state
    ok, st = ref_hwl_verify(ref, st0, dims, roots4, wt["Y"], R, Q, pf)
    assert ok and st == tr.state
    badY = wt["Y"].copy()
    badY[1] ^= 1
    assert not ref_hwl_verify(ref, st0, dims, roots4, badY, R, Q, pf)[0]
    assert not ref_hwl_verify(ref, st0, dims, roots4[1:] + roots4[:1], wt["Y"], R, Q, pf)[0]
    for off in (40, len(pf) // 2, len(pf) - 9):
        bad = bytearray(pf)
        bad[off] ^= 1
        assert not ref_hwl_verify(ref, st0, dims, roots4, wt["Y"], R, Q, bytes(bad))[0]
