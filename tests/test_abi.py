"""The C-ABI library: it loads, exports every symbol include/zkh.h declares, and its
host-side transcript entry points agree with the oracle.  No GPU work here."""
import ctypes as C
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    src = open(os.path.join(ROOT, "include", "zkh.h")).read()
    return sorted(set(re.findall(r"ZKH_API\s+[\w\s\*]+?\b(zkh_\w+)\s*\(", src)))


def test_library_exports_every_declared_symbol(zk):
    names = declared_symbols()
    assert len(names) >= 20
    L = C.CDLL(zk.lib_path())
    missing = [n for n in names if not hasattr(L, n)]
    assert not missing, missing
    assert b"sm_100a" in C.cast(zk.load_library().zkh_version(), C.c_char_p).value


def test_header_cites_reference_for_compute_entry_points():
    src = open(os.path.join(ROOT, "include", "zkh.h")).read()
    assert src.count("zkllm-src/") >= 10


def test_host_transcript_matches_oracle(zk, orc, golden):
    tr = zk.Transcript("p3-golden")
    st = orc.tr_init("p3-golden")
    assert tr.state == st and st.hex() == golden["transcript"][0]
    for label, n, sthex, a, ix in golden["transcript"][1:]:
        data = bytes((len(label) * 11 + j) & 0xFF for j in range(n))
        tr.absorb(label, data)
        assert (tr.chal(), tr.idx_from(1 << 21)) == (a, ix)
        assert tr.state.hex() == sthex
    # long seed and long data take the multi-block paths
    seed = bytes(range(200))
    assert zk.Transcript(seed).state == orc.tr_init(seed)
    tr, st = zk.Transcript("x"), orc.tr_init("x")
    for n in (0, 55, 56, 64, 1000):
        d = bytes((7 * j) & 0xFF for j in range(n))
        tr.absorb("lbl", d)
        st = orc.tr_absorb(st, "lbl", d)
        assert tr.state == st
    st, out = orc.tr_challenge_bytes(st)
    assert tr.challenge_bytes() == out and tr.state == st


def test_missing_library_fails_loudly(zk, monkeypatch, tmp_path):
    import importlib
    lib = importlib.import_module("zk_hillclimb_b200._lib")
    monkeypatch.setattr(lib, "_lib", None)
    monkeypatch.setattr(lib, "HERE", str(tmp_path))
    try:
        lib.load_library()
    except FileNotFoundError as e:
        assert "no CPU fallback" in str(e)
    else:
        raise AssertionError("a missing library must raise")


def test_misaligned_columns_are_refused_before_any_launch():
    """Columns are read with 128-bit loads: a device address that is not 16-byte aligned is refused with ZKH_ERR_ARG
    (argument check only: the pointers are never dereferenced, no kernel is launched, no GPU is needed)."""
    import ctypes as C
    import zkh_import
    zk = zkh_import.load()
    L = zk.load_library()
    err = C.create_string_buffer(256)
    z = (C.c_uint64 * 2)(1, 2)
    y = C.c_uint64(0)
    rc = L.zkh_gl_mle_eval_static(C.c_void_p(0), C.c_void_p(0x10008), z, 2, C.c_void_p(0x20000), err, len(err))
    assert rc == -1 and b"16-byte" in err.value
