"""The merged lookup (p3lu::prove_super, non-zk) on CUDA: same bytes as the oracle-backed run of the
same host logic, accepted by the reference's verifier, equal to the reference's own CUDA prover, and
its opening claims discharged by the batched opening."""
import ctypes as C

import numpy as np
import pytest

from lu_helpers import OracleLookupEngine, _Arr, make_lookup, table_id, verify_with_reference

pytestmark = pytest.mark.gpu


def gpu_groups(zk, prover, subs, R):
    import torch
    groups, roots_flat, committed = [], b"", b""
    for n, members in subs:
        mem = []
        for cols, idx in members:
            d = [zk.p3.to_device(cc) for cc in cols]
            roots = [prover.commit_gpu_rootonly(x, R) for x in d]
            mem.append((d, roots, torch.from_numpy(idx.view(np.int32)).cuda()))
            roots_flat += b"".join(roots)
            committed += b"\x01" * len(cols)
        groups.append((n, mem))
    return groups, roots_flat, committed


@pytest.mark.parametrize("m,shapes", [(4, [(5, 1)]), (6, [(7, 3), (5, 2)]), (10, [(14, 2), (12, 1)]), (16, [(18, 1)])])
def test_prove_super_matches_oracle_and_reference_verifier(orc, ref_or_none, zk, prover, m, shapes):
    R, Q = 1, 24
    tcols, subs = make_lookup(orc, m, shapes, 11 + m)
    groups, roots_flat, committed = gpu_groups(zk, prover, subs, R)
    tr = zk.Transcript("lu-main")
    pf, claims, cnt = zk.p3.prove_super(prover, tr, [zk.p3.to_device(t) for t in tcols], table_id(tcols), groups, R)
    # same host logic over the CPU oracle engine
    ogroups = [(n, [([_Arr(c) for c in cols], [orc.merkle_root(orc.rs_encode(c, R)) for c in cols], _Arr(idx))
                    for cols, idx in members]) for n, members in subs]
    tr2 = zk.Transcript("lu-main")
    pf2, claims2, cnt2 = zk.p3.prove_super(OracleLookupEngine(orc), tr2, [_Arr(t) for t in tcols], table_id(tcols), ogroups, R)
    assert pf == pf2 and tr.state == tr2.state
    assert (zk.p3.to_host(cnt) == cnt2.a).all()
    assert [(c[1], c[3]) for c in claims] == [(c[1], c[3]) for c in claims2]
    if ref_or_none:
        meta = [(n, len(mm)) for n, mm in groups]
        ok, st, vclaims = verify_with_reference(ref_or_none, zk.Transcript("lu-main").state, tcols, meta, roots_flat,
                                                committed, R, Q, pf)
        assert ok and st == tr.state and len(vclaims) == len(claims)


def test_lookup_claims_discharged_by_batched_opening(orc, ref_or_none, zk, prover):
    """End of the lookup pipeline: the ledger claims of prove_super, grouped by size class, are
    opened with prove_class and accepted by the verifiers on the continuing transcript."""
    R, Q = 1, 24
    tcols, subs = make_lookup(orc, 8, [(10, 2), (8, 1)], 5)
    groups, roots_flat, committed = gpu_groups(zk, prover, subs, R)
    tr = zk.Transcript("lu-main")
    pf, claims, cnt = zk.p3.prove_super(prover, tr, [zk.p3.to_device(t) for t in tcols], table_id(tcols), groups, R)
    classes = {}
    for col, root, pt, y in claims:          # PLedger::add: classes by size, points deduplicated in order
        cls = classes.setdefault(len(pt), {"pts": [], "ents": [], "y": []})
        key = pt.tobytes()
        keys = [p.tobytes() for p in cls["pts"]]
        if key not in keys:
            cls["pts"].append(pt)
            keys.append(key)
        cls["ents"].append((col, root, keys.index(key)))
        cls["y"].append(y)
    st_v = tr.state
    for i, (v, cls) in enumerate(classes.items()):
        pts = np.stack(cls["pts"])
        bp = prover.prove_class(tr, pts, cls["ents"], R, Q, "tf-bo%d" % i)
        roots = [e[1] for e in cls["ents"]]
        zid = [e[2] for e in cls["ents"]]
        for verifier in [orc] + ([ref_or_none] if ref_or_none else []):
            ok, st2 = verifier.bo_verify_class(st_v, pts, roots, zid, cls["y"], R, Q, "tf-bo%d" % i, bp)
            assert ok and st2 == tr.state
        st_v = tr.state


def test_reference_cuda_prove_super_same_bytes(orc, ref, zk, prover):
    if not ref.gpu_available():
        pytest.skip("reference shim sees no GPU")
    R, Q = 1, 24
    m, shapes = 8, [(12, 2), (10, 3)]
    tcols, subs = make_lookup(orc, m, shapes, 99)
    groups, roots_flat, committed = gpu_groups(zk, prover, subs, R)
    tr = zk.Transcript("lu-ref")
    pf, claims, cnt = zk.p3.prove_super(prover, tr, [zk.p3.to_device(t) for t in tcols], table_id(tcols), groups, R)
    u64p = C.POINTER(C.c_uint64)
    u32p = C.POINTER(C.c_uint32)
    tarr = [np.ascontiguousarray(t) for t in tcols]
    tp = (u64p * len(tarr))(*[a.ctypes.data_as(u64p) for a in tarr])
    wcols = [np.ascontiguousarray(c) for n, members in subs for cols, idx in members for c in cols]
    wp = (u64p * len(wcols))(*[a.ctypes.data_as(u64p) for a in wcols])
    idxs = [np.ascontiguousarray(idx) for n, members in subs for cols, idx in members]
    ip = (u32p * len(idxs))(*[a.ctypes.data_as(u32p) for a in idxs])
    sub_n = np.array([n for n, _ in subs], dtype=np.uint32)
    sub_k = np.array([len(mm) for _, mm in subs], dtype=np.uint32)
    st = (C.c_uint8 * 32)(*zk.Transcript("lu-ref").state)
    out = (C.c_uint8 * (1 << 20))()
    ms = C.c_double(0)
    f = ref.lib.ref_lu_prove_super
    f.restype = C.c_size_t
    n = f(st, tp, C.c_uint32(m), C.c_uint32(len(tarr)), C.c_uint32(len(subs)), sub_n.ctypes.data_as(C.c_void_p),
          sub_k.ctypes.data_as(C.c_void_p), wp, roots_flat, ip, C.c_uint32(R), C.c_uint32(Q), out, C.c_size_t(1 << 20),
          C.byref(ms))
    assert n > 0 and bytes(out)[:n] == pf and bytes(st) == tr.state
