"""Hiding (salted-leaf) commitments: the oracle restatement against hashlib and the reference's host functions; the CUDA
kernels against the oracle and, on a GPU machine, against the reference's own salted commitment."""
import hashlib
import struct

import pytest

from conftest import lcg_cols


def test_salted_leaf_oracle_matches_hashlib_and_reference(orc, ref_or_none):
    for v, seed, i in [(0, 0, 0), (1, 2, 3), (0xFFFFFFFF00000000, 0xDEADBEEFCAFEF00D, 1 << 40), (12345, 99, 7)]:
        salt = hashlib.sha256(struct.pack("<QQ", seed, i)).digest()
        want = hashlib.sha256(struct.pack("<Q", v) + salt).digest()
        assert orc.salted_leaf(v, seed, i) == want
        if ref_or_none:
            assert ref_or_none.salted_leaf(v, seed, i) == want


def test_salted_tree_oracle_structure(orc):
    cw = lcg_cols(orc, 8, 1, 5)[0]
    tree = orc.merkle_build_salted(cw, 77).tobytes()
    leaves = [orc.salted_leaf(int(x), 77, i) for i, x in enumerate(cw)]
    assert tree[:8 * 32] == b"".join(leaves)
    plain = orc.merkle_build(cw).tobytes()
    assert tree[:32] != plain[:32] and len(tree) == len(plain)


@pytest.mark.gpu
@pytest.mark.parametrize("v,R", [(1, 1), (3, 2), (10, 1), (16, 1)])
def test_salted_commit_kernel_matches_oracle(orc, zk, prover, v, R):
    c = lcg_cols(orc, 1 << v, 1, 40 + v)[0]
    sseed = 0x1234567890ABCDEF + v
    cw = orc.rs_encode(c, R)
    want_tree = orc.merkle_build_salted(cw, sseed).tobytes()
    d = zk.p3.to_device(c)
    assert prover.commit_salted(d, R, sseed) == want_tree[-32:]
    root, cw_dev, tree_dev = prover.commit_salted(d, R, sseed, keep=True)
    assert root == want_tree[-32:] and (zk.p3.to_host(cw_dev) == cw).all()
    # the kept tree is capped: the levels from 64 leaves per node upwards, i.e. the tail of the full tree
    got = tree_dev.cpu().numpy().tobytes()
    assert len(got) == (len(want_tree) if (v + R) < 8 else (2 * (1 << (v + R - 6)) - 1) * 32)
    assert got == want_tree[-len(got):]
    assert prover.commit_salted(d, R, sseed + 1) != root and prover.commit_gpu_rootonly(d, R) != root


@pytest.mark.gpu
def test_salted_commit_equals_reference_cuda(orc, ref, zk, prover):
    if not ref.gpu_available():
        pytest.skip("reference shim sees no GPU")
    for v, R in [(12, 1), (18, 2)]:
        c = lcg_cols(orc, 1 << v, 1, 3 + v)[0]
        assert prover.commit_salted(zk.p3.to_device(c), R, 424242) == ref.salted_commit_root(c, R, 424242)


def test_zk_randomness_oracle_matches_reference(orc, ref_or_none):
    a = orc.zprng_fill(0xABCDEF, 1000)
    assert int(a[0]) == ((lambda s: (s ^ (s >> 31)) % 0xFFFFFFFF00000001)((0xABCDEF * 6364136223846793005 + 1442695040888963407) % (1 << 64)))
    assert orc.zprng_at(5, 0) == orc.zprng_at(5, 0) and orc.zprng_at(5, 0) != orc.zprng_at(5, 1)
    if ref_or_none:
        assert (ref_or_none.zprng_fill(0xABCDEF, 1000) == a).all()
        big = 1 << 20                                      # the reference's parallel (jump-ahead) path
        assert (ref_or_none.zprng_fill(77, big) == orc.zprng_fill(77, big)).all()
        for seed, i in [(1, 0), (0xFFFFFFFFFFFFFFFF, 12345), (99, 1 << 40)]:
            assert ref_or_none.zprng_at(seed, i) == orc.zprng_at(seed, i)


@pytest.mark.gpu
def test_zk_fill_kernels_match_oracle(orc, zk, prover):
    for n in (1, 7, 2048, 2049, (1 << 18) + 3):
        want = orc.zprng_fill(424242, n + 100)
        assert (zk.p3.to_host(prover.zk_fill_chain(424242, n)) == want[:n]).all()
        assert (zk.p3.to_host(prover.zk_fill_chain(424242, n, k0=100)) == want[100:100 + n]).all()
    got = zk.p3.to_host(prover.zk_fill_at(31337, 5000, i0=10))
    assert all(int(got[i]) == orc.zprng_at(31337, 10 + i) for i in (0, 1, 17, 4999))
    col = lcg_cols(orc, 1 << 10, 1, 8)[0]
    aug = zk.p3.to_host(prover.zk_augment(zk.p3.to_device(col), 2, 555))
    assert (aug[:1 << 10] == col).all() and (aug[1 << 10:] == orc.zprng_fill(555, 3 << 10)).all()
    assert (zk.p3.to_host(prover.zk_augment(zk.p3.to_device(col), 1, 0))[1 << 10:] == 0).all()
