"""Pedersen row commitments over BLS12-381 G1 (the reference's Commitment::commit, zkllm-src/commitment.cu:41-103).
CPU: the Python-integer oracle is checked against the group itself (the byte form has no CPU pin: the reference's G1 code is
device-only).  GPU: the CUDA kernels give the bytes of the oracle and of the reference's own kernels (oracle/_ref/libfrref.so)."""
import ctypes as C
import random

import numpy as np
import pytest

import g1_oracle as g1


def test_oracle_group_law_and_commitment():
    assert g1.on_curve(g1.GEN) and g1.to_affine(g1.ZERO) is None
    rnd = random.Random(7)
    gens = [g1.scalar_mul(g1.GEN, rnd.randrange(1, 1 << 200)) for _ in range(4)]
    assert all(g1.on_curve(p) for p in gens)
    a, b, c = gens[:3]
    assert g1.to_affine(g1.add(g1.add(a, b), c)) == g1.to_affine(g1.add(a, g1.add(b, c)))
    assert g1.to_affine(g1.add(a, a)) == g1.to_affine(g1.double(a))           # the equal-points branch
    assert g1.add(g1.ZERO, a) == a and g1.add(a, g1.ZERO) == a
    rows = [[rnd.randrange(1 << 255) for _ in gens], [0, 1, 15, (1 << 256) - 1]]
    for row, com in zip(rows, g1.pedersen_commit(gens, rows)):
        naive = g1.ZERO
        for s, p in zip(row, gens):
            naive = g1.add(naive, g1.scalar_mul(p, s))
        assert g1.on_curve(com) and g1.to_affine(com) == g1.to_affine(naive)
    assert g1.from_bytes(g1.to_bytes(gens[0])) == gens[0] and len(g1.to_bytes(g1.GEN)) == 144


def _scalars(rnd, m, n):
    return [[rnd.randrange(1 << 255) if rnd.random() < 0.8 else rnd.randrange(1 << 16) for _ in range(n)] for _ in range(m)]


def _pack_scalars(rows):
    return np.frombuffer(b"".join(int(s).to_bytes(32, "little") for r in rows for s in r), dtype=np.uint32).copy()


@pytest.mark.gpu
@pytest.mark.parametrize("m,n", [(1, 1), (2, 5), (3, 16)])
def test_kernels_match_oracle(zk, prover, m, n):
    import torch
    rnd = random.Random(100 + n)
    gens = [g1.scalar_mul(g1.GEN, rnd.randrange(1, 1 << 250)) for _ in range(n)]
    rows = _scalars(rnd, m, n)
    rows[0][0] = 0
    gd = torch.from_numpy(np.frombuffer(b"".join(g1.to_bytes(p) for p in gens), dtype=np.uint8).copy()).cuda()
    sd = torch.from_numpy(_pack_scalars(rows).view(np.int32)).cuda()
    out = zk.fr.g1_pedersen_commit(prover, gd, sd, m, n)
    torch.cuda.synchronize()
    got = out.cpu().numpy().tobytes()
    want = b"".join(g1.to_bytes(p) for p in g1.pedersen_commit(gens, rows))
    assert got == want


@pytest.mark.gpu
@pytest.mark.parametrize("m,n", [(4, 64), (32, 256)])
def test_kernels_match_reference_kernels(zk, prover, m, n):
    import os
    import torch
    import fr_oracle as fo
    if not fo.ReferenceFr.available():
        pytest.skip("oracle/_ref/libfrref.so not built")
    lib = fo.ReferenceFr().lib
    if not hasattr(lib, "refA_pedersen_commit") or not lib.refA_gpu_available():
        pytest.skip("reference build without the commitment entry points, or no GPU")
    gens = (C.c_uint8 * (n * 144))()
    assert lib.refA_commit_random(C.c_uint32(n), gens) == 0
    rnd = random.Random(5)
    sc = _pack_scalars(_scalars(rnd, m, n))
    want = (C.c_uint8 * (m * 144))()
    assert lib.refA_pedersen_commit(gens, C.c_uint32(n), sc.ctypes.data_as(C.c_void_p), C.c_uint32(m), want, None) == 0
    gd = torch.from_numpy(np.frombuffer(bytes(gens), dtype=np.uint8).copy()).cuda()
    sd = torch.from_numpy(sc.view(np.int32)).cuda()
    out = zk.fr.g1_pedersen_commit(prover, gd, sd, m, n)
    torch.cuda.synchronize()
    assert out.cpu().numpy().tobytes() == bytes(want)
