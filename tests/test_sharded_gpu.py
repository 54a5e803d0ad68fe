"""The sharded sumcheck on GPU: G ranks emulated as G contexts on one device (no kernel waits on
another, so this is safe on a single GPU), and -- where two GPUs are visible -- real NCCL ranks."""
import os
import socket
import sys

import numpy as np
import pytest

from conftest import lcg_cols

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("G", [1, 2, 4])
@pytest.mark.parametrize("functor,nt,par,logn", [(0, 3, [], 15), (1, 4, [], 13), (3, 4, [5, 9], 14), (2, 4, [77], 6), (0, 3, [], 3)])
def test_emulated_ranks_equal_unsharded(orc, zk, G, functor, nt, par, logn):
    import torch
    nc = zk.p3.FUNCTOR_NC[functor]
    cols = lcg_cols(orc, 1 << logn, nc, 2468 + logn)
    st1, m0, r0, f0 = orc.sumcheck(orc.tr_init("emu"), "sc", functor, nt, cols, par, nthreads=4)
    per = (1 << logn) // G
    stream = torch.cuda.current_stream().cuda_stream
    engines = [zk.Prover(0, stream) for _ in range(G)]
    slices = [[zk.p3.to_device(c[g * per:(g + 1) * per].copy()) for c in cols] for g in range(G)]
    st0 = zk.Transcript("emu").state
    for e, sl in zip(engines, slices):
        e.shard_begin(functor, nt, sl, logn - (G.bit_length() - 1), par, "sc", st0)
    sums = [e.new_buffer(nt) for e in engines]
    for r in range(logn - (G.bit_length() - 1)):
        for e, s in zip(engines, sums):
            e.shard_round_local(r, s)
        gathered = torch.cat(sums)            # what the all-gather delivers to every rank
        for e in engines:
            e.shard_round_combine(r, gathered, G)
    fins = [e.new_buffer(nc) for e in engines]
    for e, f in zip(engines, fins):
        e.shard_finals(f)
    gfin = torch.cat(fins)
    for e in engines:
        e.shard_residual(gfin, G)
    for e in engines:
        st, m, r, fin = e.shard_end(logn)
        assert (m == m0).all() and (r == r0).all() and (fin == f0).all() and st == st1
        e.close()


def test_sharded_api_order_errors(orc, zk, prover):
    cols = [zk.p3.to_device(c) for c in lcg_cols(orc, 16, 2, 1)]
    prover.shard_begin(0, 3, cols, 4, [], "sc", zk.Transcript("x").state)
    buf = prover.new_buffer(3)
    with pytest.raises(zk.ZkhError):
        prover.shard_round_local(1, buf)        # round 0 has not run
    with pytest.raises(zk.ZkhError):
        prover.shard_finals(buf)                # local rounds unfinished
    prover.shard_round_local(0, buf)
    with pytest.raises(zk.ZkhError):
        prover.shard_round_combine(1, buf, 1)   # wrong round
    prover.shard_end(0)


def _worker(rank, world, port, logn_total, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch
    import torch.distributed as dist
    import zkh_import
    from oracle import Oracle
    zk = zkh_import.load()
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    orc = Oracle()
    ok = True
    for functor, nt, par, logn_total in [(0, 3, [], logn_total), (1, 4, [], logn_total), (3, 4, [5, 9], 8), (1, 4, [], 13)]:
        nc = zk.p3.FUNCTOR_NC[functor]
        cols, s = [], 97531
        for _ in range(nc):
            a, s = orc.lcg(1 << logn_total, s)
            cols.append(a)
        per = (1 << logn_total) // world
        mine = [zk.p3.to_device(c[rank * per:(rank + 1) * per].copy(), "cuda:%d" % rank) for c in cols]
        prover = zk.Prover(rank, torch.cuda.current_stream().cuda_stream)
        tr = zk.Transcript("nccl")
        r, m, fin = zk.p3.sc_prove_sharded(prover, tr, "sc", mine, functor, nt, dist, par)
        st1, m0, r0, f0 = orc.sumcheck(orc.tr_init("nccl"), "sc", functor, nt, cols, par, nthreads=4)
        ok &= bool((m == m0).all() and (r == r0).all() and (fin == f0).all() and tr.state == st1)
        # the same proof with every round as one kernel: sums cross NVLink as peer stores, no NCCL per round
        if prover.p2p_connect(dist):
            for rep in range(2):               # two proofs back to back: the exchange sequence carries over
                tr = zk.Transcript("nccl")
                r, m, fin = zk.p3.sc_prove_sharded(prover, tr, "sc", mine, functor, nt, dist, par)
                ok &= bool((m == m0).all() and (r == r0).all() and (fin == f0).all() and tr.state == st1)
            if functor == 0 and logn_total > 13:
                # a rank that never arrives: the wait of the others runs out (about a second) and the call
                # reports a device error instead of hanging; after reconnecting, proofs work again
                dist.barrier()
                if rank == 0:
                    prover.shard_begin(functor, nt, mine, logn_total - (world.bit_length() - 1), par, "sc",
                                       zk.Transcript("nccl").state)
                    prover.shard_round_fused(0)
                    try:
                        prover.shard_end(1)
                        ok = False
                    except zk.ZkhError as e:
                        ok &= e.code == -6
                dist.barrier()
                prover.p2p_disconnect()
                dist.barrier()
                ok &= bool(prover.p2p_connect(dist))
                tr = zk.Transcript("nccl")
                r, m, fin = zk.p3.sc_prove_sharded(prover, tr, "sc", mine, functor, nt, dist, par)
                ok &= bool((m == m0).all() and (r == r0).all() and (fin == f0).all() and tr.state == st1)
                # a rank that arrives after the others' waits ran out: the others flag their later exchanges, so the
                # late rank learns of it and EVERY rank reports the device error (no rank returns a proof built
                # from sums the others never used)
                dist.barrier()
                if rank == world - 1:
                    import time
                    time.sleep(6.0)
                try:
                    zk.p3.sc_prove_sharded(prover, zk.Transcript("nccl"), "sc", mine, functor, nt, dist, par, rendezvous=False)
                    ok = False
                except zk.ZkhError as e:
                    ok &= e.code == -6
                dist.barrier()
                prover.p2p_disconnect()
                dist.barrier()
                ok &= bool(prover.p2p_connect(dist))
                for rep in range(3):           # back to back without the host rendezvous: only kernel skew between ranks
                    tr = zk.Transcript("nccl")
                    r, m, fin = zk.p3.sc_prove_sharded(prover, tr, "sc", mine, functor, nt, dist, par, rendezvous=(rep == 0))
                    ok &= bool((m == m0).all() and (r == r0).all() and (fin == f0).all() and tr.state == st1)
            dist.barrier()
            prover.p2p_disconnect()
        dist.barrier()
        prover.close()
    q.put((rank, ok))
    dist.barrier()
    dist.destroy_process_group()


def test_nccl_ranks_equal_unsharded():
    import torch
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    world = 2 if world < 4 else 4
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = [ctx.Process(target=_worker, args=(r, world, port, 18, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    assert sorted(res) == [(r, True) for r in range(world)]
