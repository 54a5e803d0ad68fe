"""World-size-2 (and 4) gloo runs of the sharded-sumcheck host logic on CPU.

The per-GPU engine is replaced by a stand-in built on the oracle (test infrastructure), so
what is exercised here is the orchestration in zk_hillclimb_b200.p3.sc_prove_sharded:
slice ownership, the per-round all-gather order, the residual rounds and the transcript.
The result must equal the oracle's unsharded proof on the concatenated columns."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GL_P = 0xFFFFFFFF00000001


class OracleShardEngine:
    """CPU stand-in for Prover's shard_* interface (small sizes; plain Python integers)."""

    def __init__(self, orc):
        self.orc = orc

    def new_buffer(self, n):
        import torch
        return torch.zeros(n, dtype=torch.int64)

    @staticmethod
    def _F(functor, c, par):
        if functor == 0:
            return c[0] * c[1] % GL_P
        if functor == 1:
            return c[0] * c[1] * c[2] % GL_P
        if functor == 2:
            return c[0] * (c[1] * c[4] + c[2] * c[3] + par[0] * c[3] * c[4]) % GL_P
        return (par[0] * c[0] + c[2] * (c[0] * (c[1] + par[1]) - c[3])) % GL_P

    def shard_begin(self, functor, nt, dcols, logn, par, tag, state):
        self.functor, self.nt, self.par, self.tag = functor, nt, [int(x) for x in par], tag
        self.cols = [[int(x) for x in t.numpy().view(np.uint64)] for t in dcols]
        self.st, self.msgs, self.chals = state, [], []

    def shard_round_local(self, r, sums):
        if r > 0:
            a = self.chals[r - 1]
            self.cols = [[(c[2 * i] + a * (c[2 * i + 1] - c[2 * i])) % GL_P for i in range(len(c) // 2)] for c in self.cols]
        s = [0] * self.nt
        for i in range(len(self.cols[0]) // 2):
            lo = [c[2 * i] for c in self.cols]
            dd = [(c[2 * i + 1] - c[2 * i]) % GL_P for c in self.cols]
            for t in range(self.nt):
                s[t] = (s[t] + self._F(self.functor, [(l + t * d) % GL_P for l, d in zip(lo, dd)], self.par)) % GL_P
        sums.copy_(__import__("torch").from_numpy(np.array(s, dtype=np.uint64).view(np.int64)))

    def shard_round_combine(self, r, gathered, G):
        g = gathered.numpy().view(np.uint64).reshape(G, self.nt)
        m = [int(sum(int(x) for x in g[:, t]) % GL_P) for t in range(self.nt)]
        self.msgs.append(m)
        self.st = self.orc.tr_absorb(self.st, self.tag, np.array(m, dtype=np.uint64).tobytes())
        self.st, a = self.orc.tr_chal(self.st)
        self.chals.append(a)

    def shard_finals(self, fin):
        a = self.chals[-1]
        v = [(c[0] + a * (c[1] - c[0])) % GL_P for c in self.cols]
        fin.copy_(__import__("torch").from_numpy(np.array(v, dtype=np.uint64).view(np.int64)))

    def shard_residual(self, gfin, G):
        nc = len(self.cols)
        g = gfin.numpy().view(np.uint64).reshape(G, nc)
        cols = [np.ascontiguousarray(g[:, k]) for k in range(nc)]
        if G == 1:
            self.finals = np.array([int(c[0]) for c in cols], dtype=np.uint64)
            return
        self.st, m, r, fin = self.orc.sumcheck(self.st, self.tag, self.functor, self.nt, cols, self.par)
        self.msgs += [[int(x) for x in row] for row in m]
        self.chals += [int(x) for x in r]
        self.finals = fin

    def shard_end(self, rounds):
        assert rounds == len(self.chals)
        return self.st, np.array(self.msgs, dtype=np.uint64), np.array(self.chals, dtype=np.uint64), self.finals


def _worker(rank, world, port, functor, nt, logn_total, par, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import torch
    import torch.distributed as dist
    import zkh_import
    from oracle import Oracle
    zk = zkh_import.load()
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    orc = Oracle()
    nc = zk.p3.FUNCTOR_NC[functor]
    n = 1 << logn_total
    cols, s = [], 4321
    for _ in range(nc):
        a, s = orc.lcg(n, s)
        cols.append(a)
    per = n // world
    mine = [torch.from_numpy(c[rank * per:(rank + 1) * per].copy().view(np.int64)) for c in cols]
    tr = zk.Transcript("sharded")
    r, m, fin = zk.p3.sc_prove_sharded(OracleShardEngine(orc), tr, "sc", mine, functor, nt, dist, par)
    st1, m0, r0, f0 = orc.sumcheck(orc.tr_init("sharded"), "sc", functor, nt, cols, par)
    ok = bool((m == m0).all() and (r == r0).all() and (fin == f0).all() and tr.state == st1)
    q.put((rank, ok))
    dist.barrier()
    dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world,functor,nt,par", [(2, 0, 3, []), (2, 3, 4, [11, 13]), (4, 1, 4, [])])
def test_sharded_sumcheck_equals_unsharded(world, functor, nt, par):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, functor, nt, 7, par, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    assert sorted(res) == [(r, True) for r in range(world)]


def test_single_rank_path_is_the_plain_proof(orc, zk):
    import torch
    cols = []
    s = 99
    for _ in range(2):
        a, s = orc.lcg(1 << 5, s)
        cols.append(a)
    tr = zk.Transcript("one")
    r, m, fin = zk.p3.sc_prove_sharded(OracleShardEngine(orc), tr, "sc",
                                       [torch.from_numpy(c.view(np.int64)) for c in cols], 0, 3, None)
    st1, m0, r0, f0 = orc.sumcheck(orc.tr_init("one"), "sc", 0, 3, cols)
    assert (m == m0).all() and (r == r0).all() and (fin == f0).all() and tr.state == st1


def _commit_worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch.distributed as dist
    import zkh_import
    from lu_helpers import OracleLookupEngine, _Arr
    from oracle import Oracle
    zk = zkh_import.load()
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    orc = Oracle()
    eng = OracleLookupEngine(orc)
    K, s = 5, 17
    cols = []
    for j in range(K):
        a, s = orc.lcg(1 << (3 + j % 3), s)
        cols.append(a)
    mine = [_Arr(c) if j % world == rank else None for j, c in enumerate(cols)]      # only owned columns are resident
    roots = zk.p3.commit_columns_sharded(eng, mine, 1, dist)
    want = [orc.merkle_root(orc.rs_encode(c, 1)) for c in cols]
    sizes = zk.p3.run_independent(list(range(7)), lambda i: (i, rank, i * i), dist)
    # lookup multiplicities from index arrays split over the ranks
    import numpy as np
    import torch

    class _TorchHist:
        def histogram(self, idx, M):
            return torch.bincount(idx.to(torch.int64), minlength=M)
    allidx = np.random.default_rng(3).integers(0, 64, 1000).astype(np.int32)
    part = torch.from_numpy(allidx[rank::world].copy())
    cnt = zk.p3.lu_counts_sharded(_TorchHist(), [part], 64, 5, dist)
    wantc = np.bincount(allidx, minlength=64)
    wantc[0] += 5
    roots_ok = (cnt.numpy() == wantc).all()
    ok = roots_ok and roots == want and [x[0] for x in sizes] == list(range(7)) and all(x[1] == x[0] % world for x in sizes)
    q.put((rank, bool(ok)))
    dist.barrier()
    dist.destroy_process_group()


def test_column_sharded_commitments_and_independent_proofs():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_commit_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(2)]
    for p in procs:
        p.join(timeout=60)
    assert sorted(res) == [(0, True), (1, True)]


def test_column_sharded_commitments_single_rank(orc, zk):
    from lu_helpers import OracleLookupEngine, _Arr
    cols = [orc.lcg(8, 5 + j)[0] for j in range(3)]
    roots = zk.p3.commit_columns_sharded(OracleLookupEngine(orc), [_Arr(c) for c in cols], 1)
    assert roots == [orc.merkle_root(orc.rs_encode(c, 1)) for c in cols]
    assert zk.p3.run_independent([3, 4], lambda x: x + 1) == [4, 5]
