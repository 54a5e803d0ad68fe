"""Hiding mode ("zk=1") of the p3 stack: host-side mirror of the reference's p3zkc mechanisms over the CUDA library.

  ZkCtx                  p3zkc::Ctx / next_seed / e_of / vfull      zkllm-src/p3_zkc.cuh:83-137
  zpt / xpt / expt       claim-point helpers                        zkllm-src/p3_zkc.cuh:183-208
  commit_col             p3lu::commit_col_nc, zk branch             zkllm-src/p3_logup.cuh:335-360
  slice1 / mk_linked     seam mask linkage                          zkllm-src/p3_zkc.cuh:408-422
  ZLedger / claimc       p3bo::PLedger with salt seeds, p3hwl::claimc   p3_batchopen.cuh:144-178, p3_hawkeye.cuh:801-838
  sc5z                   Libra-blinded quartic sumcheck             zkllm-src/p3_hawkeye.cuh:1035-1351
  prove_class / tail_prove   class blinder + salted openings        zkllm-src/p3_batchopen.cuh:315-384, :969-1131
  imm_prove              p3imm::prove with the zk switch on         zkllm-src/p3_int_gadgets.cuh:510-605

Every random draw follows the reference's order (one counter-mode seed per draw, zkllm-src/p3_zkc.cuh:118-123), so with
the same master seed the proofs are the reference prover's bytes.  The device work is the library's: mask and blind
columns are generated on the GPU (zkh_zk_fill_chain), commitments are salted (zkh_basefold_commit_salted), the blinded
chain is one programmable zero-check whose blind terms ride as extra columns (zkh_sumcheck_zerocheck), the openings
are zkh_batchopen_prove_class_salted.  Structured blinds (chains of 2^22 points and more) add a per-round message
term that the library applies on the device (zkh_sumcheck_zerocheck_blind).

Serialised forms (little endian):
  Blind      u32 nb | nb == 5: four roots, else one root | H | nb == 6: ystar, else yB[4] |
             nb == 6: u32 rounds, rounds * 24 bytes inner-product messages, yw
  BatchProof the plain layout with a 32-byte salt per opened value after each column's values, then blinder root (32)
             and blinder claim (8) at the end
  imm proof  u32 lj, lk, li | messages vfull(lj+lk+li) * 40 | yY yX yW | Blind | u32 batches, each u32 length + BatchProof
"""
import struct

import numpy as np

from .p3 import GL_P, Ledger

M64 = (1 << 64) - 1
GOLD = 0x9E3779B97F4A7C15


class ZkCtx:
    """p3zkc::Ctx with the switch on: master seed, draw counter, query budget, structured-blind threshold."""

    def __init__(self, seed=1, Q=24, sblind_min=22):
        self.seed, self.ctr, self.Q, self.sblind_min = seed & M64, 0, Q, sblind_min

    def next_seed(self):
        """zkllm-src/p3_zkc.cuh:118-123."""
        self.ctr += 1
        self.seed = (self.seed + GOLD * self.ctr) & M64
        z = self.seed
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M64
        return z ^ (z >> 31)

    def zkb(self):
        return 4 * (2 * self.Q + 64)

    def e_of(self, v):
        """Number of extra (mask) variables of a column of 2^v real entries: zkllm-src/p3_zkc.cuh:130-136."""
        e = 1
        while (1 << v) * ((1 << e) - 1) < self.zkb():
            e += 1
        return e

    def vfull(self, v):
        return v + self.e_of(v)


def zpt(zc, z):
    """Zero-extended point: weighs the real slice only."""
    return list(z) + [0] * zc.e_of(len(z))


def xpt(zc, z, zex):
    """Hiding claim point (z | zex | 0...): real slice and mask slice 1."""
    return list(z) + [zex] + [0] * (zc.e_of(len(z)) - 1)


def expt(zc, zlow, rfull, src_v):
    """Map the extra coordinates of a full sumcheck point onto a target of another extra-variable count."""
    return list(zlow) + [int(rfull[src_v + i]) if src_v + i < len(rfull) else 0 for i in range(zc.e_of(len(zlow)))]


class ZCol:
    """A committed hiding column: augmented values [real | mask slices], salted root, salt seed."""

    def __init__(self, dev, root, vreal, sseed, cw=None, tree=None):
        self.dev, self.root, self.vreal, self.sseed, self.cw, self.tree = dev, root, vreal, sseed, cw, tree


def _salted(engine, aug, R, sseed, keep):
    if keep:
        root, cw, tree = engine.commit_salted(aug, R, sseed, keep=True)
        return root, cw, tree
    return engine.commit_salted(aug, R, sseed), None, None


def commit_col(engine, zc, vals, R, mask=None, keep=False):
    """p3lu::commit_col_nc with the switch on: a fresh mask (seed drawn first) unless a linked mask is given, then the
    salt seed, then the salted commitment of [vals | mask]."""
    v = int(vals.numel()).bit_length() - 1
    if mask is None:
        aug = engine.zk_augment(vals, zc.e_of(v), zc.next_seed())
    else:
        aug = engine.concat([vals, mask])
    sseed = zc.next_seed()
    root, cw, tree = _salted(engine, aug, R, sseed, keep)
    return ZCol(aug, root, v, sseed, cw, tree)


def slice1(engine, col):
    """The first mask slice of a committed column."""
    n = 1 << col.vreal
    return engine.slice(col.dev, n, n)


def mk_linked(engine, zc, vc, cons1):
    """Consumer mask whose slice 1 is cons1 and whose higher slices are fresh; the seed is drawn even when there are none."""
    n, e = 1 << vc, zc.e_of(vc)
    s = zc.next_seed()
    if e == 1:
        return cons1
    return engine.concat([cons1, engine.zk_fill_chain(s, n * ((1 << e) - 2))])


class ZLedger(Ledger):
    """Opening claims of hiding columns: the entries carry the salt seed and, where kept, codeword and tree."""

    def add(self, col, z, y):
        Ledger.add(self, col.dev, col.root, z, y)
        c = next(c for c in self.cls if c[0] == len(z))
        c[2][-1] = c[2][-1] + (col.sseed, col.cw, col.tree)


def claimc(engine, tr, ledger, col, z):
    """p3hwl::claimc on an augmented column."""
    y = engine.eval_h_gpu(col.dev, np.ascontiguousarray([int(x) for x in z], dtype=np.uint64))
    tr.absorb("hwl-y", struct.pack("<Q", y))
    ledger.add(col, z, y)
    return y


def prove_class(engine, zc, tr, cls, R, Q, label):
    """p3bo::prove_class with the switch on: append the class blinder (uniform column, salted commitment, claim at a fresh
    point), then the salted batched opening.  cls: one ZLedger class."""
    v, pts, ents = cls[0], list(cls[1]), list(cls[2])
    s = zc.next_seed()
    blv = engine.zk_fill_chain(s, 1 << v)
    blseed = zc.next_seed()
    root, cw, tree = _salted(engine, blv, R, blseed, False)
    tr.absorb("bo-blr", root)
    zD = np.array([tr.chal() for _ in range(v)], dtype=np.uint64)
    bl_y = engine.eval_h_gpu(blv, zD)
    tr.absorb("bo-bly", struct.pack("<Q", bl_y))
    ents.append((blv, root, len(pts), blseed, cw, tree))
    pts.append(zD)
    body = engine.prove_class_salted(tr, np.stack(pts), ents, R, Q, label)
    return body + root + struct.pack("<Q", bl_y)


def tail_prove(engine, zc, tr, ledger, R, Q, tag):
    """p3ig::tail_prove without deferred lookups."""
    return [prove_class(engine, zc, tr, c, R, Q, "%s%d" % (tag, i)) for i, c in enumerate(ledger.cls)]


def sc5z(engine, zc, tr, tag, vreal, cols, terms, konst, R, ledger):
    """p3hwl::sc5z: the sumcheck of cols[0] * (konst + sum terms) over 2^vfull(vreal) points, blinded by four committed
    uniform columns B1..B4 through rho * (B1 + E B2 + E^2 B3 + E^3 B4), E = cols[0].  Merged layout (one commitment of
    the four, one claim at (r | t0 | t1)) up to 2^24 points, four commitments above.  Returns (r, msgs, finals of cols,
    serialised Blind)."""
    from .p3 import col_sum
    v = zc.vfull(vreal)
    N = 1 << v
    if int(cols[0].numel()) != N:
        raise ValueError("sc5z: columns must cover the augmented domain")
    if v >= zc.sblind_min:
        return _sc5z_structured(engine, zc, tr, tag, v, cols, terms, konst, R, ledger)
    merged = v + 2 <= 26
    bseed = [zc.next_seed() for _ in range(4)]
    B = [engine.zk_fill_chain(s, N) for s in bseed]
    if merged:
        mb = engine.concat(B)
        ss = zc.next_seed()
        MB = ZCol(mb, engine.commit_salted(mb, R, ss), v + 2, ss)
        tr.absorb("sc5-bl", MB.root)
        roots = [MB.root]
    else:
        Bc = []
        for j in range(4):
            ss = zc.next_seed()
            Bc.append(ZCol(B[j], engine.commit_salted(B[j], R, ss), v, ss))
            tr.absorb("sc5-bl", Bc[j].root)
        roots = [c.root for c in Bc]
    E = cols[0]
    E2 = engine.mul(E, E)
    H = (col_sum(engine, B[0]) + col_sum(engine, engine.mul(E, B[1])) + col_sum(engine, engine.mul(E2, B[2]))
         + col_sum(engine, engine.mul(engine.mul(E2, E), B[3]))) % GL_P
    tr.absorb("sc5-H", struct.pack("<Q", H))
    rho = tr.chal()
    i0 = len(cols)
    blind_terms = [(rho, (i0,), True), (rho, (i0 + 1,)), (rho, (0, i0 + 2)), (rho, (0, 0, i0 + 3))]
    r, msgs, fin = engine.sc_prove_zc(tr, tag, list(cols) + B, list(terms) + blind_terms, konst)
    r = [int(x) for x in r]
    yB = [int(fin[i0 + j]) for j in range(4)]
    for y in yB:
        tr.absorb("sc5-yB", struct.pack("<Q", y))
    if merged:
        t0, t1 = tr.chal(), tr.chal()
        y01 = (yB[0] + t0 * (yB[1] - yB[0])) % GL_P
        y23 = (yB[2] + t0 * (yB[3] - yB[2])) % GL_P
        ystar = (y01 + t1 * (y23 - y01)) % GL_P
        ledger.add(MB, r + [t0, t1], ystar)
    else:
        for j in range(4):
            ledger.add(Bc[j], r, yB[j])
    blind = struct.pack("<I", 4 if merged else 5) + b"".join(roots) + struct.pack("<Q", H) + struct.pack("<4Q", *yB)
    return r, msgs, fin[:i0], blind


def _geval(c, t):
    acc = 0
    for k in range(4, -1, -1):
        acc = (acc * t + c[k]) % GL_P
    return acc


def _sc5z_structured(engine, zc, tr, tag, v, cols, terms, konst, R, ledger):
    """Structured blind g(x) = sum_j g_j(x_j), g_j uniform of degree 4 (zkllm-src/p3_hawkeye.cuh:1065-1139, :1172-1216): one
    small committed coefficient column, a per-round additive term on the messages, and an inner-product sumcheck that
    binds g(r) to the commitment."""
    u = 8
    while (1 << u) < 5 * v + 64:
        u += 1
    s = zc.next_seed()
    w = engine.zk_fill_chain(s, 1 << u)                    # the first 5v draws are the coefficients, the rest is slack
    wh = engine.download(w)
    sc = [[int(wh[5 * j + k]) for k in range(5)] for j in range(v)]
    W = commit_col(engine, zc, w, R)
    tr.absorb("sc5-bl", W.root)
    suf = [0] * (v + 1)
    for j in range(v - 1, -1, -1):
        suf[j] = (suf[j + 1] + _geval(sc[j], 0) + _geval(sc[j], 1)) % GL_P
    H = pow(2, v - 1, GL_P) * suf[0] % GL_P
    tr.absorb("sc5-H", struct.pack("<Q", H))
    rho = tr.chal()
    table = [sc[rd] + [rho * pow(2, v - 1 - rd, GL_P) % GL_P,
                       rho * pow(2, v - 2 - rd, GL_P) % GL_P * suf[rd + 1] % GL_P if rd + 1 < v else 0] for rd in range(v)]
    r, msgs, fin, ystar = engine.sc_prove_zc_blind(tr, tag, list(cols), list(terms), konst, table)
    r = [int(x) for x in r]
    tr.absorb("sc5-yB", struct.pack("<Q", ystar))
    # inner product of the augmented coefficient column with Phi[5j + k] = r_j^k
    uf = zc.vfull(u)
    phi = np.zeros(1 << uf, dtype=np.uint64)
    for j in range(v):
        p = 1
        for k in range(5):
            phi[5 * j + k] = p
            p = p * r[j] % GL_P
    from .p3 import F_PROD2
    rip, ipm, ipf = engine.sc_prove_gpu(tr, "sc5-ip", [W.dev, engine.upload(phi)], F_PROD2, 3)
    yw = int(ipf[0])
    tr.absorb("sc5-yw", struct.pack("<Q", yw))
    ledger.add(W, [int(x) for x in rip], yw)
    blind = struct.pack("<I", 6) + W.root + struct.pack("<QQ", H, ystar) + struct.pack("<I", uf) + \
        np.ascontiguousarray(ipm, dtype=np.uint64).tobytes() + struct.pack("<Q", yw)
    return r, msgs, fin, blind


def linked_y_mask(engine, zc, X, W, lj, lk, li):
    """p3imm::accum_mask1 + mk_linked for the direct layouts: slice 1 of Y's mask is the product of the operands' first mask
    slices (zkllm-src/p3_int_gadgets.cuh:510-527), the higher slices are fresh."""
    J, K, I = 1 << lj, 1 << lk, 1 << li
    xm, wm = slice1(engine, X), slice1(engine, W)
    rows = [engine.matvec(wm, J, K, engine.slice(xm, i * J, J), False) for i in range(I)]
    return mk_linked(engine, zc, lk + li, engine.concat(rows))


def imm_prove(engine, zc, tr, X, W, Y, lj, lk, li, R, Q, ledger=None):
    """p3imm::prove with the zk switch on, direct layouts X = [j | i<<lj], W = [k | j<<lk], Y = [k | i<<lk] (ZCol each; Y
    committed with linked_y_mask).  The summand eq * X * W runs over the (j, k, i, ex) domain of 2^vfull(lj+lk+li) points
    as one blinded chain."""
    own = ledger is None
    if own:
        ledger = ZLedger()
    tr.absorb("imm-dims", struct.pack("<III", lj, lk, li))
    tr.absorb("imm-X", X.root)
    tr.absorb("imm-W", W.root)
    tr.absorb("imm-Y", Y.root)
    z = [tr.chal() for _ in range(lk + li)]
    zex = tr.chal()
    yY = claimc(engine, tr, ledger, Y, xpt(zc, z, zex))
    lt = lj + lk + li
    e_p, eX, eW = zc.e_of(lt), zc.e_of(lj + li), zc.e_of(lj + lk)
    N = 1 << (lt + e_p)
    ptE = z + [zex] + [0] * (e_p - 1)
    eqv = engine.build_eq_gpu(np.array(ptE, dtype=np.uint64))
    J, K, I = 1 << lj, 1 << lk, 1 << li
    mX = (1 << min(eX, e_p)) - 1
    mW = (1 << min(eW, e_p)) - 1
    cols = [engine.bcast_rows(eqv, lj),
            engine.gather_fn(X.dev, N, lambda u: (u & (J - 1)) | (((u >> (lj + lk)) & (I - 1)) << lj) | (((u >> lt) & mX) << (lj + li))),
            engine.gather_fn(W.dev, N, lambda u: ((u >> lj) & (K - 1)) | ((u & (J - 1)) << lk) | (((u >> lt) & mW) << (lj + lk)))]
    r, msgs, _, blind = sc5z(engine, zc, tr, "imm-sc", lt, cols, [(1, (1, 2))], 0, R, ledger)
    rj, rk, ri = r[:lj], r[lj:lj + lk], r[lj + lk:lt]
    yX = claimc(engine, tr, ledger, X, expt(zc, rj + ri, r, lt))
    yW = claimc(engine, tr, ledger, W, expt(zc, rk + rj, r, lt))
    out = struct.pack("<III", lj, lk, li) + np.ascontiguousarray(msgs, dtype=np.uint64).tobytes()
    out += struct.pack("<QQQ", yY, yX, yW) + blind
    batches = tail_prove(engine, zc, tr, ledger, R, Q, "imm-bo") if own else []
    out += struct.pack("<I", len(batches)) + b"".join(struct.pack("<I", len(b)) + b for b in batches)
    return out
