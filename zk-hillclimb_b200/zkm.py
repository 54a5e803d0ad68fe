"""Hiding mode ("zk=1") of the p3 stack: host-side mirror of the reference's p3zkc mechanisms over the CUDA library.

  ZkCtx                  p3zkc::Ctx / next_seed / e_of / vfull      zkllm-src/p3_zkc.cuh:83-137
  zpt / xpt / expt       claim-point helpers                        zkllm-src/p3_zkc.cuh:183-208
  commit_col             p3lu::commit_col_nc, zk branch             zkllm-src/p3_logup.cuh:335-360
  slice1 / mk_linked     seam mask linkage                          zkllm-src/p3_zkc.cuh:408-422
  ZLedger / claimc       p3bo::PLedger with salt seeds, p3hwl::claimc   p3_batchopen.cuh:144-178, p3_hawkeye.cuh:801-838
  sc5z                   Libra-blinded quartic sumcheck             zkllm-src/p3_hawkeye.cuh:1035-1351
  prove_class / tail_prove   class blinder + salted openings        zkllm-src/p3_batchopen.cuh:315-384, :969-1131
  imm_prove              p3imm::prove with the zk switch on         zkllm-src/p3_int_gadgets.cuh:510-605
  prove_super / lu_flush p3lu::prove_super / lu_flush, zk branches  zkllm-src/p3_logup.cuh:1357-1956
  irs_prove / iadd_prove / iswg_prove   p3irs / p3iadd / p3iswg::prove with the zk switch on   p3_int_gadgets.cuh:282-340, :712-737, :1790-1832
  irope_prove / irms_prove / ismx_prove p3irope / p3irms / p3ismx::prove with the zk switch on p3_int_gadgets.cuh:1275-1322, :918-1047, :1514-1643
  linked_acc_mask / itf_commit_all / imm_prove_views / itf_prove   p3itf::commit_acc, commit_all, prove with the zk switch on   zkllm-src/p3_int_layer.cuh:331-415, :452-581

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

    def __init__(self, seed=1, Q=24, sblind_min=22, keep_bytes=0):
        self.seed, self.ctr, self.Q, self.sblind_min = seed & M64, 0, Q, sblind_min
        self.keep_bytes = keep_bytes          # HBM the prover may spend on codewords and salted trees kept for the openings

    def take(self, v, R):
        """Reserve room for the codeword and the capped tree (levels from 64 leaves per node upwards: one byte per codeword
        element) of a column of 2^v entries; False when the budget is spent."""
        need = (8 + (1 if v + R >= 8 else 64)) << (v + R)
        if need > self.keep_bytes:
            return False
        self.keep_bytes -= need
        return True

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
    root, cw, tree = _salted(engine, aug, R, sseed, keep or zc.take(int(aug.numel()).bit_length() - 1, R))
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


def _sblind_begin(engine, zc, tr, v, R):
    """Structured blind g(x) = sum_j g_j(x_j), g_j uniform of degree 4, for a chain of v rounds (zkllm-src/p3_hawkeye.cuh:
    1065-1139): commits the coefficient column, absorbs its root and H, draws rho.  Returns the state the chain and the closing
    step need; "table" holds per round the coefficients of g_rd, A_rd = rho 2^(v-1-rd), B_rd = rho 2^(v-2-rd) suf[rd+1]."""
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
    return {"v": v, "u": u, "W": W, "H": H, "table": table}


def _sblind_end(engine, zc, tr, sb, r, ystar, ledger):
    """Closing step of a structured-blind chain (zkllm-src/p3_hawkeye.cuh:1172-1216): g(r) is absorbed and bound to the committed
    coefficient column by the inner-product sumcheck with Phi[5j + k] = r_j^k.  Returns the serialised Blind."""
    from .p3 import F_PROD2
    v, W = sb["v"], sb["W"]
    tr.absorb("sc5-yB", struct.pack("<Q", ystar))
    uf = zc.vfull(sb["u"])
    phi = np.zeros(1 << uf, dtype=np.uint64)
    for j in range(v):
        p = 1
        for k in range(5):
            phi[5 * j + k] = p
            p = p * r[j] % GL_P
    rip, ipm, ipf = engine.sc_prove_gpu(tr, "sc5-ip", [W.dev, engine.upload(phi)], F_PROD2, 3)
    yw = int(ipf[0])
    tr.absorb("sc5-yw", struct.pack("<Q", yw))
    ledger.add(W, [int(x) for x in rip], yw)
    return struct.pack("<I", 6) + W.root + struct.pack("<QQ", sb["H"], ystar) + struct.pack("<I", uf) + \
        np.ascontiguousarray(ipm, dtype=np.uint64).tobytes() + struct.pack("<Q", yw)


def _sc5z_structured(engine, zc, tr, tag, v, cols, terms, konst, R, ledger):
    """The whole chain under a structured blind: the per-round term is added to the messages on the device."""
    sb = _sblind_begin(engine, zc, tr, v, R)
    r, msgs, fin, ystar = engine.sc_prove_zc_blind(tr, tag, list(cols), list(terms), konst, sb["table"])
    r = [int(x) for x in r]
    return r, msgs, fin, _sblind_end(engine, zc, tr, sb, r, ystar, ledger)


def imm_chain_factored(engine, zc, tr, X, W, views, lj, lk, li, z, zex, R, ledger):
    """The matmul chain of p3imm under a structured blind WITHOUT the 2^(lj+lk+li+e) product domain.  The summand
    eq(z, zex; k, i, ex) X(j, i, ex) W(j, k, ex) splits over the index groups, and a structured blind only adds a public
    per-round term to the messages, so the rounds over j, over k and over i are three short product chains on partially
    evaluated operands (the two slices ex = 0, 1 the weight touches, stacked and pre-weighted), stopped before the slice
    variable, and the last e rounds run over the slice variable alone.  Messages, challenges and transcript equal the chain
    over the materialised domain (zkllm-src/p3_int_gadgets.cuh:567-597 with p3_hawkeye.cuh:1329-1331).
    Returns (r, msgs as bytes, serialised Blind)."""
    from .p3 import S_A, S_J, view_point
    xv, wv, _ = views
    lt = lj + lk + li
    e_p, eX, eW = zc.e_of(lt), zc.e_of(X.vreal), zc.e_of(W.vreal)
    J, K, I = 1 << lj, 1 << lk, 1 << li
    mX, mW = (1 << min(eX, e_p)) - 1, (1 << min(eW, e_p)) - 1
    sb = _sblind_begin(engine, zc, tr, lt + e_p, R)
    table, pref = sb["table"], 0
    zk_, zi_ = z[:lk], z[lk:]
    ws = [(1 - zex) % GL_P, zex % GL_P]
    u64 = lambda a: np.array(a, dtype=np.uint64)
    Xd = [engine.gather_fn(X.dev, I * J, lambda t, s=s: _view_index(xv, {S_J: t & (J - 1), S_A: t >> lj}) | ((s & mX) << X.vreal))
          for s in (0, 1)]                                                  # [i][j]
    Wd = [engine.gather_fn(W.dev, J * K, lambda t, s=s: _view_index(wv, {S_J: t >> lk, S_A: t & (K - 1)}) | ((s & mW) << W.vreal))
          for s in (0, 1)]                                                  # [j][k]
    eq_i, eq_k = engine.build_eq_gpu(u64(zi_)), engine.build_eq_gpu(u64(zk_))
    msgs, r = [], []

    def phase(A, B, rounds, rd0):
        nonlocal pref
        ch, m, left, pref = engine.sc_prove_zc_partial(tr, "imm-sc", [A, B], [(1, (1,))], 0, rounds, table[rd0:rd0 + rounds], pref)
        msgs.append(np.ascontiguousarray(m, dtype=np.uint64).tobytes())
        return [int(x) for x in ch], left

    # rounds over j: sum_s w_s sum_j X_s(j, zi) W_s(j, zk)
    rj = []
    if lj:
        A = engine.concat([engine.scale(engine.matvec(Xd[s], I, J, eq_i, False), ws[s]) for s in (0, 1)])
        B = engine.concat([engine.matvec(Wd[s], J, K, eq_k, True) for s in (0, 1)])
        rj, _ = phase(A, B, lj, 0)
    eq_rj = engine.build_eq_gpu(u64(rj))
    X1 = [engine.matvec(Xd[s], I, J, eq_rj, True) for s in (0, 1)]          # X_s(rj, i)
    W1 = [engine.matvec(Wd[s], J, K, eq_rj, False) for s in (0, 1)]         # W_s(rj, k)
    # rounds over k: sum_s w_s [sum_i eq(zi, i) X_s(rj, i)] sum_k eq(zk, k) W_s(rj, k)
    SX = [engine.eval_h_gpu(X1[s], u64(zi_)) for s in (0, 1)]
    rk, Wrr = [], [engine.element(W1[s], 0) for s in (0, 1)]
    if lk:
        A = engine.concat([engine.scale(eq_k, ws[s] * SX[s] % GL_P) for s in (0, 1)])
        rk, left = phase(A, engine.concat(W1), lk, lj)
        Wrr = [int(left[1][s]) for s in (0, 1)]
    eqk_r = 1
    for a, b in zip(rk, zk_):
        eqk_r = eqk_r * ((a * b + (1 - a) * (1 - b)) % GL_P) % GL_P
    # rounds over i: sum_s w_s eq(zk, rk) W_s(rj, rk) sum_i eq(zi, i) X_s(rj, i)
    ri = []
    if li:
        A = engine.concat([engine.scale(eq_i, ws[s] * eqk_r % GL_P * Wrr[s] % GL_P) for s in (0, 1)])
        ri, _ = phase(A, engine.concat(X1), li, lj + lk)
    eqi_r = 1
    for a, b in zip(ri, zi_):
        eqi_r = eqi_r * ((a * b + (1 - a) * (1 - b)) % GL_P) % GL_P
    # rounds over the slice variables: eq((zex, 0..); ex) * eq(zk, rk) eq(zi, ri) * X(rj, ri, ex) * W(rj, rk, ex)
    px, pw = u64(view_point(xv, rj, ri)), u64(view_point(wv, rj, rk))
    NX, NW = 1 << X.vreal, 1 << W.vreal
    xs = [engine.eval_h_gpu(engine.slice(X.dev, (s & mX) * NX, NX), px) for s in range(1 << e_p)]
    wsl = [engine.eval_h_gpu(engine.slice(W.dev, (s & mW) * NW, NW), pw) for s in range(1 << e_p)]
    c0 = eqk_r * eqi_r % GL_P
    ecol = [c0 * ws[s] % GL_P if s < 2 else 0 for s in range(1 << e_p)]
    ch, m, _, pref = engine.sc_prove_zc_partial(tr, "imm-sc", [engine.upload(u64(ecol)), engine.upload(u64(xs)), engine.upload(u64(wsl))],
                                                [(1, (1, 2))], 0, e_p, table[lt:lt + e_p], pref)
    msgs.append(np.ascontiguousarray(m, dtype=np.uint64).tobytes())
    r = rj + rk + ri + [int(x) for x in ch]
    return r, b"".join(msgs), _sblind_end(engine, zc, tr, sb, r, pref, ledger)


def linked_y_mask(engine, zc, X, W, lj, lk, li):
    """p3imm::accum_mask1 + mk_linked for the direct layouts: slice 1 of Y's mask is the product of the operands' first mask
    slices (zkllm-src/p3_int_gadgets.cuh:510-527), the higher slices are fresh."""
    J, K, I = 1 << lj, 1 << lk, 1 << li
    xm, wm = slice1(engine, X), slice1(engine, W)
    return mk_linked(engine, zc, lk + li, engine.matmul(xm, wm, I, J, K))


def imm_prove(engine, zc, tr, X, W, Y, lj, lk, li, R, Q, ledger=None):
    """p3imm::prove with the zk switch on, direct layouts X = [j | i<<lj], W = [k | j<<lk], Y = [k | i<<lk] (ZCol each; Y
    committed with linked_y_mask).  Chains below the structured-blind threshold run over the materialised (j, k, i, ex)
    domain with four committed blind columns, chains above it in the factored form (imm_chain_factored).  Standalone (no
    shared ledger): the blinded batched openings follow."""
    if ledger is not None:
        return imm_prove_views(engine, zc, tr, X, W, Y, lj, lk, li, R, Q, ledger)
    ledger = ZLedger()
    body = imm_prove_views(engine, zc, tr, X, W, Y, lj, lk, li, R, Q, ledger)[:-4]
    batches = tail_prove(engine, zc, tr, ledger, R, Q, "imm-bo")
    return body + struct.pack("<I", len(batches)) + b"".join(struct.pack("<I", len(b)) + b for b in batches)


# ---------------------------------------------------------------------------------- merged lookups in hiding mode
def _virt(col):
    return not isinstance(col, ZCol)


def _dev(col):
    return col if _virt(col) else col.dev


def prove_super(engine, zc, tr, table_cols, table_id, subgroups, R, ledger, strict=True):
    """p3lu::prove_super with the zk switch on (zkllm-src/p3_logup.cuh:1357-1881): one merged logUp instance per table over
    GKR fraction trees whose leaves are sibling-interleaved with committed uniform mask leaves.

    subgroups: [(n, members)] in flush order; a member is (cols, idx[, bind]) with c AUGMENTED columns of 2^(n + e_of(n))
    entries (ZCol when committed, a plain engine column when virtual) and 2^n row indices; bind(tr, ledger, pm, y_virt)
    returns the values that ride in the proof.  Per subgroup two mask streams pm = sm * qm and qm are committed (salted, not
    augmented) before gamma / beta; the table side's last mask fraction is fixed so that the junk cancels.  The claims go to
    ``ledger`` in the reference's order.  Returns (proof bytes, committed multiplicity column).
    Serialised GroupProof: u32 m, c, ns | root_cnt | rt_pmT rt_qmT | gkT | per subgroup: u32 n, k | rt_pm rt_qm | gk |
    per member: u32 nW, yW.., u32 nV, y_virt.., u32 nX, extra.."""
    from .p3 import col_sum
    c = len(table_cols)
    M = int(table_cols[0].numel())
    m = M.bit_length() - 1
    tr.absorb("lug-tab", table_id)
    tr.absorb("lug-sdims", struct.pack("<III", len(subgroups), m, c))
    pad_rows, idx_all = 0, []
    for n, members in subgroups:
        k = len(members)
        g = (k - 1).bit_length()
        NA = 1 << zc.vfull(n)
        tr.absorb("lug-dims", struct.pack("<IIII", n, g, k, c))
        for cols, idx, *_ in members:
            if len(cols) != c or any(int(_dev(t).numel()) != NA for t in cols) or int(idx.numel()) != (1 << n):
                raise ValueError("p3lu: group member size")
            for t in cols:
                if _virt(t):
                    tr.absorb("lug-Wv", b"virt")
                else:
                    tr.absorb("lug-W", t.root)
            idx_all.append(idx)
        pad_rows += ((1 << g) - k) << n
    cnt = engine.lu_counts(idx_all, M, pad_rows)
    Ccnt = commit_col(engine, zc, cnt, R)
    tr.absorb("lug-cnt", Ccnt.root)
    # mask-leaf streams of every subgroup, then of the table side, all committed before gamma / beta
    masks, SmA = [], 0
    for n, members in subgroups:
        g = (len(members) - 1).bit_length()
        NM = 1 << (n + g + zc.e_of(n))
        pseed, qseed = zc.next_seed(), zc.next_seed()
        sm, qm = engine.zk_fill_at(pseed, NM), engine.zk_fill_at(qseed, NM)
        SmA = (SmA + col_sum(engine, sm)) % GL_P
        sP = zc.next_seed()
        pm_ = engine.mul(sm, qm)
        vm = n + g + zc.e_of(n)
        PM = ZCol(pm_, None, vm, sP)
        PM.root, PM.cw, PM.tree = _salted(engine, pm_, R, sP, zc.take(vm, R))
        sQ = zc.next_seed()
        QM = ZCol(qm, None, vm, sQ)
        QM.root, QM.cw, QM.tree = _salted(engine, qm, R, sQ, zc.take(vm, R))
        tr.absorb("lug-pm", PM.root)
        tr.absorb("lug-qm", QM.root)
        masks.append((PM, QM))
    MT = 1 << zc.vfull(m)
    pseedT, qseedT = zc.next_seed(), zc.next_seed()
    smT, qmT = engine.zk_fill_at(pseedT, MT), engine.zk_fill_at(qseedT, MT)
    Smcnt = (col_sum(engine, Ccnt.dev) - col_sum(engine, cnt)) % GL_P
    part = (col_sum(engine, smT) - engine.element(smT, MT - 1)) % GL_P
    pmT = engine.mul(smT, qmT)
    engine.set_element(pmT, MT - 1, (SmA - Smcnt - part) % GL_P * engine.element(qmT, MT - 1) % GL_P)
    sP = zc.next_seed()
    PMT = ZCol(pmT, None, m + zc.e_of(m), sP)
    PMT.root, PMT.cw, PMT.tree = _salted(engine, pmT, R, sP, zc.take(m + zc.e_of(m), R))
    sQ = zc.next_seed()
    QMT = ZCol(qmT, None, m + zc.e_of(m), sQ)
    QMT.root, QMT.cw, QMT.tree = _salted(engine, qmT, R, sQ, zc.take(m + zc.e_of(m), R))
    tr.absorb("lug-pmT", PMT.root)
    tr.absorb("lug-qmT", QMT.root)
    gamma, beta = tr.chal(), tr.chal()
    gp = [pow(gamma, t, GL_P) for t in range(c)]
    a0 = sum(g_ * int(engine.element(col, 0)) for g_, col in zip(gp, table_cols)) % GL_P
    accP, accQ = 0, 1
    subs = []
    for (n, members), (PM, QM) in zip(subgroups, masks):
        k = len(members)
        g = (k - 1).bit_length()
        E = zc.e_of(n)
        NR, NM, N = 1 << (n + g), 1 << (n + g + E), 1 << n
        # even leaves: numerator 1 on the real rows, 0 on the witness-mask rows; denominator A + beta on every slice
        evenQ = engine.concat([engine.lu_leaf_denominators([[engine.slice(_dev(t), ex << n, N) for t in mb[0]] for mb in members],
                                                           1 << g, n, gamma, beta, (a0 + beta) % GL_P) for ex in range(1 << E)])
        evenP = engine.concat([engine.lu_ones(NR), engine.zeros(NM - NR)])
        gk, rA, _ = engine.gkr_prove(tr, "lug-gA", engine.interleave(evenP, PM.dev), engine.interleave(evenQ, QM.dev), False)
        P, Q = (int(x) for x in np.frombuffer(gk[:16], dtype=np.uint64))
        accP, accQ = (accP * Q + P * accQ) % GL_P, accQ * Q % GL_P
        _p0, p1, _q0, q1 = (int(x) for x in np.frombuffer(gk[-32:], dtype=np.uint64))
        rA = [int(x) for x in rA]
        ledger.add(PM, rA, p1)
        ledger.add(QM, rA, q1)
        pm = rA[:n] + rA[n + g:]
        pma = np.array(pm, dtype=np.uint64)
        mem = []
        for cols, idx, *bind in members:
            yW, yv = [], []
            for t in cols:
                y = engine.eval_h_gpu(_dev(t), pma)
                if _virt(t):
                    yv.append(y)
                    tr.absorb("lug-yv", struct.pack("<Q", y))
                else:
                    yW.append(y)
                    tr.absorb("lug-yW", struct.pack("<Q", y))
                    ledger.add(t, pm, y)
            extra = bind[0](tr, ledger, pm, yv) if bind and bind[0] is not None else []
            mem.append((yW, yv, extra))
        subs.append((n, k, PM.root + QM.root, gk, mem))
    evenQ = engine.concat([engine.affine(table_cols, gamma, beta), engine.lu_ones(MT - M)]) if MT > M else engine.affine(table_cols, gamma, beta)
    gkT, rT, _ = engine.gkr_prove(tr, "lug-gT", engine.interleave(Ccnt.dev, PMT.dev), engine.interleave(evenQ, QMT.dev), False)
    PT, QT = (int(x) for x in np.frombuffer(gkT[:16], dtype=np.uint64))
    if strict and accP * QT % GL_P != PT * accQ % GL_P:
        raise ValueError("p3lu: witness not in table")
    p0, p1, _q0, q1 = (int(x) for x in np.frombuffer(gkT[-32:], dtype=np.uint64))
    rT = [int(x) for x in rT]
    ledger.add(Ccnt, rT, p0)
    ledger.add(PMT, rT, p1)
    ledger.add(QMT, rT, q1)
    out = struct.pack("<III", m, c, len(subs)) + Ccnt.root + PMT.root + QMT.root + gkT
    for n, k, rts, gk, mem in subs:
        out += struct.pack("<II", n, k) + rts + gk
        for yW, yv, extra in mem:
            for vals in (yW, yv, extra):
                out += struct.pack("<I", len(vals)) + np.array(vals, dtype=np.uint64).tobytes()
    return out, Ccnt


def lu_flush(engine, zc, tr, luq, ledger, R, strict=True):
    """p3lu::lu_flush (zkllm-src/p3_logup.cuh:1883-1956) over queued obligations {"W": augmented columns, "idx", "tab", "bind"}:
    groups by (table, log-rows) in first-appearance order, chunks of 2^(25 - n) members, bundles by table, one prove_super
    per table.  The table columns are uploaded once per flush."""
    from .p3 import LU_GCAP, table_columns
    groups = []                                       # [table id, n, [queue index]]
    for i, o in enumerate(luq):
        n = int(o["idx"].numel()).bit_length() - 1
        for grp in groups:
            if grp[0] == o["tab"]["id"] and grp[1] == n:
                grp[2].append(i)
                break
        else:
            groups.append([o["tab"]["id"], n, [i]])
    chunks = []
    for tid, n, mem in groups:
        cap = 1 if n >= LU_GCAP else 1 << (LU_GCAP - n)
        for off in range(0, len(mem), cap):
            chunks.append((tid, n, mem[off:off + cap]))
    supers = []
    for tid, n, mem in chunks:
        for sp in supers:
            if sp[0] == tid:
                sp[1].append((n, mem))
                break
        else:
            supers.append((tid, [(n, mem)]))
    out = []
    for tid, sgs in supers:
        tab = luq[sgs[0][1][0]]["tab"]
        subgroups = [(n, [(luq[j]["W"], luq[j]["idx"], luq[j].get("bind")) for j in mem]) for n, mem in sgs]
        pf, _ = prove_super(engine, zc, tr, table_columns(engine, tab), tab["id"], subgroups, R, ledger, strict)
        out.append(pf)
    del luq[:]
    return out


def irs_prove(engine, zc, tr, tables, X, Y, wit, le, sf, rng, R, Q, ledger=None, luq=None, tag="irs"):
    """p3irs::prove with the zk switch on (zkllm-src/p3_int_gadgets.cuh:282-340): y = round(x / 2^sf) through committed limb
    columns, range lookups on the limbs and on y, and the blinded zero-check of x + 2^(sf-1) - y 2^sf - L0 - 2^16 L1.
    X, Y: ZCol; wit: (limb columns, limb index columns, index column of y or None) as Prover.irs_witness returns them.
    Serialised: u32 le, sf, nl, rng | limb roots | messages vfull(le) * 40 | yX yY yL.. | Blind | standalone: u32 groups
    (u32 length + GroupProof)*, u32 batches (u32 length + BatchProof)*."""
    own = ledger is None
    if own:
        ledger, luq = ZLedger(), []
    L, iL, iY = wit
    nl = len(L)
    tr.absorb("irs-dims", struct.pack("<IIII", le, sf, nl, rng))
    tr.absorb("irs-X", X.root)
    tr.absorb("irs-Y", Y.root)
    CL = []
    for l in range(nl):
        CL.append(commit_col(engine, zc, L[l], R))
        tr.absorb("irs-L", CL[l].root)
    limb_tab = lambda l: (tables["R14"] if sf == 14 else tables["R16"]) if l == 0 else (tables["R16"] if sf == 32 else tables["RTOP"])
    for l in range(nl):
        luq.append({"W": [CL[l]], "idx": iL[l], "tab": limb_tab(l)})
    if rng:
        luq.append({"W": [Y], "idx": iY, "tab": tables["RS20"] if rng == 1 else tables["RS16"]})
    zE = [tr.chal() for _ in range(le)]
    H, P2 = 1 << (sf - 1), 1 << sf
    cols = [engine.build_eq_gpu(np.array(zpt(zc, zE), dtype=np.uint64)), X.dev, Y.dev] + [c.dev for c in CL]
    terms = [(1, (1,)), (GL_P - P2, (2,)), (GL_P - 1, (3,))] + ([(GL_P - 65536, (4,))] if nl == 2 else [])
    r, msgs, _, blind = sc5z(engine, zc, tr, "irs-sc", le, cols, terms, H, R, ledger)
    ys = [claimc(engine, tr, ledger, col, r) for col in [X, Y] + CL]
    out = struct.pack("<IIII", le, sf, nl, rng) + b"".join(c.root for c in CL)
    out += np.ascontiguousarray(msgs, dtype=np.uint64).tobytes() + struct.pack("<%dQ" % len(ys), *ys) + blind
    return out + (_tail(engine, zc, tr, luq, ledger, R, Q, "irs-bo") if own else _EMPTY_TAIL)


def _tail(engine, zc, tr, luq, ledger, R, Q, tag):
    """p3ig::tail_prove: the lookup flush, then one blinded batched opening per size class; serialised as u32 groups (u32 length
    + GroupProof)*, u32 batches (u32 length + BatchProof)*."""
    lug = lu_flush(engine, zc, tr, luq, ledger, R)
    batches = tail_prove(engine, zc, tr, ledger, R, Q, tag)
    blob = lambda bs: struct.pack("<I", len(bs)) + b"".join(struct.pack("<I", len(b)) + b for b in bs)
    return blob(lug) + blob(batches)


_EMPTY_TAIL = struct.pack("<II", 0, 0)


def iadd_prove(engine, zc, tr, tables, A, B, OUT, idxO, le, R, Q, ledger=None, luq=None):
    """p3iadd::prove with the zk switch on (zkllm-src/p3_int_gadgets.cuh:712-737): OUT = A + B through one blinded zero-check
    and the signed range lookup on OUT.  A, B, OUT: ZCol.  Serialised: u32 le | messages vfull(le)*40 | yA yB yO | Blind | tail."""
    own = ledger is None
    if own:
        ledger, luq = ZLedger(), []
    tr.absorb("iad-dims", struct.pack("<I", le))
    tr.absorb("iad-A", A.root)
    tr.absorb("iad-B", B.root)
    tr.absorb("iad-O", OUT.root)
    luq.append({"W": [OUT], "idx": idxO, "tab": tables["RS20"]})
    zE = [tr.chal() for _ in range(le)]
    cols = [engine.build_eq_gpu(np.array(zpt(zc, zE), dtype=np.uint64)), A.dev, B.dev, OUT.dev]
    r, msgs, _, blind = sc5z(engine, zc, tr, "iad-sc", le, cols, [(1, (1,)), (1, (2,)), (GL_P - 1, (3,))], 0, R, ledger)
    ys = [claimc(engine, tr, ledger, col, r) for col in (A, B, OUT)]
    out = struct.pack("<I", le) + np.ascontiguousarray(msgs, dtype=np.uint64).tobytes() + struct.pack("<QQQ", *ys) + blind
    return out + (_tail(engine, zc, tr, luq, ledger, R, Q, "iad-bo") if own else _EMPTY_TAIL)


def iswg_prove(engine, zc, tr, tables, G, U, MO, wit, le, R, Q, ledger=None, luq=None):
    """p3iswg::prove with the zk switch on (zkllm-src/p3_int_gadgets.cuh:1790-1832): MO = round(SILU[G] * U / 2^16) through the
    committed SILU values and remainders, the two-column SILU lookup, two range lookups and one blinded zero-check.
    G, U, MO: ZCol; wit = (sil, rem, idxG, idxR, idxM).  Serialised: u32 le | rSIL rREM | messages vfull(le)*40 |
    ySIL yU yM yR | Blind | tail."""
    own = ledger is None
    if own:
        ledger, luq = ZLedger(), []
    sil, rem, idxG, idxR, idxM = wit
    tr.absorb("isw-dims", struct.pack("<I", le))
    tr.absorb("isw-G", G.root)
    tr.absorb("isw-U", U.root)
    tr.absorb("isw-M", MO.root)
    SIL = commit_col(engine, zc, sil, R)
    REM = commit_col(engine, zc, rem, R)
    tr.absorb("isw-s", SIL.root)
    tr.absorb("isw-r", REM.root)
    luq.append({"W": [G, SIL], "idx": idxG, "tab": tables["SILU"]})
    luq.append({"W": [REM], "idx": idxR, "tab": tables["R16"]})
    luq.append({"W": [MO], "idx": idxM, "tab": tables["RS20"]})
    zE = [tr.chal() for _ in range(le)]
    cols = [engine.build_eq_gpu(np.array(zpt(zc, zE), dtype=np.uint64)), SIL.dev, U.dev, MO.dev, REM.dev]
    terms = [(1, (1, 2)), (GL_P - 65536, (3,)), (GL_P - 1, (4,))]
    r, msgs, _, blind = sc5z(engine, zc, tr, "isw-sc", le, cols, terms, 32768, R, ledger)
    ys = [claimc(engine, tr, ledger, col, r) for col in (SIL, U, MO, REM)]
    out = struct.pack("<I", le) + SIL.root + REM.root + np.ascontiguousarray(msgs, dtype=np.uint64).tobytes()
    out += struct.pack("<QQQQ", *ys) + blind
    return out + (_tail(engine, zc, tr, luq, ledger, R, Q, "isw-bo") if own else _EMPTY_TAIL)


def irope_prove(engine, zc, tr, tables, pub, Qc, Y, wit, lT, ld, R, Q, ledger=None, luq=None):
    """p3irope::prove with the zk switch on (zkllm-src/p3_int_gadgets.cuh:1275-1322).  pub = (C, S2, ldh): the public
    broadcasts over the 2^(lT+ld) real entries (zero on the mask slices, as the reference's pub_col); Qc, Y: ZCol;
    wit = (rem, idxR, idxY).  The rotate-half partner is the bit flip of the whole augmented array, so its claim sits at
    the flipped point.  Serialised: u32 lT, ld, fb | rREM | messages vfull(le)*40 | yQ yQx yY yR | Blind | tail."""
    own = ledger is None
    if own:
        ledger, luq = ZLedger(), []
    Ccol, Scol, ldh = pub
    rem, idxR, idxY = wit
    le, fb = lT + ld, ldh - 1
    tr.absorb("irp-dims", struct.pack("<III", lT, ld, fb))
    tr.absorb("irp-Q", Qc.root)
    tr.absorb("irp-Y", Y.root)
    REM = commit_col(engine, zc, rem, R)
    tr.absorb("irp-r", REM.root)
    luq.append({"W": [REM], "idx": idxR, "tab": tables["R14"]})
    luq.append({"W": [Y], "idx": idxY, "tab": tables["RS20"]})
    zE = [tr.chal() for _ in range(le)]
    pad = (1 << zc.vfull(le)) - (1 << le)
    cols = [engine.build_eq_gpu(np.array(zpt(zc, zE), dtype=np.uint64)), Qc.dev, engine.flip_bit(Qc.dev, fb), Y.dev, REM.dev,
            engine.concat([Ccol, engine.zeros(pad)]), engine.concat([Scol, engine.zeros(pad)])]
    terms = [(1, (1, 5)), (1, (2, 6)), (GL_P - 16384, (3,)), (GL_P - 1, (4,))]
    r, msgs, _, blind = sc5z(engine, zc, tr, "irp-sc", le, cols, terms, 8192, R, ledger)
    rf = list(r)
    rf[fb] = (1 - rf[fb]) % GL_P
    ys = [claimc(engine, tr, ledger, Qc, r), claimc(engine, tr, ledger, Qc, rf), claimc(engine, tr, ledger, Y, r),
          claimc(engine, tr, ledger, REM, r)]
    out = struct.pack("<III", lT, ld, fb) + REM.root + np.ascontiguousarray(msgs, dtype=np.uint64).tobytes()
    out += struct.pack("<QQQQ", *ys) + blind
    return out + (_tail(engine, zc, tr, luq, ledger, R, Q, "irp-bo") if own else _EMPTY_TAIL)


def irms_prove(engine, zc, tr, tables, X, G, Y, wit, lT, ld, R, Q, ledger=None, luq=None):
    """p3irms::prove with the zk switch on (zkllm-src/p3_int_gadgets.cuh:918-1047).  X, Y: ZCol over 2^(lT+ld) entries, G over
    2^ld; wit: ig.irms_witness output with db / de as engine columns.  The first mask slice of the row column M is LINKED:
    CEPS plus the row sums of squares of X's first mask slice, so that the row-sum binding holds slice by slice at the
    hiding point (z | zex | 0..).  Three blinded chains.  Serialised: u32 lT, ld | 18 row roots | 3 element roots | yM yMX |
    mS | mB yB[18] | mE yE[3] yEX yEY yER yEG | three Blinds | tail."""
    from . import ig
    own = ledger is None
    if own:
        ledger, luq = ZLedger(), []
    le = lT + ld
    tr.absorb("irm-dims", struct.pack("<II", lT, ld))
    tr.absorb("irm-X", X.root)
    tr.absorb("irm-G", G.root)
    tr.absorb("irm-Y", Y.root)
    x1 = slice1(engine, X)
    rows = engine.matvec(engine.mul(x1, x1), 1 << lT, 1 << ld, engine.lu_ones(1 << ld), True)
    mM = mk_linked(engine, zc, lT, engine.affine([rows], 1, ig.CEPS))
    CB, CE = [], []
    for k, c in enumerate(wit["db"]):
        CB.append(commit_col(engine, zc, c, R, mask=mM if k == ig.B_M else None))
        tr.absorb("irm-cb", CB[k].root)
    for k, c in enumerate(wit["de"]):
        CE.append(commit_col(engine, zc, c, R))
        tr.absorb("irm-ce", CE[k].root)
    defer = lambda cols, idx, tab: luq.append({"W": cols, "idx": idx, "tab": tables[tab]})
    defer([CB[ig.B_P4], CB[ig.B_P2], CB[ig.B_H2]], wit["idxE4"], "EXP4")
    defer([CB[ig.B_MM]], wit["idxM16"], "R16")
    defer([CB[ig.B_MS]], wit["idxMS"], "R16")
    defer([CB[ig.B_MM], CB[ig.B_RP]], wit["idxISQ"], "ISQ")
    for l, c in enumerate((ig.B_L40, ig.B_L41, ig.B_L42, ig.B_D40, ig.B_D41, ig.B_D42, ig.B_L20, ig.B_D20, ig.B_LR0)):
        defer([CB[c]], wit["idxL"][l], "R16")
    defer([CB[ig.B_LR1]], wit["idxLR1"], "R16")
    defer([CE[1]], wit["idxRW"], "R16")
    defer([CE[0]], wit["idxW"], "RS20")
    defer([CE[2]], wit["idxRY"], "R16")
    defer([Y], wit["idxY"], "RS20")
    eX = zc.e_of(le)
    NeA = 1 << (le + eX)
    # M row-sum binding at the hiding point: sum_j X^2 = M - CEPS on the real slice and on mask slice 1
    zb = [tr.chal() for _ in range(lT)]
    zex = tr.chal()
    yM = claimc(engine, tr, ledger, CB[ig.B_M], xpt(zc, zb, zex))
    eqb = engine.build_eq_gpu(np.array(zb + [zex] + [0] * (eX - 1), dtype=np.uint64))
    EQb = engine.gather_fn(eqb, NeA, lambda q: ((q >> le) << lT) | ((q & ((1 << le) - 1)) >> ld))
    rS, mS, _, bl0 = sc5z(engine, zc, tr, "irm-scS", le, [EQb, X.dev], [(1, (1, 1))], 0, R, ledger)
    yMX = claimc(engine, tr, ledger, X, rS)
    # per-row zero-check
    zB = [tr.chal() for _ in range(lT)]
    termsB, konstB = ig.irms_terms_rows(tr.chal())
    colsB = [engine.build_eq_gpu(np.array(zpt(zc, zB), dtype=np.uint64))] + [c.dev for c in CB]
    rB, mB, _, bl1 = sc5z(engine, zc, tr, "irm-scB", lT, colsB, termsB, konstB, R, ledger)
    yB = [claimc(engine, tr, ledger, c, rB) for c in CB]
    # per-element zero-check; the row value R and the gains are broadcast over the augmented element domain
    zE = [tr.chal() for _ in range(le)]
    termsE, konstE = ig.irms_terms_elements(tr.chal())
    eR, eG = zc.e_of(lT), zc.e_of(ld)
    mR, mG = (1 << min(eR, eX)) - 1, (1 << min(eG, eX)) - 1
    Rb = engine.gather_fn(CB[ig.B_R].dev, NeA, lambda q: ((q & ((1 << le) - 1)) >> ld) | (((q >> le) & mR) << lT))
    Gb = engine.gather_fn(G.dev, NeA, lambda q: (q & ((1 << ld) - 1)) | (((q >> le) & mG) << ld))
    colsE = [engine.build_eq_gpu(np.array(zpt(zc, zE), dtype=np.uint64)), X.dev, Y.dev, CE[0].dev, CE[1].dev, CE[2].dev, Rb, Gb]
    rE, mE, _, bl2 = sc5z(engine, zc, tr, "irm-scE", le, colsE, termsE, konstE, R, ledger)
    yEX = claimc(engine, tr, ledger, X, rE)
    yEY = claimc(engine, tr, ledger, Y, rE)
    yE = [claimc(engine, tr, ledger, c, rE) for c in CE]
    yER = claimc(engine, tr, ledger, CB[ig.B_R], expt(zc, rE[ld:le], rE, le))
    yEG = claimc(engine, tr, ledger, G, expt(zc, rE[:ld], rE, le))
    u64 = lambda m: np.ascontiguousarray(m, dtype=np.uint64).tobytes()
    out = struct.pack("<II", lT, ld) + b"".join(c.root for c in CB) + b"".join(c.root for c in CE)
    out += struct.pack("<QQ", yM, yMX) + u64(mS) + u64(mB) + struct.pack("<18Q", *yB) + u64(mE) + struct.pack("<3Q", *yE)
    out += struct.pack("<QQQQ", yEX, yEY, yER, yEG) + bl0 + bl1 + bl2
    return out + (_tail(engine, zc, tr, luq, ledger, R, Q, "irm-bo") if own else _EMPTY_TAIL)


def _eqb_col(engine, ptb, lb, lcols, le, NeA):
    """p3ig::eqb_col (zkllm-src/p3_int_gadgets.cuh:150-162): the row weight over the augmented element domain,
    EQb[e | ex << le] = eq(ptb)[(ex << lb) | row(e)]."""
    eqb = engine.build_eq_gpu(np.array(ptb, dtype=np.uint64))
    return engine.gather_fn(eqb, NeA, lambda q: ((q >> le) << lb) | ((q & ((1 << le) - 1)) >> lcols))


def ismx_prove(engine, zc, tr, tables, Z, P, wit, la, lseq, R, Q, ledger=None, luq=None):
    """p3ismx::prove with the zk switch on (zkllm-src/p3_int_gadgets.cuh:1514-1643): causal softmax rows.  Z, P: ZCol over
    2^(la + 2 lseq) entries; wit: ig.ismx_witness output with xe / xb as engine columns.  The first mask slice of the row sums
    S is LINKED to the row sums of EE's first mask slice.  The SEL row sums are bound at the zero-extended point (public
    base 1), the S row sums at the hiding point.  Serialised: u32 la, lseq | 7 element roots | 2 row roots | mSel ySel |
    ySrow mS ySE | mE yEZ yE[7] yEP yEMX yES | three Blinds | tail."""
    from . import ig
    own = ledger is None
    if own:
        ledger, luq = ZLedger(), []
    lr, le = la + lseq, la + 2 * lseq
    tr.absorb("ism-dims", struct.pack("<II", la, lseq))
    tr.absorb("ism-Z", Z.root)
    tr.absorb("ism-P", P.root)
    CE = []
    for c in wit["xe"]:
        CE.append(commit_col(engine, zc, c, R))
        tr.absorb("ism-ce", CE[-1].root)
    e1 = slice1(engine, CE[ig.X_EE])
    mS_ = mk_linked(engine, zc, lr, engine.matvec(e1, 1 << lr, 1 << lseq, engine.lu_ones(1 << lseq), True))
    CB = [commit_col(engine, zc, wit["xb"][0], R), commit_col(engine, zc, wit["xb"][1], R, mask=mS_)]
    for c in CB:
        tr.absorb("ism-cb", c.root)
    luq.append({"W": [CE[ig.X_DM], CE[ig.X_EE]], "idx": wit["idxDM"], "tab": tables["EXPT"]})
    for l in range(4):
        luq.append({"W": [CE[ig.X_L0 + l]], "idx": wit["idxL"][l], "tab": tables["R16"]})
    luq.append({"W": [CB[0]], "idx": wit["idxMX"], "tab": tables["RS16"]})
    eX = zc.e_of(le)
    NeA = 1 << (le + eX)
    # SEL row sums = 1: zero-extended row point
    zb = [tr.chal() for _ in range(lr)]
    rS, mSel, _, bl0 = sc5z(engine, zc, tr, "ism-scsel", le, [_eqb_col(engine, zb + [0] * eX, lr, lseq, le, NeA), CE[ig.X_SEL].dev],
                            [(1, (1,))], 0, R, ledger)
    ySel = claimc(engine, tr, ledger, CE[ig.X_SEL], rS)
    # S row sums: hiding claim on S, linked masks
    zb = [tr.chal() for _ in range(lr)]
    zex = tr.chal()
    ySrow = claimc(engine, tr, ledger, CB[1], xpt(zc, zb, zex))
    rS2, mS, _, bl1 = sc5z(engine, zc, tr, "ism-scs", le,
                           [_eqb_col(engine, zb + [zex] + [0] * (eX - 1), lr, lseq, le, NeA), CE[ig.X_EE].dev], [(1, (1,))], 0, R, ledger)
    ySE = claimc(engine, tr, ledger, CE[ig.X_EE], rS2)
    # per-element zero-check
    zE = [tr.chal() for _ in range(le)]
    terms, konst = ig.ismx_terms(tr.chal())
    mB = (1 << min(zc.e_of(lr), eX)) - 1
    bc = lambda col: engine.gather_fn(col.dev, NeA, lambda q: ((q & ((1 << le) - 1)) >> lseq) | (((q >> le) & mB) << lr))
    mask = engine.concat([engine.causal_mask(la, lseq), engine.zeros(NeA - (1 << le))])
    cols = [engine.build_eq_gpu(np.array(zpt(zc, zE), dtype=np.uint64)), Z.dev] + [c.dev for c in CE] + [P.dev, bc(CB[0]), bc(CB[1]), mask]
    rE, mE, _, bl2 = sc5z(engine, zc, tr, "ism-sce", le, cols, terms, konst, R, ledger)
    yEZ = claimc(engine, tr, ledger, Z, rE)
    yE = [claimc(engine, tr, ledger, c, rE) for c in CE]
    yEP = claimc(engine, tr, ledger, P, rE)
    yEMX = claimc(engine, tr, ledger, CB[0], expt(zc, rE[lseq:le], rE, le))
    yES = claimc(engine, tr, ledger, CB[1], expt(zc, rE[lseq:le], rE, le))
    u64 = lambda m: np.ascontiguousarray(m, dtype=np.uint64).tobytes()
    out = struct.pack("<II", la, lseq) + b"".join(c.root for c in CE) + b"".join(c.root for c in CB)
    out += u64(mSel) + struct.pack("<QQ", ySel, ySrow) + u64(mS) + struct.pack("<Q", ySE)
    out += u64(mE) + struct.pack("<Q", yEZ) + struct.pack("<7Q", *yE) + struct.pack("<QQQ", yEP, yEMX, yES) + bl0 + bl1 + bl2
    return out + (_tail(engine, zc, tr, luq, ledger, R, Q, "ism-bo") if own else _EMPTY_TAIL)


# ---------------------------------------------------------------------------------- operand views and the integer layer
def _view_index(view, vals):
    """p3imm::op_off / y_off (zkllm-src/p3_int_gadgets.cuh:448-470) on index arrays: bit t of the element index comes from bit
    `bit` of vals[src] (S_J, S_A, S_I) or is the constant `bit` (S_C)."""
    from .p3 import S_C
    idx = 0
    for t, (src, bit) in enumerate(view):
        if src == S_C:
            idx = idx | (bit << t)
        elif src in vals:
            idx = idx | (((vals[src] >> bit) & 1) << t)
    return idx


def direct_views(lj, lk, li):
    """p3imm::direct_x / direct_w / direct_y: X = [j | i<<lj], W = [k | j<<lk], Y = [k | i<<lk]."""
    from .p3 import S_A, S_I, S_J
    xv = [(S_J, t) for t in range(lj)] + [(S_A, t) for t in range(li)]
    wv = [(S_A, t) for t in range(lk)] + [(S_J, t) for t in range(lj)]
    yv = [(S_A, t) for t in range(lk)] + [(S_I, t) for t in range(li)]
    return xv, wv, yv


def linked_acc_mask(engine, zc, vY, insts):
    """p3itf::commit_acc (zkllm-src/p3_int_layer.cuh:331-340): the mask of a matmul accumulator grid whose first slice is, per
    instance (X, W, views, lj, lk, li), the product of the operands' first mask slices placed at the instance's Y view."""
    from .p3 import S_A, S_I, S_J
    m1 = engine.zeros(1 << vY)
    for X, W, (xv, wv, yv), lj, lk, li in insts:
        J, K, I = 1 << lj, 1 << lk, 1 << li
        xd = engine.gather_fn(slice1(engine, X), I * J, lambda u: _view_index(xv, {S_J: u & (J - 1), S_A: u >> lj}))
        wd = engine.gather_fn(slice1(engine, W), J * K, lambda u: _view_index(wv, {S_J: u >> lk, S_A: u & (K - 1)}))
        rows = engine.matmul(xd, wd, I, J, K)
        m1 = engine.scatter_fn(m1, K * I, lambda u: _view_index(yv, {S_A: u & (K - 1), S_I: u >> lk}), rows)
    return mk_linked(engine, zc, vY, m1)


def imm_prove_views(engine, zc, tr, X, W, Y, lj, lk, li, R, Q, ledger, views=None):
    """p3imm::prove with the zk switch on for operand views into larger committed grids (per-head attention matmuls): the
    broadcast columns read the augmented grids through the views, every claim sits at the view's point extended by the
    chain's extra coordinates (expt).  Composed mode only (shared ledger; no tail)."""
    from .p3 import S_A, S_I, S_J, view_point
    xv, wv, yv = views or direct_views(lj, lk, li)
    tr.absorb("imm-dims", struct.pack("<III", lj, lk, li))
    tr.absorb("imm-X", X.root)
    tr.absorb("imm-W", W.root)
    tr.absorb("imm-Y", Y.root)
    z = [tr.chal() for _ in range(lk + li)]
    zex = tr.chal()
    yY = claimc(engine, tr, ledger, Y, xpt(zc, view_point(yv, z[:lk], z[lk:], S_A, S_I), zex))
    lt = lj + lk + li
    e_p, eX, eW = zc.e_of(lt), zc.e_of(X.vreal), zc.e_of(W.vreal)
    N = 1 << (lt + e_p)
    J, K, I = 1 << lj, 1 << lk, 1 << li
    mX, mW = (1 << min(eX, e_p)) - 1, (1 << min(eW, e_p)) - 1
    if lt + e_p >= zc.sblind_min and not getattr(zc, "materialise", False):
        r, msgs, blind = imm_chain_factored(engine, zc, tr, X, W, (xv, wv, yv), lj, lk, li, z, zex, R, ledger)
    else:
        eqv = engine.build_eq_gpu(np.array(z + [zex] + [0] * (e_p - 1), dtype=np.uint64))
        cols = [engine.bcast_rows(eqv, lj),
                engine.gather_fn(X.dev, N, lambda u: _view_index(xv, {S_J: u & (J - 1), S_A: (u >> (lj + lk)) & (I - 1)})
                                 | (((u >> lt) & mX) << X.vreal)),
                engine.gather_fn(W.dev, N, lambda u: _view_index(wv, {S_J: u & (J - 1), S_A: (u >> lj) & (K - 1)})
                                 | (((u >> lt) & mW) << W.vreal))]
        r, msgs, _, blind = sc5z(engine, zc, tr, "imm-sc", lt, cols, [(1, (1, 2))], 0, R, ledger)
        msgs = np.ascontiguousarray(msgs, dtype=np.uint64).tobytes()
    rj, rk, ri = r[:lj], r[lj:lj + lk], r[lj + lk:lt]
    yX = claimc(engine, tr, ledger, X, expt(zc, view_point(xv, rj, ri), r, lt))
    yW = claimc(engine, tr, ledger, W, expt(zc, view_point(wv, rj, rk), r, lt))
    out = struct.pack("<III", lj, lk, li) + msgs
    return out + struct.pack("<QQQ", yY, yX, yW) + blind + struct.pack("<I", 0)


def itf_commit_all(engine, zc, c, w, Wt, R, col):
    """p3itf::commit_all with the zk switch on (zkllm-src/p3_int_layer.cuh:343-415), in the reference's commitment order:
    every chain grid, weight and gain with a fresh mask, the matmul accumulator grids with linked masks.  Returns {name: ZCol}
    (weights under "w", accumulators under "acc")."""
    from . import ig
    ld, lT, ldff, lseq, ldh, la = c.ld, c.lT, c.ldff, c.lseq, c.ldh, c.la
    le, lef, lez = ld + lT, ldff + lT, la + 2 * lseq
    o = {"acc": [None] * 7}
    com = lambda a: commit_col(engine, zc, col(a), R)
    heads = [(h, b) for b in range(c.batch) for h in range(c.nh)]

    def acc(i, vY, insts):
        o["acc"][i] = commit_col(engine, zc, col(w["acc"][i]), R, mask=linked_acc_mask(engine, zc, vY, insts))

    o["x0"] = com(w["x0"])
    o["g1"], o["g2"] = com(Wt["g1"]), com(Wt["g2"])
    o["w"] = [com(x) for x in Wt["w"]]
    o["h1"] = com(w["h1"])
    for i in (ig.W_Q, ig.W_K, ig.W_V):
        acc(i, le, [(o["h1"], o["w"][i], direct_views(ld, ld, lT), ld, ld, lT)])
    for k in ("yq", "yk", "yv", "rq", "rk"):
        o[k] = com(w[k])
    o["sc"] = commit_col(engine, zc, col(w["sc"]), R, mask=linked_acc_mask(
        engine, zc, lez, [(o["rq"], o["rk"], ig.views_qk(c, h, b), ldh, lseq, lseq) for h, b in heads]))
    o["z"], o["p"] = com(w["z"]), com(w["p"])
    o["pva"] = commit_col(engine, zc, col(w["pva"]), R, mask=linked_acc_mask(
        engine, zc, le, [(o["p"], o["yv"], ig.views_pv(c, h, b), lseq, ldh, lseq) for h, b in heads]))
    o["at"] = com(w["at"])
    acc(ig.W_O, le, [(o["at"], o["w"][ig.W_O], direct_views(ld, ld, lT), ld, ld, lT)])
    for k in ("yo", "res1", "h2"):
        o[k] = com(w[k])
    for i in (ig.W_G, ig.W_U):
        acc(i, lef, [(o["h2"], o["w"][i], direct_views(ld, ldff, lT), ld, ldff, lT)])
    for k in ("gg", "uu", "mo"):
        o[k] = com(w[k])
    acc(ig.W_D, le, [(o["mo"], o["w"][ig.W_D], direct_views(ldff, ld, lT), ldff, ld, lT)])
    o["yd"], o["out"] = com(w["yd"]), com(w["out"])
    return o


def itf_prove(engine, zc, tr, c, w, o, Wt, T, R, Q, col, stages=None):
    """p3itf::prove with the zk switch on (zkllm-src/p3_int_layer.cuh:452-581): the decoder layer's 24 + 2A sub-proofs in fixed
    order on one transcript with one ledger and one lookup queue, one merged-lookup flush, the public input / output
    bindings at zero-extended points, one blinded batched opening per size class.  Same serialised layout as the plain
    layer proof, every part in its hiding form."""
    from . import ig
    ld, lT, ldff, lseq, ldh, la = c.ld, c.lT, c.ldff, c.lseq, c.ldh, c.la
    le, lef, lez = ld + lT, ldff + lT, la + 2 * lseq
    import time
    t0 = time.perf_counter()
    ledger, luq = ZLedger(), []
    tr.absorb("itf-dims", struct.pack("<6I", c.seq, c.d, c.nh, c.dh, c.dff, c.batch))
    for i in range(7):
        luq.append({"W": [o["w"][i]], "idx": col(w["idxW"][i]), "tab": T["RS20"]})
    luq.append({"W": [o["g1"]], "idx": col(w["idxG1"]), "tab": T["RS20"]})
    luq.append({"W": [o["g2"]], "idx": col(w["idxG2"]), "tab": T["RS20"]})
    luq.append({"W": [o["x0"]], "idx": col(w["idxX0"]), "tab": T["RS20"]})
    subs = []
    up = lambda wit: {k: ([col(x) for x in v] if isinstance(v, (list, tuple)) else col(v)) for k, v in wit.items() if k not in ("y", "p")}

    def lift_any(a):
        if isinstance(a, np.ndarray):
            return ig.lift(a)
        from . import ig_dev
        return ig_dev.lift(a)

    rms = lambda name, X, G, Y: subs.append(irms_prove(engine, zc, tr, T, X, G, Y, up(w[name]), lT, ld, R, Q, ledger, luq))
    mm = lambda X, Wc, Y, lj, lk, li, views=None: subs.append(imm_prove_views(engine, zc, tr, X, Wc, Y, lj, lk, li, R, Q, ledger, views))

    def irs(name, X, Y, lev, sf, rng):
        y, L, iL, iY = w[name]
        subs.append(irs_prove(engine, zc, tr, T, X, Y, ([col(l) for l in L], [col(i) for i in iL], col(iY) if iY is not None else None),
                              lev, sf, rng, R, Q, ledger, luq))

    def rope(name, Qc, Y):
        y, rem, iR, iY, Cc, S2 = w[name]
        subs.append(irope_prove(engine, zc, tr, T, (col(lift_any(Cc)), col(lift_any(S2)), ldh), Qc, Y, (col(rem), col(iR), col(iY)),
                                lT, ld, R, Q, ledger, luq))

    heads = [(h, b) for b in range(c.batch) for h in range(c.nh)]
    rms("rms1", o["x0"], o["g1"], o["h1"])
    for i in (ig.W_Q, ig.W_K, ig.W_V):
        mm(o["h1"], o["w"][i], o["acc"][i], ld, ld, lT)
    irs("rsq", o["acc"][ig.W_Q], o["yq"], le, 16, 1)
    irs("rsk", o["acc"][ig.W_K], o["yk"], le, 16, 1)
    irs("rsv", o["acc"][ig.W_V], o["yv"], le, 16, 1)
    rope("rpq", o["yq"], o["rq"])
    rope("rpk", o["yk"], o["rk"])
    for h, b in heads:
        mm(o["rq"], o["rk"], o["sc"], ldh, lseq, lseq, ig.views_qk(c, h, b))
    irs("rsz", o["sc"], o["z"], lez, c.sfz, 2)
    subs.append(ismx_prove(engine, zc, tr, T, o["z"], o["p"], up(w["smx"]), la, lseq, R, Q, ledger, luq))
    for h, b in heads:
        mm(o["p"], o["yv"], o["pva"], lseq, ldh, lseq, ig.views_pv(c, h, b))
    irs("rsat", o["pva"], o["at"], le, 16, 1)
    mm(o["at"], o["w"][ig.W_O], o["acc"][ig.W_O], ld, ld, lT)
    irs("rso", o["acc"][ig.W_O], o["yo"], le, 16, 1)
    subs.append(iadd_prove(engine, zc, tr, T, o["x0"], o["yo"], o["res1"], col(w["idxRes1"]), le, R, Q, ledger, luq))
    rms("rms2", o["res1"], o["g2"], o["h2"])
    for i in (ig.W_G, ig.W_U):
        mm(o["h2"], o["w"][i], o["acc"][i], ld, ldff, lT)
    irs("rsg", o["acc"][ig.W_G], o["gg"], lef, 16, 1)
    irs("rsu", o["acc"][ig.W_U], o["uu"], lef, 16, 1)
    sil, rem, mo, iG, iR, iM = w["swg"]
    subs.append(iswg_prove(engine, zc, tr, T, o["gg"], o["uu"], o["mo"], (col(sil), col(rem), col(iG), col(iR), col(iM)), lef, R, Q,
                           ledger, luq))
    mm(o["mo"], o["w"][ig.W_D], o["acc"][ig.W_D], ldff, ld, lT)
    irs("rsd", o["acc"][ig.W_D], o["yd"], le, 16, 1)
    subs.append(iadd_prove(engine, zc, tr, T, o["res1"], o["yd"], o["out"], col(w["idxOut"]), le, R, Q, ledger, luq))
    t1 = time.perf_counter()
    lug = lu_flush(engine, zc, tr, luq, ledger, R)
    t2 = time.perf_counter()
    ioin = claimc(engine, tr, ledger, o["x0"], zpt(zc, [tr.chal() for _ in range(le)]))
    ioout = claimc(engine, tr, ledger, o["out"], zpt(zc, [tr.chal() for _ in range(le)]))
    batches = tail_prove(engine, zc, tr, ledger, R, Q, "itf-bo")
    if stages is not None:
        stages.update(subs_s=t1 - t0, lookups_s=t2 - t1, openings_s=time.perf_counter() - t2, lookup_groups=len(lug),
                      opening_classes=len(batches))
    blob = lambda b: struct.pack("<I", len(b)) + b
    roots = [o["x0"].root, o["h1"].root] + [a.root for a in o["acc"]] + [o[k].root for k in
             ("yq", "yk", "yv", "rq", "rk", "sc", "z", "p", "pva", "at", "yo", "res1", "h2", "gg", "uu", "mo", "yd", "out")]
    out = struct.pack("<6I", c.seq, c.d, c.nh, c.dh, c.dff, c.batch) + b"".join(blob(s) for s in subs) + b"".join(roots)
    out += struct.pack("<I", len(lug)) + b"".join(blob(b) for b in lug) + struct.pack("<QQ", ioin, ioout)
    return out + struct.pack("<I", len(batches)) + b"".join(blob(b) for b in batches)
