"""TEST ORACLE (never part of the product): Pedersen row commitments over BLS12-381 G1 in Python integers, a restatement of
the reference's commitment path for checking the CUDA kernels.

Follows zkllm-src/commitment.cu:41-103 (Commitment::commit -> commit_pippenger: 4-bit windows of the scalar's raw limbs,
buckets filled in generator order, running-sum reduction from bucket 15 down, Horner over the 64 windows from the top)
over the group law of zkllm-src/bls12-381.cu:1361-1386 (dbl-2009-l) and :1429-1464 (add-2007-bl with its early returns).
A point is a Jacobian triple of plain integers mod p; `to_bytes` gives the reference's 144-byte form (each coordinate times
2^384 mod p, twelve little-endian 32-bit limbs).

Pins: on a CPU-only machine this file is checked against the group itself (curve equation, associativity with affine
arithmetic, commitment == naive sum of scalar multiples as a group element) -- the byte form is "parity unpinned" there;
on a GPU box the tests compare these bytes with the reference's own kernels (oracle/_ref/libfrref.so).
"""
P = 0x1a0111ea397fe69a4b1ba7b6434bacd764774b84f38512bf6730d2a0f6b0f6241eabfffeb153ffffb9feffffffffaaab
R384 = (1 << 384) % P
GX = 0x17f1d3a73197d7942695638c4fa9ac0fc3688c4f9774b905a14e3a3f171bac586c55e83ff97a1aeffb3af00adb22c6bb
GY = 0x08b3f481e3aaa0f1a09e30ed741d8ae4fcf5e095d5d00af600db18cb2c04b3edd03cc744a2888ae40caa232946c5e7e1
ZERO = (0, 1, 0)
GEN = (GX, GY, 1)


def double(p):
    X, Y, Z = p
    if Z == 0:
        return p
    a, b = X * X % P, Y * Y % P
    c = b * b % P
    d = 2 * ((X + b) ** 2 - a - c) % P
    e = 3 * a % P
    f = e * e % P
    z3 = 2 * Y * Z % P
    x3 = (f - 2 * d) % P
    y3 = (e * (d - x3) - 8 * c) % P
    return (x3, y3, z3)


def add(p, q):
    X1, Y1, Z1 = p
    X2, Y2, Z2 = q
    if Z1 == 0:
        return q
    if Z2 == 0:
        return p
    z1z1, z2z2 = Z1 * Z1 % P, Z2 * Z2 % P
    u1, u2 = X1 * z2z2 % P, X2 * z1z1 % P
    s1, s2 = Y1 * Z2 * z2z2 % P, Y2 * Z1 * z1z1 % P
    if u1 == u2 and s1 == s2:
        return double(p)
    h = (u2 - u1) % P
    i = (2 * h) ** 2 % P
    j = h * i % P
    r = 2 * (s2 - s1) % P
    v = u1 * i % P
    x3 = (r * r - j - 2 * v) % P
    y3 = (r * (v - x3) - 2 * s1 * j) % P
    z3 = ((Z1 + Z2) ** 2 - z1z1 - z2z2) * h % P
    return (x3, y3, z3)


def to_affine(p):
    X, Y, Z = p
    if Z == 0:
        return None
    zi = pow(Z, P - 2, P)
    return (X * zi * zi % P, Y * zi * zi * zi % P)


def on_curve(p):
    a = to_affine(p)
    return a is None or (a[1] * a[1] - a[0] ** 3 - 4) % P == 0


def scalar_mul(p, k):
    acc = ZERO
    for bit in bin(k)[2:] if k else "":
        acc = double(acc)
        if bit == "1":
            acc = add(acc, p)
    return acc


def to_bytes(p):
    out = b""
    for c in p:
        out += ((c * R384) % P).to_bytes(48, "little")
    return out


def from_bytes(b):
    rinv = pow(R384, P - 2, P)
    return tuple(int.from_bytes(b[48 * k:48 * k + 48], "little") * rinv % P for k in range(3))


def pedersen_commit(gens, scalars):
    """gens: n Jacobian points; scalars: rows of n integers below 2^256 (the RAW limb value the reference multiplies by).
    Returns one Jacobian point per row, the triple the reference's kernels produce."""
    out = []
    for row in scalars:
        partial = []
        for w in range(64):
            bucket = [ZERO] * 16
            for g, s in zip(gens, row):
                d = (s >> (4 * w)) & 15
                if d:
                    bucket[d] = add(bucket[d], g)
            acc, run = ZERO, ZERO
            for b in range(15, 0, -1):
                acc = add(acc, bucket[b])
                run = add(run, acc)
            partial.append(run)
        acc = ZERO
        for w in range(63, -1, -1):
            for _ in range(4):
                acc = double(acc)
            acc = add(acc, partial[w])
        out.append(acc)
    return out


# ---------------------------------------------------------------------------------------------------------------------
# Openings of the first proof stack: scalar multiples in the reference's order, its multi-scalar product, the pair-fold
# chains and the Fiat-Shamir inner-product argument (zkllm-src/vrf_common.cuh).  Scalars are plain integers below the
# scalar field's modulus; `tr` is oracle/fr_oracle.py's Transcript.
FR_P = 0x73eda753299d7d483339d80809a1d80553bda402fffe5bfeffffffff00000001
ZERO_BYTES = (0, 0, 0)          # a record of zero bytes (the reference pads odd fold levels with cudaMemset)


def neg(p):
    """G1Jacobian_minus (zkllm-src/g1-tensor.cu:11-21): (X, 0 - Y, Z)."""
    return (p[0], (-p[1]) % P, p[2])


def jac_mul(p, k):
    """G1Jacobian_mul (zkllm-src/g1-tensor.cu:445-453): from the lowest bit up, out += a on a set bit, a doubles."""
    out, a = ZERO, p
    for i in range(256):
        if (k >> i) & 1:
            out = add(out, a)
        a = double(a)
    return out


def msm_tree(g, a):
    """dev_msm (vrf_common.cuh:165-184): x[i] = a[i] g[i], then x[i] += x[i + half] while halving; n a power of two."""
    x = [jac_mul(gi, ai) for gi, ai in zip(g, a)]
    sz = len(x)
    while sz > 1:
        half = sz // 2
        x = [add(x[i], x[i + half]) for i in range(half)]
        sz = half
    return x[0]


def fold_chain(c, us, orientation):
    """fold_chain (vrf_common.cuh:144-163) over k_com_me (orientation 0: c0 + u (c1 - c0)) or k_gen_fold
    (orientation 1: g1 + u (g0 - g1)), :52-66; odd levels are padded with a record of zero bytes."""
    c = list(c)
    for u in us:
        if len(c) % 2:
            c.append(ZERO_BYTES)
        if orientation == 0:
            c = [add(c[2 * i], jac_mul(add(c[2 * i + 1], neg(c[2 * i])), u)) for i in range(len(c) // 2)]
        else:
            c = [add(c[2 * i + 1], jac_mul(add(c[2 * i], neg(c[2 * i + 1])), u)) for i in range(len(c) // 2)]
    return c[0]


def ipa_prove(a, b, g, Q, tr):
    """ipa_prove (vrf_common.cuh:302-336).  Returns (L, R, a_final); tr is advanced as the reference advances it."""
    a, b, g = list(a), list(b), list(g)
    Ls, Rs = [], []
    while len(a) > 1:
        h = len(a) // 2
        ip = lambda x, y: sum(p * q for p, q in zip(x, y)) % FR_P
        Lp = add(msm_tree(g[h:], a[:h]), jac_mul(Q, ip(a[:h], b[h:])))
        Rp = add(msm_tree(g[:h], a[h:]), jac_mul(Q, ip(a[h:], b[:h])))
        tr.absorb("L", to_bytes(Lp))
        tr.absorb("R", to_bytes(Rp))
        x = tr.challenge_fr()
        xi = pow(x, FR_P - 2, FR_P)
        a = [(x * a[i] + xi * a[i + h]) % FR_P for i in range(h)]
        b = [(xi * b[i] + x * b[i + h]) % FR_P for i in range(h)]
        g = [add(jac_mul(g[i], xi), jac_mul(g[i + h], x)) for i in range(h)]
        Ls.append(Lp)
        Rs.append(Rp)
    return Ls, Rs, a[0]


def me_weights(u):
    """me_weights (vrf_common.cuh:205-216): b_k = prod_i (bit i of k ? u[i] : 1 - u[i])."""
    out = []
    for k in range(1 << len(u)):
        w = 1
        for i, ui in enumerate(u):
            w = w * (ui if (k >> i) & 1 else (1 - ui)) % FR_P
        out.append(w)
    return out


def same_point(p, q):
    """g1_eq (vrf_common.cuh:115-122): p - q is the point at infinity."""
    return add(p, neg(q))[2] == 0


def ipa_verify(g, Q, P0, u_b, Ls, Rs, a_final, tr):
    """ipa_verify (vrf_common.cuh:340-371): witness-free check of an argument against P0 = <g, a> + <a, b> Q."""
    rounds = len(Ls)
    if rounds != len(Rs) or len(g) != 1 << rounds or len(u_b) != rounds:
        return False
    b = me_weights(u_b)
    Pt, xs, xis = P0, [], []
    for r in range(rounds):
        tr.absorb("L", to_bytes(Ls[r]))
        tr.absorb("R", to_bytes(Rs[r]))
        x = tr.challenge_fr()
        xi = pow(x, FR_P - 2, FR_P)
        xs.append(x)
        xis.append(xi)
        Pt = add(add(jac_mul(Ls[r], x * x % FR_P), Pt), jac_mul(Rs[r], xi * xi % FR_P))
        h = len(b) // 2
        b = [(xi * b[k] + x * b[k + h]) % FR_P for k in range(h)]
    s = []
    for i in range(len(g)):
        w = 1
        for r in range(rounds):
            w = w * (xs[r] if (i >> (rounds - 1 - r)) & 1 else xis[r]) % FR_P
        s.append(w)
    g_f = msm_tree(g, s)
    return same_point(Pt, add(jac_mul(g_f, a_final), jac_mul(Q, a_final * b[0] % FR_P)))
