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
