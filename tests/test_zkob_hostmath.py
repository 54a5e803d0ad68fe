"""The host-side field arithmetic of the driver programs (zk-hillclimb_b200/host/zkob_common.hpp, behind the line program
zkob_hostmath) against exact Python integers: add, sub, mul, inverse, the signed lift, the Lagrange evaluations of the degree-2, -3
and -4 round polynomials and the one-variable eq factor.  No GPU."""
import os
import random
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "zk-hillclimb_b200", "zkob_hostmath")
P = 0x73EDA753299D7D483339D80809A1D80553BDA402FFFE5BFEFFFFFFFF00000001


def ask(lines):
    r = subprocess.run([EXE], input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    return [int(x, 16) for x in r.stdout.split()]


def lagrange(ps, v):
    """The value at v of the polynomial through (i, ps[i])."""
    acc = 0
    for i, pi in enumerate(ps):
        num, den = 1, 1
        for j in range(len(ps)):
            if j != i:
                num = num * (v - j) % P
                den = den * (i - j) % P
        acc = (acc + pi * num * pow(den, P - 2, P)) % P
    return acc


def test_field_operations_against_python_integers():
    assert os.path.exists(EXE), "build() makes the program"
    rng = random.Random(5)
    edge = [0, 1, 2, P - 1, P - 2, (P + 1) // 2, (1 << 255) % P, 0xFFFFFFFF, 1 << 32, (1 << 64) - 1]
    vals = edge + [rng.randrange(P) for _ in range(40)]
    lines, want = [], []
    for a in vals[:25]:
        for b in (vals[0], vals[3], rng.choice(vals), rng.randrange(P)):
            lines += ["add %x %x" % (a, b), "sub %x %x" % (a, b), "mul %x %x" % (a, b), "eq1 %x %x" % (a, b)]
            want += [(a + b) % P, (a - b) % P, a * b % P, (a * b + (1 - a) * (1 - b)) % P]
    for a in vals[1:20]:
        lines.append("inv %x" % a)
        want.append(pow(a, P - 2, P))
    for x in (0, 1, -1, 65536, -65536, (1 << 63) - 1, -(1 << 63), -123456789012345):
        lines.append("i64 %d" % x)
        want.append(x % P)
    assert ask(lines) == want


def test_round_polynomial_evaluations_against_lagrange_interpolation():
    rng = random.Random(9)
    lines, want = [], []
    for n, op in ((3, "lag3"), (4, "lag4"), (5, "lag5")):
        for _ in range(12):
            ps = [rng.randrange(P) for _ in range(n)]
            v = rng.choice([0, 1, n - 1, n, P - 1, rng.randrange(P), rng.randrange(P)])
            lines.append(op + " " + " ".join("%x" % x for x in ps + [v]))
            want.append(lagrange(ps, v))
    assert ask(lines) == want
