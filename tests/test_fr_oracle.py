"""The Python-integer restatement of the Fr path (oracle/fr_oracle.py) on CPU: its transcript against the
pinned fs::Transcript restatement and golden vectors, and the algebraic identities the reference's
prover asserts round by round."""
import random

import fr_oracle as fo


def test_transcript_matches_pinned_restatement(golden, orc):
    tr = fo.Transcript("p3-golden")
    assert tr.state.hex() == golden["transcript"][0]
    st = orc.tr_init("p3-golden")
    for label, n in [("z", 24), ("p0", 32), ("hp3", 32)]:
        data = bytes((len(label) * 11 + j) & 0xFF for j in range(n))
        tr.absorb(label, data)
        st = orc.tr_absorb(st, label, data)
        assert tr.state == st
        st, cb = orc.tr_challenge_bytes(st)
        assert tr.challenge_bytes() == cb and tr.state == st


def test_challenge_fr_mapping():
    tr = fo.Transcript("fr")
    t2 = fo.Transcript("fr")
    x = tr.challenge_fr()
    b = t2.challenge_bytes()
    limbs = [int.from_bytes(b[4 * i:4 * i + 4], "little") for i in range(8)]
    limbs[7] %= 1944954707
    assert x == sum(l << (32 * i) for i, l in enumerate(limbs)) and 0 < x < fo.P


def test_folds_agree_with_eq_tensor():
    rng = random.Random(3)
    u = [rng.randrange(fo.P) for _ in range(5)]
    t = [rng.randrange(fo.P) for _ in range(32)]
    E = fo.eq_build(u)
    assert fo.mle_eval(t, u) == sum(e * x for e, x in zip(E, t)) % fo.P
    # partial_me over [other=2][D=4][window=4] equals the eq-weighted sum over d
    t = [rng.randrange(fo.P) for _ in range(2 * 4 * 4)]
    out = fo.partial_me(t, 2, 2, 4, u[:2])
    E2 = fo.eq_build(u[:2])
    for o in range(2):
        for w in range(4):
            assert out[o * 4 + w] == sum(E2[d] * t[(o * 4 + d) * 4 + w] for d in range(4)) % fo.P


def test_product_sumcheck_round_identities():
    rng = random.Random(4)
    for nc in (2, 3, 4):
        cols = [[rng.randrange(fo.P) for _ in range(16)] for _ in range(nc)]
        claim = 0
        for i in range(16):
            p = 1
            for c in cols:
                p = p * c[i] % fo.P
            claim = (claim + p) % fo.P
        ev, ch, fin = fo.product_sumcheck(fo.Transcript("s"), cols, ["l%d" % t for t in range(nc + 1)])
        for e, x in zip(ev, ch):
            assert (e[0] + e[1]) % fo.P == claim
            claim = fo.lagrange(e, x)
        p = 1
        for f in fin:
            p = p * f % fo.P
        assert p == claim
        # finals are the columns' multilinear extensions at the reversed challenges
        assert fin[0] == fo.mle_eval(cols[0], list(reversed(ch)))
