"""CPU evaluation of the programmable zero-check sumcheck with Python integers (test infrastructure): the
engine stand-in for gadget host logic, and the checker of the CUDA engine."""
import numpy as np

GL_P = 0xFFFFFFFF00000001


def zc_sumcheck(orc, st, tag, cols, terms, konst):
    """Sumcheck of cols[0] * (konst + sum coef * prod cols[idx]) + (terms flagged as outside the factor) with 5 evaluations per round, LSB-first binding,
    messages absorbed under `tag` (p3hwl::sc5_prove's schedule, zkllm-src/p3_hawkeye.cuh:641-700)."""
    cols = [[int(x) for x in c] for c in cols]
    terms = [(int(t[0]) % GL_P, tuple(t[1]), bool(len(t) > 2 and t[2])) for t in terms]
    konst = int(konst) % GL_P
    msgs, chals = [], []
    while len(cols[0]) > 1:
        h = len(cols[0]) // 2
        s = [0] * 5
        for i in range(h):
            lo = [c[2 * i] for c in cols]
            df = [c[2 * i + 1] - c[2 * i] for c in cols]
            for t in range(5):
                v = [(l + t * d) % GL_P for l, d in zip(lo, df)]
                acc, free = konst, 0
                for coef, idx, outside in terms:
                    p = coef
                    for k in idx:
                        p = p * v[k] % GL_P
                    if outside:
                        free += p
                    else:
                        acc += p
                s[t] = (s[t] + v[0] * (acc % GL_P) + free) % GL_P
        m = np.array(s, dtype=np.uint64)
        st = orc.tr_absorb(st, tag, m.tobytes())
        st, a = orc.tr_chal(st)
        msgs.append(s)
        chals.append(a)
        cols = [[(c[2 * i] + a * (c[2 * i + 1] - c[2 * i])) % GL_P for i in range(h)] for c in cols]
    return st, np.array(msgs, dtype=np.uint64), np.array(chals, dtype=np.uint64), np.array([c[0] for c in cols], dtype=np.uint64)
