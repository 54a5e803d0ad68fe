"""Canonical table artefacts of the fp8 transformer layer (the pinned public tables the reference's bf16 gadgets look
up: zkllm-src/transformer_ref.py:145-332, loaded by the C++ side as p3rms::Art, zkllm-src/p3_rmsnorm.cuh:55-82).

Every table is defined by exact integer rounding (round to nearest, ties to even) of a rational or of a float64 libm
value, so it is reproducible bit for bit; tests compare the tables with the reference's own generator and with committed
digests.  bf16 conventions: pattern = sign<<15 | biased exponent<<7 | 7 mantissa bits; exponent field 0 is zero
(subnormals flush), exponent 255 is an ordinary binade and results saturate at 0x7F7F.
"""
import math
import struct

import numpy as np

BF_MAXFIN = 0x7F7F
RMS_T = 16
SM_EMIN = 100
QE4M3_DEXP = 32
EPS_BITS = int(np.float32(1e-6).view(np.uint32))


def rne_bf16(s, m, t):
    """(-1)^s * m * 2^t with integer m > 0 -> bf16 pattern (round to nearest even, flush below the normal range,
    saturate above)."""
    w = m.bit_length()
    eb = t + w + 126
    if w > 8:
        sh = w - 8
        q, r = m >> sh, m & ((1 << sh) - 1)
        if 2 * r > (1 << sh) or (2 * r == (1 << sh) and q & 1):
            q += 1
            if q == 256:
                q, eb = 128, eb + 1
    else:
        q = m << (8 - w)
    if eb >= 255:
        return (s << 15) | BF_MAXFIN
    if eb <= 0:
        return s << 15
    return (s << 15) | (eb << 7) | (q - 128)


def bf_from_f64(x):
    """float64 -> bf16 pattern through its exact 53-bit significand."""
    if x == 0.0:
        return 0x8000 if math.copysign(1.0, x) < 0 else 0
    if math.isnan(x) or math.isinf(x):
        return BF_MAXFIN if (math.isnan(x) or x > 0) else 0x8000 | BF_MAXFIN
    fm, fe = math.frexp(abs(x))
    return rne_bf16(1 if x < 0 else 0, int(fm * (1 << 53)), fe - 53)


def bf_value(p):
    """pattern -> (sign, integer significand in [128, 256) or 0, exponent of its unit)."""
    s, e, mb = (p >> 15) & 1, (p >> 7) & 255, p & 127
    return (s, 0, 0) if e == 0 else (s, 128 + mb, e - 134)


def mul7_table():
    """Rounded product of two 8-bit significands: index (ma-128)<<7 | (mb-128) -> (mo-128, exponent increment 0..2)."""
    j = np.arange(16384, dtype=np.int64)
    mm = (128 + (j >> 7)) * (128 + (j & 127))
    c = (mm >= (1 << 15)).astype(np.int64)
    sh = 7 + c
    q, r, half = mm >> sh, mm & ((1 << sh) - 1), 1 << (sh - 1)
    q = q + ((r > half) | ((r == half) & ((q & 1) == 1)))
    carry = q == 256
    return np.where(carry, 0, q - 128).astype(np.uint8), (c + carry).astype(np.uint8)


def _round_ratio_sqrt(v, C):
    """nearest integer (ties to even) to 2^C / sqrt(v), exactly"""
    q = math.isqrt((1 << (2 * C)) // v)
    while (q + 1) * (q + 1) * v <= (1 << (2 * C)):
        q += 1
    edge = (2 * q + 1) ** 2 * v                     # (q + 1/2)^2 * v against 2^(2C), scaled by 4
    if edge < (1 << (2 * C + 2)) or (edge == (1 << (2 * C + 2)) and q & 1):
        q += 1
    return q


def rsq_table():
    """bf16 of 1/sqrt(u * 2^pp) for u in [2^15, 2^16), pp in {0, 1}: index pp<<15 | (u - 2^15) -> (mantissa bits, binade bit);
    the bf16 exponent field is 118 + binade bit."""
    mr, hb = np.zeros(65536, np.uint8), np.zeros(65536, np.uint8)
    for j in range(65536):
        v = (32768 + (j & 32767)) << (j >> 15)
        C, h = (15, 1) if v <= (1 << 16) else (16, 0)
        q = _round_ratio_sqrt(v, C)
        if q == 256:
            q, h = 128, h + 1
        if not (128 <= q < 256 and h < 2):
            raise AssertionError("rsq table out of range")
        mr[j], hb[j] = q - 128, h
    return mr, hb


def rcp_table():
    """bf16 of 1/u for u in [2^15, 2^16): index u - 2^15 -> (mantissa bits, binade bit); exponent field 111 + binade bit."""
    u = 32768 + np.arange(32768, dtype=np.int64)
    q, rem = (1 << 23) // u, (1 << 23) % u
    q = q + ((2 * rem > u) | ((2 * rem == u) & ((q & 1) == 1)))
    h = (q == 256).astype(np.int64)
    q = np.where(q == 256, 128, q)
    q[0], h[0] = 128, 1                              # u = 2^15: exactly 2^-15
    return (q - 128).astype(np.uint8), h.astype(np.uint8)


def _real(p):
    s, m, t = bf_value(p)
    return (-1.0 if s else 1.0) * m * 2.0 ** t


def exp_table():
    """bf16 of e^x for every bf16 pattern x (float64 libm exp, then exact rounding)."""
    out = np.zeros(65536, np.uint16)
    for p in range(65536):
        s, m, t = bf_value(p)
        if m == 0:
            out[p] = 0x3F80
        elif math.log2(m) + t > 7.1:
            out[p] = 0 if s else BF_MAXFIN
        else:
            out[p] = bf_from_f64(math.exp(_real(p)))
    return out


def silu_table():
    """bf16 of x / (1 + e^-x) for every bf16 pattern x."""
    out = np.zeros(65536, np.uint16)
    for p in range(65536):
        s, m, _ = bf_value(p)
        if m == 0:
            out[p] = s << 15
            continue
        x = _real(p)
        v = x if x > 30 else x * math.exp(x) if x < -85 else x / (1.0 + math.exp(-x))
        out[p] = bf_from_f64(v)
    return out


def qe4m3_table():
    """e4m3fn magnitude code nearest (ties to the even code) to (128 + mb)/128 * 2^(8 - dexp): index dexp<<7 | mb,
    dexp < 32.  Code c < 128 has magnitude (c & 7) * 2^-9 when its exponent field is 0, else (8 + (c & 7)) * 2^((c>>3) - 10);
    the all-ones code (NaN in e4m3fn) takes part like any other, as in the reference's table."""
    codes = np.arange(128, dtype=np.int64)
    e4, m4 = codes >> 3, codes & 7
    vm = np.where(e4 == 0, m4, m4 + 8)
    vt = np.where(e4 == 0, -9, e4 - 10)
    grid = vm << (vt + 9)                              # magnitudes in units of 2^-9
    tab = np.zeros(QE4M3_DEXP * 128, np.uint8)
    for j in range(QE4M3_DEXP * 128):
        dexp, mb = j >> 7, j & 127
        # (128 + mb) * 2^(1 - dexp) in units of 2^-9 = (128 + mb) * 2^(10 - dexp): scale both sides to keep integers
        up = max(dexp - 10, 0)
        val = (128 + mb) << (10 - dexp + up)
        d = np.abs((grid << up) - val)
        best = np.lexsort((codes, codes & 1, d))[0]
        tab[j] = best
    return tab


def epsa_table(ld):
    """(EMIN, table): table[E] = floor(eps * 2^(268 + ld - E)) for E in [EMIN, 512), 0 below; EMIN is the first E whose
    entry is below 2^18."""
    e, mb = (EPS_BITS >> 23) & 255, EPS_BITS & 0x7FFFFF
    em, et = (1 << 23) | mb, e - 150
    val = lambda E: em << (et + 268 + ld - E) if et + 268 + ld - E >= 0 else em >> (E - et - 268 - ld)
    emin = 0
    while val(emin) >= (1 << 18):
        emin += 1
    tab = np.zeros(512, np.int64)
    for E in range(emin, 512):
        tab[E] = val(E)
    return emin, tab


_FIXED = {}


def build_art(ld):
    """The artefact set for rows of 2^ld elements (p3rms::Art)."""
    if not _FIXED:
        mo, einc = mul7_table()
        rmr, rhb = rsq_table()
        cmr, chb = rcp_table()
        _FIXED.update(mul_mo=mo, mul_einc=einc, rsq_mr=rmr, rsq_hb=rhb, rcp_mr=cmr, rcp_hb=chb, exp_tab=exp_table(),
                      silu_tab=silu_table(), qe4m3=qe4m3_table())
    emin, epsa = epsa_table(ld)
    art = dict(_FIXED)
    art.update(ld=ld, EMIN=emin, T=RMS_T, eps_bits=EPS_BITS, sm_emin=SM_EMIN, epsa=epsa)
    return art


def art_bytes(art):
    """The artefact file the reference's loader reads (p3rms::load_art): 7 int64 header words 'RMST', 1, ld, EMIN, T, eps
    bits, softmax EMIN, then the tables in declaration order."""
    out = struct.pack("<7q", 0x524D5354, 1, art["ld"], art["EMIN"], art["T"], art["eps_bits"], art["sm_emin"])
    for k in ("mul_mo", "mul_einc", "rsq_mr", "rsq_hb", "rcp_mr", "rcp_hb"):
        out += art[k].astype(np.uint8).tobytes()
    out += art["epsa"].astype(np.int64).tobytes()
    out += art["exp_tab"].astype(np.uint16).tobytes() + art["silu_tab"].astype(np.uint16).tobytes()
    return out + art["qe4m3"].astype(np.uint8).tobytes()
