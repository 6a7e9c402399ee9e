"""CPU oracle of the sampler and of the FP8 KV codec. TEST INFRASTRUCTURE: only tests/, the smoke check and the
bench's CPU-baseline leg may import it; the product path never does.

Restates the reference's own CPU reference, src/sampler/sampler.zig:112-250 (`reference`, `deviation`, `process`,
`filter`: bias, penalties and temperature in f32 - "the same f32 operations as the GPU, so these values match it
exactly" - then the filters and the draw in f64 over sorted values), and src/ref/fp8.zig:12-62 (`encode`, `decode`,
`rowScale`). Pinned by the reference's own test vectors (sampler.zig:252-300, fp8.zig:64-86) in tests/test_oracle.py."""
from __future__ import annotations

import numpy as np

GREEDY_BELOW = 1e-5  # sampler.zig:19


class Params:
    """sampler.Params (sampler.zig:26-38)."""

    def __init__(self, temperature=1.0, top_k=0, top_p=1.0, min_p=0.0, repetition_penalty=1.0, presence_penalty=0.0,
                 frequency_penalty=0.0, logit_bias=(), seed=0):
        self.temperature, self.top_k, self.top_p, self.min_p = np.float32(temperature), int(top_k), np.float32(top_p), np.float32(min_p)
        self.repetition_penalty = np.float32(repetition_penalty)
        self.presence_penalty, self.frequency_penalty = np.float32(presence_penalty), np.float32(frequency_penalty)
        self.logit_bias, self.seed = list(logit_bias), seed

    @property
    def greedy(self) -> bool:
        return bool(self.temperature < GREEDY_BELOW)

    def validate(self, vocab: int, max_bias: int = 1024) -> bool:
        """Params.validate (sampler.zig:42-56): vLLM's checks plus the list limits."""
        p = self
        ok = (p.temperature >= 0 and np.isfinite(p.temperature) and 0 < p.top_p <= 1 and 0 <= p.min_p <= 1
              and p.repetition_penalty > 0 and np.isfinite(p.repetition_penalty) and -2 <= p.presence_penalty <= 2
              and -2 <= p.frequency_penalty <= 2 and len(p.logit_bias) <= max_bias)
        if not ok:
            return False
        seen = set()
        for tok, b in p.logit_bias:
            if tok >= vocab or not np.isfinite(b) or tok in seen:
                return False
            seen.add(tok)
        return True

    def bias_words(self) -> np.ndarray:
        """Params.biasWords (sampler.zig:82-93): (token, f32 bits) pairs sorted by token."""
        rows = sorted((int(t), int(np.float32(b).view(np.uint32))) for t, b in self.logit_bias)
        return np.array(rows if rows else [(0, 0)], dtype=np.uint32).reshape(-1, 2)


def process(logits: np.ndarray, p: Params, prompt: np.ndarray, counts: np.ndarray) -> np.ndarray:
    """sampler.zig:171-183, every operation rounded to f32 in the same order."""
    l = np.array(logits, dtype=np.float32, copy=True)
    for tok, b in p.logit_bias:
        l[tok] = np.float32(l[tok] + np.float32(b))
    seen = prompt.astype(bool) | (counts != 0)
    pos = l > 0
    l = np.where(seen, np.where(pos, (l / p.repetition_penalty).astype(np.float32), (l * p.repetition_penalty).astype(np.float32)), l)
    l = (l - (p.frequency_penalty * counts.astype(np.float32)).astype(np.float32)).astype(np.float32)
    l = (l - (p.presence_penalty * (counts != 0).astype(np.float32)).astype(np.float32)).astype(np.float32)
    if not p.greedy:
        l = (l / p.temperature).astype(np.float32)
    return l


def _filter(l: np.ndarray, p: Params, slack: float):
    """sampler.zig:199-250: min-p, top-k and top-p over temperature-scaled logits, in f64. Returns (keep, e, z)."""
    n = l.size
    top = np.float64(l.max())
    e = np.exp(l.astype(np.float64) - top)
    keep = np.ones(n, dtype=bool)
    if p.min_p > 0:
        z = e.sum()
        keep = e / z >= np.float64(p.min_p) * (1 - slack) / z
    if p.top_k > 0:
        idx = np.flatnonzero(keep)
        if idx.size > p.top_k:
            kth = np.sort(l[idx])[::-1][p.top_k - 1]
            keep &= l >= kth
    if p.top_p < 1:
        idx = np.flatnonzero(keep)
        z = e[idx].sum()
        order = idx[np.argsort(-l[idx], kind="stable")]
        above = np.concatenate([[0.0], np.cumsum(e[order])[:-1]])
        stays = above / z < np.float64(p.top_p) * (1 + slack)   # monotone: a prefix of the order
        last = int(np.flatnonzero(stays)[-1])
        keep &= l >= l[order[last]]
    return keep, e, float(e[keep].sum())


def reference(logits, p: Params, prompt, counts, u: float) -> int:
    """sampler.zig:112-129."""
    l = process(logits, p, prompt, counts)
    if p.greedy:
        return int(np.argmax(l))          # the first maximum
    keep, e, z = _filter(l, p, 0.0)
    at = np.float64(np.float32(u)) * z
    idx = np.flatnonzero(keep)
    c = np.cumsum(e[idx])
    hit = np.flatnonzero(c > at)
    return int(idx[hit[0]] if hit.size else idx[-1])


def deviation(logits, p: Params, prompt, counts, u: float, token: int, slack: float) -> float:
    """sampler.zig:138-167: the distance from u to `token`'s CDF interval as a fraction of the kept mass, minimised
    over the min-p and top-p cuts moved by +-slack; 1 when the token is kept under none; greedy must match."""
    l = process(logits, p, prompt, counts)
    if p.greedy:
        return 0.0 if token == int(np.argmax(l)) else 1.0
    best = 1.0
    u = float(np.float32(u))
    for s in (0.0, slack, -slack):
        keep, e, z = _filter(l, p, s)
        if not keep[token]:
            continue
        lo = float(e[:token][keep[:token]].sum())
        a, b = lo / z, (lo + float(e[token])) / z
        best = min(best, a - u if u < a else (u - b if u >= b else 0.0))
    return best


# ---- FP8 E4M3FN (src/ref/fp8.zig)
FP8_MAX = 448.0


def fp8_encode(x) -> int:
    """fp8.zig:12-35: |x| <= 448 (clamped) -> bits, round to nearest, ties to even."""
    x = np.float32(x)
    sign = 0x80 if np.signbit(x) else 0
    a = np.float32(min(abs(float(x)), FP8_MAX))
    if a < np.float32(2.0 ** -6):
        s = np.float32(a * np.float32(512))
        q = int(np.floor(s))
        r = float(s) - q
        if r > 0.5 or (r == 0.5 and q & 1 == 1):
            q += 1
        return sign | q
    ab = int(a.view(np.uint32))
    e = (ab >> 23) - 120
    mant = ab & 0x7FFFFF
    q = mant >> 20
    rem = mant & 0xFFFFF
    if rem > 0x80000 or (rem == 0x80000 and q & 1 == 1):
        q += 1
    if q == 8:
        q, e = 0, e + 1
    return sign | min((e << 3) | q, 0x7E)


def fp8_decode(b: int) -> float:
    """fp8.zig:37-42."""
    e, m = (b >> 3) & 15, float(b & 7)
    mag = m * 2.0 ** -9 if e == 0 else (1 + m / 8) * 2.0 ** (e - 7)
    return float(np.float32(-mag if b & 0x80 else mag))


FP8_TABLE = np.array([fp8_decode(b) if b & 0x7F != 0x7F else np.nan for b in range(256)], dtype=np.float32)


def fp8_row_scale(row) -> float:
    """fp8.zig:47-55: the smallest power of two 2^k with max|row| <= 448 * 2^k; 1 for a zero or subnormal maximum."""
    m = np.float32(np.max(np.abs(np.asarray(row, dtype=np.float32)))) if len(row) else np.float32(0)
    bits = int(m.view(np.uint32))
    e = (bits >> 23) & 255
    if e == 0:
        return 1.0
    k = e - 127 - 8 + int((bits & 0x7FFFFF) > 0x600000)
    return float(2.0 ** k)
