"""Plain sampler: the order and the cuts of mashbox-labs/mashbox's sampler (src/mashbox/runtime/sampler.py), in NumPy,
one row at a time, with sorting where the reference bisects.  The random draw is Gumbel-max like the reference's
(sampler.py:130-133); the reference keys threefry by (seed, token index), this engine keys Philox4x32-10 by the seed and
counts by (vocabulary index, token index) -- the generator is this engine's own, so it is restated here bit for bit.
"""
import numpy as np

M0, M1 = 0xD2511F53, 0xCD9E8D57
W0, W1 = 0x9E3779B9, 0xBB67AE85
MASK = 0xFFFFFFFF


def philox_word(seed, index, step):
    """first output word of Philox4x32-10 with key = the 64-bit seed's (low, high) words, counter (index, step, 0, 0)"""
    k0, k1 = seed & MASK, (seed >> 32) & MASK
    c = [index & MASK, step & MASK, 0, 0]
    for _ in range(10):
        p0, p1 = M0 * c[0], M1 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k0) & MASK, p1 & MASK, ((p0 >> 32) ^ c[3] ^ k1) & MASK, p0 & MASK]
        k0, k1 = (k0 + W0) & MASK, (k1 + W1) & MASK
    return c[0]


def gumbel(word):
    u = (np.float32(word >> 8) + np.float32(0.5)) * np.float32(1.0 / 16777216.0)
    return -np.log(-np.log(u, dtype=np.float32), dtype=np.float32)


def penalise(lg, cnt, seen, rep, freq, pres):
    """sampler.py:78-83: repetition penalty on seen tokens (positive logits divided, negative multiplied), then minus
    freq x count of generated tokens, minus pres where the count is positive"""
    lg = np.asarray(lg, np.float32)
    x = np.where(seen, np.where(lg > 0, lg / np.float32(rep), lg * np.float32(rep)), lg)
    x = x - np.float32(freq) * cnt.astype(np.float32)
    return (x - np.float32(pres) * (cnt > 0).astype(np.float32)).astype(np.float32)


def softmax(x):
    e = np.exp((x - x.max()).astype(np.float64))
    return e / e.sum()


def transform(x, temperature, top_k=0, top_p=1.0, min_p=0.0):
    """sampler.py:136-157: temperature -> top_k -> top_p -> min_p; cut tokens become -inf; ties at a cut are kept"""
    x = (np.asarray(x, np.float32) / np.float32(temperature if temperature > 0 else 1.0)).astype(np.float32)
    if top_k > 0:
        kth = np.sort(x)[::-1][min(top_k, len(x)) - 1]
        x = np.where(x < kth, -np.inf, x).astype(np.float32)
    if top_p < 1.0:
        p = softmax(x)
        # smallest value t with mass(x > t) < top_p (sampler.py:107-120); keeping x >= t keeps the smallest set of top
        # tokens whose mass reaches top_p, ties included
        cut = next(v for v in np.unique(x) if p[x > v].sum() < top_p)
        x = np.where(x < cut, -np.inf, x).astype(np.float32)
    if min_p > 0.0:
        p = softmax(x)
        x = np.where(p < min_p * p.max(), -np.inf, x).astype(np.float32)
    return x


def draw(x, seed, step):
    """sampler.py:130-133 with this engine's generator: argmax(x + Gumbel), lowest index at a tie"""
    best, arg = -np.inf, -1
    for v in range(len(x)):
        if x[v] == -np.inf:
            continue
        s = np.float32(x[v]) + gumbel(philox_word(seed, v, step))
        if s > best:
            best, arg = s, v
    return arg


def sample(lg, temperature=0.0, top_k=0, top_p=1.0, min_p=0.0, rep=1.0, freq=0.0, pres=0.0, seed=0, step=0,
           cnt=None, seen=None):
    V = len(lg)
    cnt = np.zeros(V, np.int32) if cnt is None else cnt
    seen = np.zeros(V, bool) if seen is None else seen
    x = penalise(lg, cnt, seen, rep, freq, pres)
    if temperature <= 0:
        return int(np.argmax(x))              # sampler.py:125-127: greedy on the processed logits; first maximum
    return draw(transform(x, temperature, top_k, top_p, min_p), seed, step)
