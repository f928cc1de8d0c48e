"""Second, independent restatement of the reference's arithmetic in numpy (small shapes only).

TEST INFRASTRUCTURE ONLY.  It exists to cross-check oracle/qw3_oracle.cpp: the two share no
code.  numpy evaluates float16 arithmetic as one float32 operation followed by one rounding to
float16, which is what __hadd/__hsub/__hmul produce.  PARITY UNPINNED, as for the C++ oracle.
"""
import numpy as np

_GOLD = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)


def mix64(x):
    with np.errstate(over="ignore"):
        x = np.asarray(x, np.uint64) + _GOLD
        z = (x ^ (x >> np.uint64(30))) * _M1
        z = (z ^ (z >> np.uint64(27))) * _M2
        return z ^ (z >> np.uint64(31))


def stream_key(seed, tag):
    return mix64(np.uint64(seed) ^ mix64(np.uint64(tag) ^ np.uint64(0xA5A5A5A55A5A5A5A)))


def draw(key, k):
    with np.errstate(over="ignore"):
        return mix64(key + np.asarray(k, np.uint64) * _GOLD)


def gen_codes(seed, tag, n_bytes):
    key = stream_key(seed, tag)
    words = draw(key, np.arange((n_bytes + 7) // 8, dtype=np.uint64))
    return words.view(np.uint8)[:n_bytes].copy()  # little-endian: byte b of word w = (r >> 8b) & 255


def gen_uniform_int_f16(seed, tag, n, lo, hi):
    r = draw(stream_key(seed, tag), np.arange(n, dtype=np.uint64))
    return (lo + (r % np.uint64(hi - lo + 1)).astype(np.int64)).astype(np.float16)


def gen_tokens(seed, tag, n, vocab):
    r = draw(stream_key(seed, tag), np.arange(n, dtype=np.uint64))
    return (r % np.uint64(vocab)).astype(np.int32)


def gen_normal(seed, tag, n):
    key = stream_key(seed, tag)
    k = np.arange(n, dtype=np.uint64)
    u1 = ((draw(key, 2 * k) >> np.uint64(11)).astype(np.float64) + 0.5) / 9007199254740992.0
    u2 = ((draw(key, 2 * k + np.uint64(1)) >> np.uint64(11)).astype(np.float64) + 0.5) / 9007199254740992.0
    return np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)


def unpack_nibbles(packed, rows, cols):
    """Inference.cu:92-99: element (r, c) is the low nibble of byte r*ceil(cols/2)+c/2 for even c."""
    pc = (cols + 1) // 2
    b = packed[: rows * pc].reshape(rows, pc)
    q = np.empty((rows, pc * 2), np.uint8)
    q[:, 0::2] = b & 15
    q[:, 1::2] = b >> 4
    return q[:, :cols]


def dequant(packed, scale, zp, rows, cols, group=128):
    """Inference.cu:84-105 with the group index wrapped to the allocated length."""
    q = unpack_nibbles(packed, rows, cols).astype(np.float16)
    g = (np.arange(cols) // group) % scale.size
    sub = q - zp.astype(np.float16)[g][None, :]           # __hsub
    return sub * scale.astype(np.float16)[g][None, :]     # __hmul


def gemv(packed, scale, zp, M, K, x, group=128):
    """Inference.cu:1052-1065: the row-major dequant buffer read column-major with lda = M."""
    wflat = dequant(packed, scale, zp, M, K, group).reshape(-1)
    a = wflat.reshape(K, M).T.astype(np.float64)          # a[i, j] = wflat[i + j*M]
    return a @ x.astype(np.float64)


def group_index_bruteforce(M, K, group, n_alloc):
    """g[i, j] for flat element f = i + j*M: ((f mod K) / group) mod n_alloc."""
    i = np.arange(M, dtype=np.int64)[:, None]
    j = np.arange(K, dtype=np.int64)[None, :]
    return (((i + j * M) % K) // group) % n_alloc


def group_index_blocked(M, K, group, n_alloc):
    """The closed form the kernels use: ((i/group + j*(M/group)) mod (K/group)) mod n_alloc."""
    ib = (np.arange(M, dtype=np.int64) // group)[:, None]
    j = np.arange(K, dtype=np.int64)[None, :]
    return ((ib + j * (M // group)) % (K // group)) % n_alloc


def rmsnorm(x, gamma, eps=1e-6):
    xf = x.astype(np.float32)
    mean_sq = np.float32(np.sum(xf.astype(np.float64) ** 2)) / np.float32(x.size)
    scale = np.float16(np.float32(1.0) / np.sqrt(mean_sq + np.float32(eps)))
    return (x * scale) * gamma


def rope(qk, heads, head_dim, cos_t, sin_t, pos):
    v = qk.reshape(heads, head_dim // 2, 2).astype(np.float16)
    c = cos_t[pos][None, :].astype(np.float16)
    s = sin_t[pos][None, :].astype(np.float16)
    x0, x1 = v[:, :, 0].astype(np.float64), v[:, :, 1].astype(np.float64)
    c, s = c.astype(np.float64), s.astype(np.float64)
    r16 = lambda a: a.astype(np.float16).astype(np.float64)
    # as the reference's build executes Inference.cu:172-173: the first product of each line is contracted into
    # the add (fma, exact in float64 here), the second product is rounded to fp16 first
    t0 = (x0 * c - r16(x1 * s)).astype(np.float16)
    t1 = (x0 * s + r16(x1 * c)).astype(np.float16)
    return np.stack([t0, t1], axis=-1).reshape(-1)


def attention(q, k_cache, v_cache, heads, head_dim, max_pos, length):
    q = q.reshape(heads, head_dim).astype(np.float64)
    k = k_cache.reshape(heads, max_pos, head_dim)[:, :length].astype(np.float64)
    v = v_cache.reshape(heads, max_pos, head_dim)[:, :length].astype(np.float64)
    s = np.einsum("hd,hkd->hk", q, k) / np.sqrt(head_dim)
    p = np.exp(s - s.max(axis=1, keepdims=True))
    p /= p.sum(axis=1, keepdims=True)
    return np.einsum("hk,hkd->hd", p, v).reshape(-1)


def gelu(x):
    import math
    v = x.astype(np.float64)
    erf = np.vectorize(math.erf)
    return 0.5 * v * (1.0 + erf(v * 0.70710678))
