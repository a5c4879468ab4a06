"""CPU restatement of the arithmetic of metal/turboquant_qjl.metal (the reference's QJL shader).

TEST INFRASTRUCTURE ONLY: imported by tests/ as the checker of tq_qjl_compress / tq_qjl_dot_correction.

The shader is the only place the reference defines this variant (a dense +-1 projection, sign bits of the
projected residual, a popcount estimate of the inner product) and the reference ships no test or golden
vector for it: parity here is "the same arithmetic, statement by statement", pinned only by reading
(lines cited below), which is all a shader that cannot run on this machine allows.
"""
import numpy as np


def proj_sign(seed, rows, cols):
    """qjl_proj_sign (lines 39-44) for all (row, col): +1.0 / -1.0 as float32 [rows, cols]."""
    r = (np.arange(rows, dtype=np.uint64)[:, None] * 2654435761) & 0xFFFFFFFF
    c = (np.arange(cols, dtype=np.uint64)[None, :] * 2246822519) & 0xFFFFFFFF
    h = (np.uint64(seed & 0xFFFFFFFF) ^ r ^ c) & 0xFFFFFFFF
    h ^= h >> 16
    h = (h * 0x45D9F3B) & 0xFFFFFFFF
    return np.where(h & 1, np.float32(1.0), np.float32(-1.0)).astype(np.float32)


def compress(residual, proj_dim, seed):
    """tq_qjl_compress (lines 52-137). residual fp32 [tokens, heads, head_dim]."""
    r = np.asarray(residual, np.float32)
    tokens, heads, head_dim = r.shape
    words = (proj_dim + 31) // 32
    signs = np.zeros((tokens, heads, words), np.uint32)
    norms = np.zeros((tokens, heads), np.float32)
    S = proj_sign(seed, proj_dim, head_dim)
    for t in range(tokens):
        for h in range(heads):
            v = r[t, h]
            dot = np.zeros(proj_dim, np.float32)
            for c in range(head_dim):                       # lines 78-82: columns in order, fp32
                dot = (dot + S[:, c] * v[c]).astype(np.float32)
            buf = np.zeros(proj_dim, np.float32)             # lines 91-96
            m = min(head_dim, proj_dim)
            buf[:m] = (v[:m] * v[:m]).astype(np.float32)
            stride = proj_dim // 2
            while stride > 0:                               # lines 102-107
                buf[:stride] = (buf[:stride] + buf[stride:2 * stride]).astype(np.float32)
                stride >>= 1
            norms[t, h] = np.sqrt(buf[0], dtype=np.float32)
            bits = (dot >= 0).astype(np.uint32)             # line 117
            for w in range(words):
                seg = bits[32 * w: 32 * w + 32]
                signs[t, h, w] = np.uint32(sum(int(b) << i for i, b in enumerate(seg)))
    return signs, norms


def dot_correction(signs_q, signs_k, norms_k, head_idx, proj_dim):
    """tq_qjl_dot_correction (lines 163-216) -> fp32 [num_queries, num_keys]."""
    sq = np.asarray(signs_q, np.uint32)[:, head_idx]
    sk = np.asarray(signs_k, np.uint32)[:, head_idx]
    nk = np.asarray(norms_k, np.float32)[:, head_idx]
    x = ~(sq[:, None, :] ^ sk[None, :, :])
    matches = np.zeros(x.shape[:2], np.uint32)
    for w in range(x.shape[2]):
        matches += np.array([[bin(int(v)).count("1") for v in row] for row in x[:, :, w]], np.uint32)
    signed = (2 * matches).astype(np.float32) - np.float32(proj_dim)
    scale = np.float32(1.2533141) / np.float32(proj_dim)
    return ((scale * signed).astype(np.float32) * nk[None, :]).astype(np.float32)
