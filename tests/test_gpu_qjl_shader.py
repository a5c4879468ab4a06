"""tq_qjl_compress / tq_qjl_dot_correction against the statement-by-statement restatement of
metal/turboquant_qjl.metal (oracle/qjl_shader.py): sign words, norms and corrections bit for bit."""
import numpy as np
import pytest

from oracle import qjl_shader


@pytest.mark.gpu
@pytest.mark.parametrize("tokens,heads,head_dim,proj_dim", [(5, 2, 128, 128), (3, 4, 64, 256), (4, 1, 128, 32), (2, 3, 32, 16), (1, 1, 256, 1024)])
def test_qjl_shader_kernels_bit_exact(tq, tokens, heads, head_dim, proj_dim):
    rng = np.random.default_rng(tokens * 1000 + proj_dim)
    resid = (rng.standard_normal((tokens, heads, head_dim)) * 0.1).astype(np.float32)
    resid[0, 0, :3] = 0.0
    seed = int(rng.integers(1 << 32))
    want_s, want_n = qjl_shader.compress(resid, proj_dim, seed)
    got_s, got_n = tq.qjl_compress(resid, proj_dim, seed)
    assert np.array_equal(got_s, want_s)
    assert np.array_equal(got_n.view(np.uint32), want_n.view(np.uint32))
    q = (rng.standard_normal((2, heads, head_dim)) * 0.1).astype(np.float32)
    q_s, _ = tq.qjl_compress(q, proj_dim, seed)
    for head in range(heads):
        want_c = qjl_shader.dot_correction(q_s, want_s, want_n, head, proj_dim)
        got_c = tq.qjl_dot_correction(q_s, got_s, got_n, head, proj_dim)
        assert np.array_equal(got_c.view(np.uint32), want_c.view(np.uint32))


def test_qjl_shader_projection_is_rank_one():
    """A property of the shader's hash that its users should know: the sign of entry (row, col) is bit 0 of
    (h ^ h >> 16) * odd with h = seed ^ row * A ^ col * B, i.e. bit0 ^ bit16 of an XOR of a row term and a column
    term, so sign(row, col) = a(row) * b(col).  Every projection of a vector is therefore +- the same number and the
    sign word of a vector is one fixed pattern or its complement."""
    S = qjl_shader.proj_sign(99, 64, 128)
    assert np.all(S * S[0:1, :] * S[:, 0:1] * S[0, 0] == 1)
    assert np.linalg.matrix_rank(S) == 1
    rng = np.random.default_rng(0)
    signs, _ = qjl_shader.compress(rng.standard_normal((6, 1, 128)).astype(np.float32), 32, 99)
    words = set(int(w) for w in signs.ravel())
    assert len(words) <= 2 and (len(words) < 2 or (min(words) ^ max(words)) == 0xFFFFFFFF)


def test_qjl_shader_checker_signs_are_hash_bits():
    s = qjl_shader.proj_sign(123, 4, 5)
    h = (123 ^ ((2 * 2654435761) & 0xFFFFFFFF) ^ ((3 * 2246822519) & 0xFFFFFFFF)) & 0xFFFFFFFF
    h ^= h >> 16
    h = (h * 0x45D9F3B) & 0xFFFFFFFF
    assert s[2, 3] == (1.0 if h & 1 else -1.0)
    signs, norms = qjl_shader.compress(np.ones((1, 1, 4), np.float32), 8, 7)
    assert norms[0, 0] == 2.0 and signs.shape == (1, 1, 1)
