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


@pytest.mark.gpu
def test_qjl_shader_estimate_tracks_the_inner_product(tq):
    """What the correction is for: over many keys, sqrt(pi/2)/m * <sign(Sq), sign(Sr)> * |r| follows <q, r> / |q|."""
    rng = np.random.default_rng(3)
    resid = rng.standard_normal((300, 1, 128)).astype(np.float32)
    q = rng.standard_normal((1, 1, 128)).astype(np.float32)
    k_s, k_n = tq.qjl_compress(resid, 1024, 99)
    q_s, _ = tq.qjl_compress(q, 1024, 99)
    est = tq.qjl_dot_correction(q_s, k_s, k_n, 0, 1024)[0]
    true = resid[:, 0] @ q[0, 0] / np.linalg.norm(q)
    assert np.corrcoef(est, true)[0, 1] > 0.7


def test_qjl_shader_checker_signs_are_hash_bits():
    s = qjl_shader.proj_sign(123, 4, 5)
    h = (123 ^ ((2 * 2654435761) & 0xFFFFFFFF) ^ ((3 * 2246822519) & 0xFFFFFFFF)) & 0xFFFFFFFF
    h ^= h >> 16
    h = (h * 0x45D9F3B) & 0xFFFFFFFF
    assert s[2, 3] == (1.0 if h & 1 else -1.0)
    signs, norms = qjl_shader.compress(np.ones((1, 1, 4), np.float32), 8, 7)
    assert norms[0, 0] == 2.0 and signs.shape == (1, 1, 1)
