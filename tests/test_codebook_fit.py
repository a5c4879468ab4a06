"""Lloyd-Max fit on the device and the converter's per-layer rules.

CPU: the three converter rules (adaptive block size, layer index, sensitive layers) against the
reference's definitions (src/converter.cpp:52-59, 81-93, 228-240).  GPU: tq_codebook_fit against the CPU
checker's generate_codebook_from_data (oracle/tq_oracle.c, pinned to the reference bit for bit), and
the per-layer fit against samples built with the checker's own rotation."""
import numpy as np
import pytest

import turboquant_mlx_core_b200 as tq


def test_adaptive_block_size_rule():
    tq.load()
    for in_f, mx in [(3584, 512), (18944, 512), (27648, 1024), (4096, 128), (96, 512), (7, 512), (1024, 32), (5120, 1 << 19)]:
        best = 1
        for p in range(1, 20):
            c = 1 << p
            if c > mx:
                break
            if in_f % c == 0:
                best = c
        assert tq.adaptive_block_size(in_f, mx) == best


def test_layer_index_and_sensitive_layers():
    tq.load()
    assert tq.layer_index("model.layers.12.self_attn.q_proj.weight") == 12
    assert tq.layer_index("model.layers.0.mlp.down_proj.weight") == 0
    assert tq.layer_index("lm_head.weight") == -1
    assert tq.layer_index("model.layers.x.foo") == -1
    assert tq.layer_index("a.layers.notanumber.b.layers.7.c") == 7
    assert tq.layer_index("model.layers.5") == -1            # the pattern wants a dot on both sides
    got = [tq.is_sensitive_layer(i, 31, 2, 3) for i in range(-1, 32)]
    want = [False] + [i < 2 or i > 31 - 3 for i in range(32)]
    assert got == want


@pytest.fixture(scope="module")
def gpu():
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    tq.load()
    return torch


@pytest.mark.gpu
@pytest.mark.parametrize("bits,n,dist", [(4, 100_000, "normal"), (3, 70_000, "skewed"), (2, 65_536, "normal"), (5, 300_000, "normal"),
                                         (1, 1000, "normal"), (4, 3_000_000, "residual"), (4, 17, "normal")])
def test_fit_matches_checker(gpu, oracle, bits, n, dist):
    """Same centroids as the reference's CPU fit (double sums, lower_bound bins): the device sums the same
    doubles in another order, so a centroid may differ in its last bit; bins and iteration counts agree."""
    rng = np.random.default_rng(bits * 1000 + n)
    if dist == "normal":
        data = rng.standard_normal(n).astype(np.float32)
    elif dist == "skewed":
        data = (rng.gamma(2.0, 1.0, n) - 1.5).astype(np.float32)
    else:
        x = rng.standard_normal(n).astype(np.float32)
        cb = tq.generate_codebook(4)
        data = (x - cb.centroids[np.searchsorted(cb.boundaries, x, side="left")]).astype(np.float32)
    want_c, want_b = oracle.fit_codebook(data, bits, 100)
    got = tq.generate_codebook_from_data(data, bits, 100)
    assert np.allclose(got.centroids, want_c, rtol=3e-6, atol=3e-7), np.abs(got.centroids - want_c).max()
    assert np.allclose(got.boundaries, want_b, rtol=3e-6, atol=3e-7)
    assert np.all(np.diff(got.centroids) > 0)
    again = tq.generate_codebook_from_data(gpu.from_numpy(data).cuda(), bits, 100)
    assert np.array_equal(again.centroids.view(np.uint32), got.centroids.view(np.uint32))     # run-to-run and host/device identical


@pytest.mark.gpu
def test_fit_edge_cases(gpu, oracle):
    """No data gives the analytic codebook; zero iterations too; constant data leaves empty bins where they were;
    a value exactly on a boundary goes to the lower bin."""
    cb = tq.generate_codebook(3)
    assert np.array_equal(tq.generate_codebook_from_data(np.zeros(0, np.float32), 3).centroids, cb.centroids)
    assert np.array_equal(tq.generate_codebook_from_data(np.ones(10, np.float32), 3, 0).centroids, cb.centroids)
    const = np.full(1000, 0.3, np.float32)
    want_c, _ = oracle.fit_codebook(const, 3, 100)
    got, run = tq.generate_codebook_from_data(const, 3, 100, return_iterations=True)
    assert np.array_equal(got.centroids, want_c) and run >= 1
    b = cb.boundaries[3]
    tie = np.array([b] * 64 + [cb.centroids[0]] * 3, np.float32)
    want_c, _ = oracle.fit_codebook(tie, 3, 1)
    assert np.array_equal(tq.generate_codebook_from_data(tie, 3, 1).centroids, want_c)
    with pytest.raises(ValueError):
        tq.generate_codebook_from_data(const, 6)


@pytest.mark.gpu
@pytest.mark.parametrize("out_f,in_f,block", [(256, 512, 128), (96, 1024, 512), (64, 96, 32)])
def test_layer_fit_matches_checker_on_the_quantisers_samples(gpu, oracle, out_f, in_f, block):
    """Primary codebook fitted to sqrt(in) * WHT(row / |row|), residual codebook to what the shared analytic
    primary codebook leaves (src/converter.cpp:303-368); the samples come from the checker's rotation."""
    rng = np.random.default_rng(out_f + in_f)
    w = (rng.standard_normal((out_f, in_f)) * 0.02).astype(np.float32)
    w[3] *= 5.0
    cb = tq.generate_codebook(4)
    qw = tq.quantize_weight(w, cb, cb, tq.QuantizerConfig(4, 4, block, True))
    # row norms summed left to right in fp32, as the quantiser does (src/quantizer.cpp:43-49 on the CPU path)
    norms = np.maximum(np.sqrt(np.cumsum(w * w, axis=1, dtype=np.float32)[:, -1]), np.float32(1e-10))
    scaled = oracle.wht(w / norms[:, None], int(qw.seeds[0]), block) * np.float32(np.sqrt(np.float32(in_f)))
    flat = scaled.reshape(-1).astype(np.float32)
    resid = (flat - cb.centroids[np.searchsorted(cb.boundaries, flat, side="left")]).astype(np.float32)
    want_p, _ = oracle.fit_codebook(flat, 4, 100)
    want_r, _ = oracle.fit_codebook(resid, 4, 100)
    got_p, got_r = tq.fit_layer_codebooks(w, block, 4, 4, 100)
    assert np.allclose(got_p.centroids, want_p, rtol=3e-6, atol=3e-7), np.abs(got_p.centroids - want_p).max()
    assert np.allclose(got_r.centroids, want_r, rtol=3e-6, atol=3e-7), np.abs(got_r.centroids - want_r).max()
    only_p, none_r = tq.fit_layer_codebooks(gpu.from_numpy(w).cuda(), block, 4, 0, 100)
    assert none_r is None and np.array_equal(only_p.centroids.view(np.uint32), got_p.centroids.view(np.uint32))
