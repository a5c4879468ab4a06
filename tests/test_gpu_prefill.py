"""GPU parity of the prefill path: TurboQuantLinear.forward with many activation rows runs the
tensor-core GEMM (tcgen05 / tensor memory); it must agree with dequantize_weight_cpu + matmul
(the reference's ground truth for a linear layer, tests/integration/test_linear.cpp:82-145)
and with the decode (GEMV) path on the same rows."""
import numpy as np
import pytest

from tests.conftest import rel_l2

pytestmark = pytest.mark.gpu

LINEAR_TOL = 1e-3   # relative L2 of the layer output, fp32 accumulate (the stated tolerance)

CASES = [
    # rows, cols, block, activation rows, primary bits, residual bits, shared rotation
    (256, 512, 128, 256, 4, 4, True),      # exactly one tile
    (200, 1024, 128, 300, 4, 4, True),     # ragged weight rows and ragged activation rows, two tiles
    (130, 256, 64, 40, 4, 4, False),       # dual rotation: two passes over K, small batch
    (64, 896 + 128, 128, 77, 5, 3, True),  # 5+3-bit joint codes
    (48, 512, 512, 33, 4, 0, False),       # primary only, one WHT block spans several K blocks
    (384, 2048, 1024, 520, 4, 4, True),    # three row tiles x three activation tiles
    (128, 4096, 128, 40, 4, 4, True),      # one output tile: K split over 8 CTAs, partial sums added in order
    (130, 768, 64, 64, 4, 4, False),       # dual rotation with K split in 3: one split spans both planes
    (3584, 2048, 128, 64, 4, 4, True),     # 28 row tiles, K split in 4
]


@pytest.mark.parametrize("case", CASES, ids=[f"{c[0]}x{c[1]}_b{c[2]}_m{c[3]}_{c[4]}{c[5]}{'s' if c[6] else 'd'}" for c in CASES])
def test_prefill_gemm_matches_oracle(tq, oracle, case):
    rows, cols, bs, m, pb, rb, shared = case
    rng = np.random.default_rng(rows * 7 + cols + m)
    cbp, cbr = oracle.codebook(pb)[0], oracle.codebook(rb if rb else 4)[0]
    w = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float16).astype(np.float32)
    pp, pr, norms, seeds = oracle.quantize_weight(w, cbp, cbr, pb, rb, bs, shared)
    deq = oracle.dequantize_weight(pp, pr, norms, seeds, cbp, cbr, bs)
    x = rng.standard_normal((m, cols)).astype(np.float16)
    want = oracle.linear_from_dequant(deq, x.astype(np.float32))
    lin = tq.TurboQuantLinear(cols, rows, tq.QuantizedWeight(pp, pr, norms, seeds), tq.codebook_from_centroids(cbp),
                              tq.codebook_from_centroids(cbr), bs)
    y = lin.forward(x)
    assert y.dtype == np.float16 and y.shape == (m, rows)
    assert np.all(np.isfinite(y.astype(np.float32)))
    assert rel_l2(y, want) < LINEAR_TOL, rel_l2(y, want)
    # per activation row as well: no row of the tile may be off
    num = np.linalg.norm(y.astype(np.float64) - want, axis=1)
    den = np.linalg.norm(want.astype(np.float64), axis=1) + 1e-30
    assert np.max(num / den) < 3 * LINEAR_TOL, float(np.max(num / den))
    # the decode path on the first rows agrees to the same tolerance
    y8 = lin.forward(x[:8])
    assert rel_l2(y[:8], y8.astype(np.float32)) < LINEAR_TOL
    # run-to-run identical
    y2 = lin.forward(x)
    assert np.array_equal(y.view(np.uint16), y2.view(np.uint16))
    lin.close()


def test_prefill_falls_back_when_k_is_not_a_multiple_of_64(tq, oracle):
    """in_features = 96 cannot feed 64-column K blocks: the call still succeeds (passes of 8
    through the decode kernel)."""
    rng = np.random.default_rng(3)
    cb = oracle.codebook(4)[0]
    w = (rng.standard_normal((40, 96)) * 0.02).astype(np.float16).astype(np.float32)
    pp, pr, norms, seeds = oracle.quantize_weight(w, cb, cb, 4, 4, 32, True)
    deq = oracle.dequantize_weight(pp, pr, norms, seeds, cb, cb, 32)
    x = rng.standard_normal((50, 96)).astype(np.float16)
    lin = tq.TurboQuantLinear(96, 40, tq.QuantizedWeight(pp, pr, norms, seeds), tq.codebook_from_centroids(cb),
                              tq.codebook_from_centroids(cb), 32)
    y = lin.forward(x)
    assert rel_l2(y, oracle.linear_from_dequant(deq, x.astype(np.float32))) < LINEAR_TOL
    lin.close()


def test_prefill_device_tensors_and_status(tq, oracle):
    """Device-resident x and y on a side stream (no host round trip), then the status query."""
    import torch
    rng = np.random.default_rng(5)
    cb = oracle.codebook(4)[0]
    rows, cols, m = 256, 1024, 384
    w = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float16).astype(np.float32)
    pp, pr, norms, seeds = oracle.quantize_weight(w, cb, cb, 4, 4, 128, True)
    deq = oracle.dequantize_weight(pp, pr, norms, seeds, cb, cb, 128)
    lin = tq.TurboQuantLinear(cols, rows, tq.QuantizedWeight(pp, pr, norms, seeds), tq.codebook_from_centroids(cb),
                              tq.codebook_from_centroids(cb), 128)
    xh = rng.standard_normal((m, cols)).astype(np.float16)
    x = torch.from_numpy(xh).cuda()
    y = torch.empty((m, rows), dtype=torch.float16, device="cuda")
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        lin.forward(x, out=y, stream=st)
        lin.forward(x, out=y, stream=st)      # scratch reuse on the second call
    st.synchronize()
    lin.check_status()
    assert rel_l2(y.cpu().numpy(), oracle.linear_from_dequant(deq, xh.astype(np.float32))) < LINEAR_TOL
    lin.close()
