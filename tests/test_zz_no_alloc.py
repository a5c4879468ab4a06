"""GPU test of tq_linear_forward_noalloc, the forward pass that allocates nothing.

It is for callers that cannot let a library allocate: a server that has handed the rest of
the GPU's memory to its own pool, or code running inside an open stream capture.  The entry
takes device pointers only and draws its working memory from a fixed 2 MiB array built into
the library, shared by all calls on the device — so the test calls it twice in a row (the
second call finds the first one's leftovers in that array) and checks both results bit for bit
against the ordinary tq_linear_forward on the same inputs and, within the linear tolerance,
against the CPU checker; it also checks that the device's free memory did not shrink.
Collected last on purpose: a run that stops at the first failure has then already run every
other test.
"""
import ctypes as C

import numpy as np
import pytest

from tests.conftest import rel_l2

pytestmark = pytest.mark.gpu

LINEAR_TOL = 1e-3   # the tolerance of the linear-forward parity tests


def _layer(tq, oracle, rows, cols, block, shared, seed, with_dequant=False):
    rng = np.random.default_rng(seed)
    cb = oracle.codebook(4)[0]
    w = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float16).astype(np.float32)
    pp, pr, norms, seeds = oracle.quantize_weight(w, cb, cb, 4, 4, block, shared)
    c = tq.codebook_from_centroids(cb)
    lin = tq.TurboQuantLinear(cols, rows, tq.QuantizedWeight(pp, pr, norms, seeds), c, c, block)
    if with_dequant:
        return lin, oracle.dequantize_weight(pp, pr, norms, seeds, cb, cb, block)
    return lin


@pytest.mark.parametrize("rows,cols,block,shared,batch", [
    (300, 8192, 128, True, 3),     # two column chunks: partial sums and arrival counters in the array
    (512, 1024, 256, False, 8),    # dual rotation: two planes
    (4096, 4096, 128, True, 1),    # the headline shape
    (96, 2048, 512, True, 2),      # WHT block above 256: the rotated activation goes through the array too
    (40, 5120, 1024, False, 5),    # the same with two planes and two column chunks
])
def test_noalloc_forward_matches_ordinary_forward_twice(tq, oracle, rows, cols, block, shared, batch):
    torch = pytest.importorskip("torch")
    L = tq.load()
    lin, deq = _layer(tq, oracle, rows, cols, block, shared, seed=rows + cols, with_dequant=True)
    g = torch.Generator(device="cuda").manual_seed(3)
    xs = [torch.randn((batch, cols), generator=g, device="cuda").half() for _ in range(2)]
    free_before = None
    for x in xs:                                   # two calls in a row share the built-in array
        want = lin.forward(x)
        got = torch.full((batch, rows), float("nan"), device="cuda", dtype=torch.float16)
        torch.cuda.synchronize()
        if free_before is None:
            free_before = torch.cuda.mem_get_info()[0]
        rc = L.tq_linear_forward_noalloc(lin.handle, C.c_void_p(x.data_ptr()), batch, C.c_void_p(got.data_ptr()), None)
        assert rc == 0, L.tq_last_error().decode()
        torch.cuda.synchronize()
        assert torch.isfinite(got).all()
        # same kernels, same summation order, only the scratch pointer differs: the bits must agree
        assert torch.equal(got, want)
        ref = oracle.linear_from_dequant(deq, x.float().cpu().numpy())
        assert rel_l2(got.float().cpu().numpy(), ref) < LINEAR_TOL
    # neither call took memory from the device (the first one only looked up the array's address)
    assert torch.cuda.mem_get_info()[0] >= free_before
    lin.close()


def test_noalloc_refuses_what_it_cannot_serve(tq, oracle):
    torch = pytest.importorskip("torch")
    L = tq.load()
    assert L.tq_linear_noalloc_scratch_limit() == 2 << 20
    lin = _layer(tq, oracle, 64, 256, 128, True, seed=1)
    x = torch.zeros((1, 256), device="cuda", dtype=torch.float16)
    y = torch.zeros((1, 64), device="cuda", dtype=torch.float16)
    host = np.zeros((1, 256), np.float16)
    assert L.tq_linear_forward_noalloc(lin.handle, host.ctypes.data, 1, C.c_void_p(y.data_ptr()), None) != 0
    assert b"device pointers" in L.tq_last_error()
    assert L.tq_linear_forward_noalloc(lin.handle, C.c_void_p(x.data_ptr()), 9, C.c_void_p(y.data_ptr()), None) != 0
    assert L.tq_linear_forward_noalloc(None, C.c_void_p(x.data_ptr()), 1, C.c_void_p(y.data_ptr()), None) != 0
    lin.close()
    # a layer whose working set exceeds the built-in array is refused, with the sizes in the message
    rows, cols = 64, 32768                        # dual rotation: the rotated activation alone fills the 2 MiB
    rng = np.random.default_rng(5)
    planes = [rng.integers(0, 256, (rows, cols // 2), dtype=np.uint8) for _ in range(2)]
    cb = tq.generate_codebook(4)
    qw = tq.QuantizedWeight(planes[0], planes[1], np.ones(rows, np.float32), np.array([11, 22, 128], np.uint32))
    big = tq.TurboQuantLinear(cols, rows, qw, cb, cb, 128)
    xb = torch.zeros((1, cols), device="cuda", dtype=torch.float16)
    yb = torch.zeros((1, rows), device="cuda", dtype=torch.float16)
    assert L.tq_linear_forward_noalloc(big.handle, C.c_void_p(xb.data_ptr()), 1, C.c_void_p(yb.data_ptr()), None) != 0
    assert b"scratch" in L.tq_last_error()
    big.close()
