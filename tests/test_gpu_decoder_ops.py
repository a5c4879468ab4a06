"""GPU tests of the decoder-layer glue (RMSNorm, rotary embedding, SwiGLU, residual + slot sum) against
fp64 numpy restatements of their definitions, and of attention inside a captured CUDA graph."""
import ctypes as C

import numpy as np
import pytest

from tests.conftest import rel_l2

pytestmark = pytest.mark.gpu

TOL = 2e-3   # fp16 outputs: one rounding of the result (2^-11 relative) plus fp32 arithmetic


def test_rmsnorm_rope_swiglu_match_their_definitions(tq):
    torch = pytest.importorskip("torch")
    L = tq.load()
    rng = np.random.default_rng(0)
    rows, cols = 5, 5120
    x = rng.standard_normal((rows, cols)).astype(np.float16)
    w = (1 + 0.1 * rng.standard_normal(cols)).astype(np.float16)
    xd, wd = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    y = torch.empty_like(xd)
    assert L.tq_rmsnorm_f16(C.c_void_p(xd.data_ptr()), C.c_void_p(wd.data_ptr()), C.c_void_p(y.data_ptr()), rows, cols, 1e-6, None) == 0
    x64 = x.astype(np.float64)
    want = x64 / np.sqrt((x64 ** 2).mean(axis=1, keepdims=True) + 1e-6) * w.astype(np.float64)
    assert rel_l2(y.cpu().numpy(), want) < TOL

    heads, dim, theta = 5, 128, 1e6
    q = rng.standard_normal((rows, heads, dim)).astype(np.float16)
    pos = np.array([0, 1, 77, 8191, 40000], np.int32)
    qd, pd = torch.from_numpy(q).cuda(), torch.from_numpy(pos).cuda()
    assert L.tq_rope_f16(C.c_void_p(qd.data_ptr()), C.c_void_p(pd.data_ptr()), rows, heads, dim, theta, None) == 0
    half = dim // 2
    inv = theta ** (-2.0 * np.arange(half) / dim)
    ang = pos[:, None].astype(np.float64) * inv[None, :]
    a, b = q[..., :half].astype(np.float64), q[..., half:].astype(np.float64)
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    want = np.concatenate([a * c - b * s, b * c + a * s], axis=-1)
    assert rel_l2(qd.cpu().numpy(), want) < TOL

    inter = 3456
    gu = rng.standard_normal((rows, 2 * inter)).astype(np.float16)
    gud = torch.from_numpy(gu).cuda()
    act = torch.empty((rows, inter), dtype=torch.float16, device="cuda")
    assert L.tq_swiglu_f16(C.c_void_p(gud.data_ptr()), C.c_void_p(act.data_ptr()), rows, inter, None) == 0
    g64, u64 = gu[:, :inter].astype(np.float64), gu[:, inter:].astype(np.float64)
    want = g64 / (1 + np.exp(-g64)) * u64
    assert rel_l2(act.cpu().numpy(), want) < TOL

    # slot sum with a residual: fixed order, fp32
    slots = torch.from_numpy(rng.standard_normal((3, rows * cols)).astype(np.float16)).cuda()
    res = torch.from_numpy(rng.standard_normal(rows * cols).astype(np.float16)).cuda()
    out = torch.empty(rows * cols, dtype=torch.float16, device="cuda")
    assert L.tq_exchange_sum_f16(C.c_void_p(slots.data_ptr()), 3, rows * cols, rows * cols, C.c_void_p(res.data_ptr()),
                                 C.c_void_p(out.data_ptr()), None) == 0
    torch.cuda.synchronize()
    want = (((res.float() + slots[0].float()) + slots[1].float()) + slots[2].float()).half()
    assert torch.equal(out, want)
    assert L.tq_rmsnorm_f16(C.c_void_p(xd.data_ptr()), C.c_void_p(wd.data_ptr()), C.c_void_p(y.data_ptr()), rows, 5121, 1e-6, None) != 0

    # the same sum with the RMSNorm of the summed rows in one kernel: both results bit-equal to the two separate calls
    out2 = torch.empty_like(out)
    normed, normed2 = torch.empty_like(out), torch.empty_like(out)
    assert L.tq_exchange_sum_f16_rmsnorm(C.c_void_p(slots.data_ptr()), 3, rows * cols, rows, cols, C.c_void_p(res.data_ptr()),
                                         C.c_void_p(out2.data_ptr()), C.c_void_p(wd.data_ptr()), C.c_void_p(normed2.data_ptr()),
                                         1e-6, None) == 0
    assert L.tq_rmsnorm_f16(C.c_void_p(out.data_ptr()), C.c_void_p(wd.data_ptr()), C.c_void_p(normed.data_ptr()), rows, cols, 1e-6, None) == 0
    torch.cuda.synchronize()
    assert torch.equal(out2, out) and torch.equal(normed2, normed)

    # queries and keys through the rotary embedding in one launch: the bits of the two separate calls
    kv_heads = 2
    k = rng.standard_normal((rows, kv_heads, dim)).astype(np.float16)
    q1, k1 = torch.from_numpy(q).cuda(), torch.from_numpy(k).cuda()
    q2, k2 = q1.clone(), k1.clone()
    assert L.tq_rope_f16(C.c_void_p(q1.data_ptr()), C.c_void_p(pd.data_ptr()), rows, heads, dim, theta, None) == 0
    assert L.tq_rope_f16(C.c_void_p(k1.data_ptr()), C.c_void_p(pd.data_ptr()), rows, kv_heads, dim, theta, None) == 0
    assert L.tq_rope_qk_f16(C.c_void_p(q2.data_ptr()), C.c_void_p(k2.data_ptr()), C.c_void_p(pd.data_ptr()), rows, heads, kv_heads, dim,
                            theta, None) == 0
    torch.cuda.synchronize()
    assert torch.equal(q1, q2) and torch.equal(k1, k2) and torch.equal(q1, qd)


def test_attention_replays_inside_a_cuda_graph(tq):
    """A decode-attention call whose descriptors repeat the previous call's enqueues kernels only: captured
    in a graph and replayed, it gives the bits of the eager call."""
    torch = pytest.importorskip("torch")
    from tests.golden.make_golden import kv_inputs
    heads, dim, q_heads, n = 2, 128, 14, 700
    k, v = kv_inputs(31, n, heads, dim)
    c = tq.TQKVCache(1, heads, dim)
    c.append(0, k, v)
    q = torch.randn((1, q_heads, dim), device="cuda").half()
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        eager = tq.compressed_attention([c], 0, q, use_qjl=True, stream=st).clone()
        out = torch.empty_like(eager)
        tq.compressed_attention([c], 0, q, use_qjl=True, out=out, stream=st)      # the call to be captured, once eagerly
        st.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=st):
            tq.compressed_attention([c], 0, q, use_qjl=True, out=out, stream=st)
        out.zero_()
        g.replay()
        st.synchronize()
    c.check_attention_status()
    assert torch.equal(out, eager)
    c.close()
