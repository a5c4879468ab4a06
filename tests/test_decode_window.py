"""The fp16 decode window and hybrid_attention's window branch.

CPU part: the reference's unit tests for DecodeBuffer (tests/unit/test_decode_buffer.cpp:31-190)
restated against the numpy checker, which pins it.  GPU part: the same cases through the C-ABI, the
device ring against the checker value for value, and hybrid_attention on both branches
(tests/integration/test_attention_dispatch.cpp: short context, exactly a full window, long context,
empty cache)."""
import numpy as np
import pytest

from oracle.decode_window import DecodeWindow, window_attention

WINDOW, N_HEADS, HEAD_DIM = 8, 2, 32


def make_kv(tokens, base):
    # tests/unit/test_decode_buffer.cpp:13-24: element i of the flat array is base + i * 0.001
    n = tokens * N_HEADS * HEAD_DIM
    return (base + np.arange(n, dtype=np.float32) * np.float32(0.001)).reshape(tokens, N_HEADS, HEAD_DIM)


def single(token_idx, base):
    return make_kv(1, np.float32(base) + np.float32(token_idx) * np.float32(0.1))


def check_buffer_semantics(make, read_error):
    buf = make(WINDOW, N_HEADS, HEAD_DIM)
    assert buf.current_length() == 0 if callable(buf.current_length) else buf.current_length == 0
    length = (lambda b: b.current_length() if callable(b.current_length) else b.current_length)
    buf.rebuild(make_kv(5, 1.0), make_kv(5, 2.0))
    assert length(buf) == 5                                        # rebuild sets current_length
    b2 = make(WINDOW, N_HEADS, HEAD_DIM)
    for i in range(4):                                             # append increments by one
        before = length(b2)
        b2.append_token(single(i, 0.5), single(i, 1.5))
        assert length(b2) == before + 1
    b3 = make(WINDOW, N_HEADS, HEAD_DIM)
    b3.rebuild(make_kv(6, 1.0), make_kv(6, 2.0))
    assert b3.keys(1, 4).shape == (3, N_HEADS, HEAD_DIM) and b3.values(2, 6).shape == (4, N_HEADS, HEAD_DIM)
    for bad in ((-1, 2), (3, 3), (2, 7)):                          # out-of-range requests are refused
        with pytest.raises(read_error):
            b3.keys(*bad)
    # incremental append == rebuild
    n = 5
    all_k, all_v = make_kv(n, 3.0), make_kv(n, 4.0)
    ref = make(WINDOW, N_HEADS, HEAD_DIM)
    ref.rebuild(all_k, all_v)
    inc = make(WINDOW, N_HEADS, HEAD_DIM)
    for t in range(n):
        inc.append_token(all_k[t:t + 1], all_v[t:t + 1])
    assert np.array_equal(ref.keys(0, n).view(np.uint16), inc.keys(0, n).view(np.uint16))
    assert np.array_equal(ref.values(0, n).view(np.uint16), inc.values(0, n).view(np.uint16))
    assert np.array_equal(ref.keys(0, n), all_k.astype(np.float16))
    # wrap beyond the window
    w = make(WINDOW, N_HEADS, HEAD_DIM)
    for i in range(WINDOW):
        w.append_token(single(i, 0.0), single(i, 1.0))
    assert length(w) == WINDOW
    for i in range(3):
        w.append_token(single(WINDOW + i, 5.0), single(WINDOW + i, 6.0))
    assert length(w) == WINDOW + 3
    k_out = w.keys(3, WINDOW + 3)
    assert k_out.shape[0] == WINDOW
    want = np.concatenate([single(i, 0.0) for i in range(3, WINDOW)] + [single(WINDOW + i, 5.0) for i in range(3)])
    assert np.array_equal(k_out, want.astype(np.float16))
    return True


def test_checker_passes_the_reference_unit_tests():
    assert check_buffer_semantics(DecodeWindow, IndexError)


def test_checker_slide_window_and_long_rebuild():
    """slide_window overwrites from the slide position and wraps (src/decode_buffer.cpp:72-103); a rebuild
    longer than the window keeps the first `window` tokens but reports the full length (lines 26, 45)."""
    b = DecodeWindow(4, 1, 2)
    k = np.arange(12, dtype=np.float32).reshape(6, 1, 2)
    b.rebuild(k, k + 100)
    assert b.current_length == 6
    assert np.array_equal(b.keys(0, 4), k[:4].astype(np.float16))
    assert np.array_equal(b.keys(4, 6), k[:2].astype(np.float16))      # slots 0, 1 again: the ring is only 4 deep
    b.slide_window(k[4:6] * 10, k[4:6] * 10)
    assert b.window_start == 2
    assert np.array_equal(b.keys(0, 2), (k[4:6] * 10).astype(np.float16))
    b.slide_window(k[:3] + 50, k[:3] + 50)                              # slots 2, 3, 0
    assert b.window_start == 1
    assert np.array_equal(b.keys(2, 5), (k[:3] + 50).astype(np.float16))


def test_window_attention_is_softmax_over_scaled_scores():
    rng = np.random.default_rng(0)
    k = rng.standard_normal((7, 2, 32)).astype(np.float16)
    v = rng.standard_normal((7, 2, 32)).astype(np.float16)
    q = rng.standard_normal((4, 32)).astype(np.float16)
    out = window_attention(q, k, v)
    s = (k[:, 1].astype(np.float64) @ q[3].astype(np.float64)) / np.sqrt(32)
    p = np.exp(s) / np.exp(s).sum()
    assert np.allclose(out[3], p @ v[:, 1].astype(np.float64), atol=1e-6)


# ---- GPU -----------------------------------------------------------------------------------------

def rel_l2(a, b):
    a = np.asarray(a, np.float32)
    b = np.asarray(b, np.float32)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


@pytest.fixture(scope="module")
def tq():
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import turboquant_mlx_core_b200 as tq
    tq.load()
    return tq


@pytest.mark.gpu
def test_device_ring_passes_the_reference_unit_tests(tq):
    assert check_buffer_semantics(tq.DecodeBuffer, IndexError)


@pytest.mark.gpu
def test_device_ring_matches_checker_through_wraps_and_slides(tq):
    rng = np.random.default_rng(5)
    heads, dim, window = 3, 64, 16
    dev, ref = tq.DecodeBuffer(window, heads, dim), DecodeWindow(window, heads, dim)
    for step in range(40):
        op = int(rng.integers(3)) if step else 0
        n = int(rng.integers(1, 24 if op == 0 else 12))
        k = rng.standard_normal((n, heads, dim)).astype(np.float32 if step % 2 else np.float16)
        v = rng.standard_normal((n, heads, dim)).astype(k.dtype)
        if op == 0:
            dev.rebuild(k, v)
            ref.rebuild(k, v)
        elif op == 1:
            dev.append_token(k[:1], v[:1])
            ref.append_token(k[:1], v[:1])
        else:
            dev.slide_window(k, v)
            ref.slide_window(k, v)
        assert dev.current_length() == ref.current_length
        end = ref.current_length
        start = int(rng.integers(0, end))
        assert np.array_equal(dev.keys(start, end).view(np.uint16), ref.keys(start, end).view(np.uint16))
        assert np.array_equal(dev.values(start, end).view(np.uint16), ref.values(start, end).view(np.uint16))
    dev.close()


@pytest.mark.gpu
@pytest.mark.parametrize("heads,q_heads,dim,window,tokens", [(2, 2, 32, 64, 20), (2, 2, 32, 64, 64), (4, 28, 128, 4096, 1500),
                                                            (8, 32, 64, 512, 333), (1, 8, 256, 300, 300)])
def test_hybrid_attention_window_branch_matches_checker(tq, heads, q_heads, dim, window, tokens):
    """seq_len <= window: attention over the window's fp16 keys and values, exactly a full window included."""
    rng = np.random.default_rng(tokens)
    k = rng.standard_normal((tokens, heads, dim)).astype(np.float32)
    v = rng.standard_normal((tokens, heads, dim)).astype(np.float32)
    cache = tq.TQKVCache(1, heads, dim)
    cache.append(0, k, v)
    buf = tq.DecodeBuffer(window, heads, dim)
    buf.rebuild(k[: tokens - 1], v[: tokens - 1])
    buf.append_token(k[tokens - 1:], v[tokens - 1:])
    q = rng.standard_normal((q_heads, dim)).astype(np.float32)
    out = tq.hybrid_attention(cache, buf, 0, q)
    want = window_attention(q, k.astype(np.float16), v.astype(np.float16))
    assert np.all(np.isfinite(out.astype(np.float32)))
    assert rel_l2(out, want) < 1e-3, rel_l2(out, want)
    import torch
    qd = torch.from_numpy(q.astype(np.float16)).cuda()
    outd = tq.hybrid_attention(cache, buf, 0, qd)
    assert np.array_equal(outd.cpu().numpy().view(np.uint16), out.view(np.uint16))     # host and device pointers agree
    cache.close()
    buf.close()


@pytest.mark.gpu
def test_hybrid_attention_long_context_and_empty_cache(tq, ):
    """seq_len > window: the compressed cache is attended (centroid values, residual bits unused), equal to
    attention over what get_keys_fp16 / get_values_fp16 return; an empty cache gives zeros
    (src/attention_dispatch.cpp:29-32, 58-73)."""
    rng = np.random.default_rng(9)
    heads, q_heads, dim, window, tokens = 2, 4, 128, 32, 100
    cache = tq.TQKVCache(1, heads, dim)
    buf = tq.DecodeBuffer(window, heads, dim)
    q = rng.standard_normal((q_heads, dim)).astype(np.float32)
    assert not np.any(tq.hybrid_attention(cache, buf, 0, q).view(np.uint16))
    k = rng.standard_normal((tokens, heads, dim)).astype(np.float32)
    v = rng.standard_normal((tokens, heads, dim)).astype(np.float32)
    cache.append(0, k, v)
    out = tq.hybrid_attention(cache, buf, 0, q)
    want = window_attention(q, cache.get_keys_fp16(0, 0, tokens), cache.get_values_fp16(0, 0, tokens))
    assert rel_l2(out, want) < 2e-3, rel_l2(out, want)
    # a context that fits the window but was never put there is the reference's out-of-range error
    short = tq.TQKVCache(1, heads, dim)
    short.append(0, k[:10], v[:10])
    with pytest.raises(tq.TQError):
        tq.hybrid_attention(short, buf, 0, q)
    for c in (cache, short):
        c.close()
    buf.close()
