"""GPU parity tests for the compressed KV cache: encoder bits, range decode, attention."""
import ctypes as C

import numpy as np
import pytest

from tests.conftest import rel_l2
from tests.golden.make_golden import kv_inputs

pytestmark = pytest.mark.gpu

ATTN_TOL = 1e-3   # relative L2 against the oracle, as the task states

KV_CASES = [("kv4x128", 2, 4, 128, 24, 5), ("kv2x32", 1, 2, 32, 40, 6), ("kv1x64", 1, 1, 64, 9, 8)]


def bits_equal(a, b):
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    return a.shape == b.shape and np.array_equal(a.view(np.uint8), b.view(np.uint8))


@pytest.mark.parametrize("case", KV_CASES, ids=[c[0] for c in KV_CASES])
@pytest.mark.parametrize("dtype", [np.float16, np.float32])
def test_append_bits_and_decode(tq, golden, case, dtype):
    name, layers, heads, dim, tokens, seed = case
    lay = layers - 1
    k, v = kv_inputs(seed, tokens, heads, dim)
    cache = tq.TQKVCache(layers, heads, dim)
    assert cache.seq_length() == 0
    cache.append(lay, k[: tokens // 2].astype(dtype), v[: tokens // 2].astype(dtype))
    for t in range(tokens // 2, tokens):                      # then one token per step, as in decode
        cache.append(lay, k[t:t + 1].astype(dtype), v[t:t + 1].astype(dtype))
    assert cache.seq_length() == tokens
    ex = cache.export(lay)
    assert ex["tokens"] == tokens
    for key in ("k_words", "v_words", "k_norms", "v_norms", "qjl_words", "qjl_norms"):
        assert bits_equal(ex[key], golden[f"{name}_{key}"]), key
    assert bits_equal(cache.get_keys_fp16(lay, 0, tokens).view(np.uint16), golden[f"{name}_keys_fp16"])
    assert bits_equal(cache.get_values_fp16(lay, 0, tokens).view(np.uint16), golden[f"{name}_values_fp16"])
    part = cache.get_keys_fp16(lay, 3, 7)
    assert bits_equal(part.view(np.uint16), golden[f"{name}_keys_fp16"][3:7])
    with pytest.raises(IndexError):
        cache.get_keys_fp16(lay, 0, tokens + 1)               # tests/unit/test_kv_cache.cpp:203-211
    with pytest.raises(IndexError):
        cache.get_keys_fp16(lay, 5, 5)
    with pytest.raises(IndexError):
        cache.append(layers, k, v)
    cache.close()


@pytest.mark.parametrize("heads,dim,tokens", [(4, 128, 300), (2, 64, 700), (1, 256, 530), (3, 32, 200), (1, 512, 515)])
@pytest.mark.parametrize("dtype", [np.float16, np.float32])
def test_bulk_append_bits_match_the_checker(tq, oracle, heads, dim, tokens, dtype):
    """Appends of 512 vectors or more run the batched encoder (one thread per vector for the two
    left-to-right sums of src/kv_cache.cpp:84-88, 226-231): every stored bit equals the CPU
    restatement's, also when a later single-token append lands behind the bulk."""
    k, v = kv_inputs(tokens + dim, tokens, heads, dim)
    c = tq.TQKVCache(1, heads, dim)
    c.append(0, k[:-1].astype(dtype), v[:-1].astype(dtype))
    c.append(0, k[-1:].astype(dtype), v[-1:].astype(dtype))
    ex = c.export(0)
    kw, kn, qw, qn = oracle.kv_encode(k.astype(np.float32), oracle.kv_seed(0, 1), oracle.kv_seed(0, 3))
    vw, vn, _, _ = oracle.kv_encode(v.astype(np.float32), oracle.kv_seed(0, 2))
    for key, want in (("k_words", kw), ("k_norms", kn), ("qjl_words", qw), ("qjl_norms", qn), ("v_words", vw), ("v_norms", vn)):
        assert bits_equal(np.asarray(ex[key]).reshape(np.asarray(want).shape), want), key
    c.close()


@pytest.mark.parametrize("case", KV_CASES, ids=[c[0] for c in KV_CASES])
@pytest.mark.parametrize("use_qjl", [False, True])
def test_attention_matches_oracle(tq, golden, case, use_qjl):
    name, layers, heads, dim, tokens, seed = case
    lay = layers - 1
    k, v = kv_inputs(seed, tokens, heads, dim)
    cache = tq.TQKVCache(layers, heads, dim)
    cache.append(lay, k, v)
    q_heads = heads * (7 if heads == 4 else 1)
    q = np.random.default_rng(seed + 100).standard_normal((q_heads, dim)).astype(np.float16).astype(np.float32)
    out = tq.compressed_attention([cache], lay, q[None], use_qjl=use_qjl)
    want = golden[f"{name}_attn_qjl{int(use_qjl)}"]
    assert out.shape == (1, q_heads, dim) and out.dtype == np.float16
    assert rel_l2(out[0], want) < ATTN_TOL, rel_l2(out[0], want)
    cache.close()


def test_attention_long_context_batch_and_ranges(tq, oracle):
    """Several sequences of different lengths, many context splits, sub-ranges, GQA 7."""
    rng = np.random.default_rng(9)
    heads, dim, q_heads = 4, 128, 28
    lens = [700, 1301]
    caches, stores = [], []
    for n in lens:
        k, v = kv_inputs(int(rng.integers(1 << 30)), n, heads, dim)
        c = tq.TQKVCache(1, heads, dim)
        c.append(0, k, v)
        caches.append(c)
        stores.append(c.export(0))
    q = rng.standard_normal((len(lens), q_heads, dim)).astype(np.float16)
    for use_qjl in (False, True):
        out = tq.compressed_attention(caches, 0, q, use_qjl=use_qjl)
        for i, ex in enumerate(stores):
            want = oracle.attention(q[i].astype(np.float32), heads, ex["k_words"], ex["k_norms"], ex["v_words"],
                                    ex["v_norms"], ex["qjl_words"], ex["qjl_norms"], layer=0, use_qjl=use_qjl)
            assert rel_l2(out[i], want) < ATTN_TOL, (i, use_qjl, rel_l2(out[i], want))
    out = tq.compressed_attention(caches[:1], 0, q[:1], start=100, end=333)
    ex = stores[0]
    want = oracle.attention(q[0].astype(np.float32), heads, ex["k_words"], ex["k_norms"], ex["v_words"], ex["v_norms"],
                            ex["qjl_words"], ex["qjl_norms"], layer=0, start=100, end=333)
    assert rel_l2(out[0], want) < ATTN_TOL
    with pytest.raises(tq.TQError):
        tq.compressed_attention(caches[:1], 0, q[:1], start=0, end=10_000)
    for c in caches:
        c.close()


def test_reference_c_api_with_arrays(tq, golden):
    """The reference's own entry points (tq_kv_cache_append / get_keys_fp16 / attention) driven
    through tq_array handles, plus multi-layer independence (tests/unit/test_kv_cache.cpp)."""
    L = tq.load()
    name, layers, heads, dim, tokens, seed = KV_CASES[0]
    k, v = kv_inputs(seed, tokens, heads, dim)
    shape = (C.c_int * 3)(tokens, heads, dim)
    ka = L.tq_array_create(k.ctypes.data, 1, 3, shape)
    va = L.tq_array_create(v.ctypes.data, 1, 3, shape)
    assert ka and va
    cache = L.tq_kv_cache_create(layers, heads, dim, 3, 4096, 128)
    L.tq_kv_cache_append(cache, layers - 1, ka, va)
    L.tq_kv_cache_append(cache, layers + 5, ka, va)           # silently ignored, as in the reference
    assert L.tq_kv_cache_seq_length(cache) == tokens
    arr = L.tq_kv_cache_get_keys_fp16(cache, layers - 1, 0, tokens)
    assert arr and L.tq_array_ndim(arr) == 3 and L.tq_array_dim(arr, 2) == dim
    host = np.zeros((tokens, heads, dim), np.uint16)
    assert L.tq_array_to_host(arr, host.ctypes.data, host.nbytes) == 0
    assert np.array_equal(host, golden[f"{name}_keys_fp16"])
    L.tq_array_free(arr)
    assert L.tq_kv_cache_get_keys_fp16(cache, 0, 0, 1) is None  # layer 0 is empty
    assert L.tq_kv_cache_get_values_fp16(cache, layers - 1, 4, 2) is None
    q = np.random.default_rng(seed + 100).standard_normal((heads * 7, dim)).astype(np.float16)
    qa = L.tq_array_create(q.ctypes.data, 1, 2, (C.c_int * 2)(heads * 7, dim))
    oa = L.tq_kv_cache_attention(cache, layers - 1, qa, 0, tokens)
    assert oa
    out = np.zeros((heads * 7, dim), np.float16)
    assert L.tq_array_to_host(oa, out.ctypes.data, out.nbytes) == 0
    assert rel_l2(out, golden[f"{name}_attn_qjl0"]) < ATTN_TOL
    for a in (oa, qa, ka, va):
        L.tq_array_free(a)
    L.tq_kv_cache_free(cache)


def test_attention_lse_merges_context_parts(tq):
    """Attention over [0, n) equals the merge of attention over three disjoint token ranges using
    the log-sum-exp output: the rule by which a sequence's context is split across GPUs."""
    from turboquant_mlx_core_b200.sharding import context_range, merge_attention_parts
    rng = np.random.default_rng(21)
    heads, dim, tokens, q_heads = 4, 128, 700, 28
    caches = []
    for s_ in range(2):
        c = tq.TQKVCache(1, heads, dim)
        c.append(0, rng.standard_normal((tokens, heads, dim)).astype(np.float16),
                 rng.standard_normal((tokens, heads, dim)).astype(np.float16))
        caches.append(c)
    q = rng.standard_normal((2, q_heads, dim)).astype(np.float16)
    for use_qjl in (False, True):
        full, lse_full = tq.compressed_attention(caches, 0, q, use_qjl=use_qjl, return_lse=True)
        assert lse_full.shape == (2, q_heads) and np.all(np.isfinite(lse_full))
        outs, lses = [], []
        for part in range(3):
            a, b = context_range(0, tokens, part, 3)
            o, l = tq.compressed_attention(caches, 0, q, start=a, end=b, use_qjl=use_qjl, return_lse=True)
            outs.append(o.astype(np.float32))
            lses.append(l)
        merged = merge_attention_parts(np.stack(outs), np.stack(lses))
        assert rel_l2(merged, full.astype(np.float32)) < ATTN_TOL
        # the parts' denominators add up to the whole
        m = np.max(np.stack(lses), axis=0)
        assert np.allclose(m + np.log(np.sum(np.exp(np.stack(lses) - m), axis=0)), lse_full, rtol=0, atol=2e-3)
    for c in caches:
        c.close()


def test_append_batch_equals_single_appends(tq):
    """A decode step appended to many caches at once stores exactly what one-token appends store,
    also across the 32-sequence launch boundary and after a reserve()."""
    import torch
    rng = np.random.default_rng(31)
    heads, dim, n = 2, 128, 37
    a = [tq.TQKVCache(1, heads, dim) for _ in range(n)]
    b = [tq.TQKVCache(1, heads, dim) for _ in range(n)]
    for c in a[:5]:
        c.reserve(0, 1000)
    prefix = rng.standard_normal((3, heads, dim)).astype(np.float16)
    for c in a + b:
        c.append(0, prefix, prefix)
    for step in range(3):
        k = rng.standard_normal((n, heads, dim)).astype(np.float16)
        v = rng.standard_normal((n, heads, dim)).astype(np.float16)
        tq.append_batch(a, 0, torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda())
        for i, c in enumerate(b):
            c.append(0, k[i:i + 1], v[i:i + 1])
    torch.cuda.synchronize()
    for ca, cb in zip(a, b):
        ea, eb = ca.export(0), cb.export(0)
        assert ea["tokens"] == eb["tokens"] == 6
        for key in ("k_words", "v_words", "k_norms", "v_norms", "qjl_words", "qjl_norms"):
            assert bits_equal(ea[key], eb[key]), key
    for c in a + b:
        c.close()


def test_snapshot_is_byte_identical_and_restores(tq, golden):
    """tq_kv_snapshot writes the reference's serialized snapshot byte for byte; restoring it (or
    the reference's own stream) into a fresh cache reproduces storage and attention."""
    name, layers, heads, dim, tokens, seed = KV_CASES[0]
    k, v = kv_inputs(seed, tokens, heads, dim)
    cache = tq.TQKVCache(layers, heads, dim)
    cache.append(layers - 1, k[: tokens // 2], v[: tokens // 2])
    cache.append(layers - 1, k[tokens // 2:], v[tokens // 2:])
    snap = cache.snapshot(model_hash=0x1234ABCD, codebook_hash=0x0BADF00D)
    assert bits_equal(snap, golden[f"{name}_snapshot"])
    other = tq.TQKVCache(layers, heads, dim)
    other.append(0, k[:3], v[:3])                     # replaced by the restore
    other.restore(golden[f"{name}_snapshot"])
    assert other.seq_length() == tokens
    ea, eb = cache.export(layers - 1), other.export(layers - 1)
    for key in ("k_words", "v_words", "k_norms", "v_norms", "qjl_words", "qjl_norms"):
        assert bits_equal(ea[key], eb[key]), key
    assert other.export(0)["tokens"] == 0
    q = np.random.default_rng(1).standard_normal((1, heads * 7, dim)).astype(np.float16)
    a = tq.compressed_attention([cache], layers - 1, q, use_qjl=True)
    b = tq.compressed_attention([other], layers - 1, q, use_qjl=True)
    assert bits_equal(a, b)
    other.append(layers - 1, k[:1], v[:1])            # still appendable
    assert other.seq_length() == tokens + 1
    # malformed streams are refused and leave the cache as it was
    for bad in (snap[:40], np.concatenate([snap[:8], snap[8:] ^ 0]).astype(np.uint8)[:-5], np.zeros(64, np.uint8)):
        with pytest.raises(ValueError):
            other.restore(bad)
    wrong = tq.TQKVCache(layers, heads * 2, dim)
    with pytest.raises(ValueError):
        wrong.restore(snap)
    assert other.seq_length() == tokens + 1
    for c in (cache, other, wrong):
        c.close()


@pytest.mark.parametrize("heads,q_heads", [(1, 4), (2, 14), (4, 28), (8, 32), (3, 6), (12, 12)])
def test_attention_head_counts_and_ragged_ranges(tq, oracle, heads, q_heads):
    """head_dim 128 over every way the cache is fetched: all heads of a 16-token tile as one slab
    (1, 2, 4 KV heads), a group of four heads as per-token rows (8, 12), and the load-based kernel
    (3); token ranges that start and end inside a tile, and shorter than one tile."""
    rng = np.random.default_rng(heads * 100 + q_heads)
    dim, n = 128, 333
    k, v = kv_inputs(int(rng.integers(1 << 30)), n, heads, dim)
    c = tq.TQKVCache(1, heads, dim)
    c.append(0, k, v)
    ex = c.export(0)
    q = rng.standard_normal((1, q_heads, dim)).astype(np.float16)
    for start, end, use_qjl in [(0, n, True), (0, n, False), (5, 330, True), (17, 30, True), (32, 48, False), (331, 333, True)]:
        # the automatic choice would run a job this small on the load-based kernel: ask for the pipeline
        c.set_attention_kernel(c.ATTENTION_PIPELINE)
        out = tq.compressed_attention([c], 0, q, start=start, end=end, use_qjl=use_qjl)
        c.set_attention_kernel(c.ATTENTION_LOADS)
        other = tq.compressed_attention([c], 0, q, start=start, end=end, use_qjl=use_qjl)
        assert rel_l2(out[0], other[0].astype(np.float32)) < ATTN_TOL
        want = oracle.attention(q[0].astype(np.float32), heads, ex["k_words"], ex["k_norms"], ex["v_words"], ex["v_norms"],
                                ex["qjl_words"], ex["qjl_norms"], layer=0, start=start, end=end, use_qjl=use_qjl)
        assert np.all(np.isfinite(out.astype(np.float32)))
        assert rel_l2(out[0], want) < ATTN_TOL, (start, end, use_qjl, rel_l2(out[0], want))
        if heads == 4:
            # the tensor-memory kernel (tcgen05): tiles of 32 tokens, partial first and last tiles
            c.set_attention_kernel(c.ATTENTION_TENSOR_MEMORY)
            tm = tq.compressed_attention([c], 0, q, start=start, end=end, use_qjl=use_qjl)
            c.check_attention_status()
            assert np.all(np.isfinite(tm.astype(np.float32)))
            assert rel_l2(tm[0], want) < ATTN_TOL, ("tensor memory", start, end, use_qjl, rel_l2(tm[0], want))
    c.close()


@pytest.mark.parametrize("tokens", [4096, 32768])
def test_attention_at_benchmark_contexts_matches_oracle(tq, oracle, tokens):
    """One sequence, 4 KV / 28 query heads, at the context lengths the throughput figures are quoted
    on: the three CUDA kernels (bulk-copy pipeline, load-based, tensor memory), residual bits off and on, each against
    the CPU checker (mirrors src/attention_dispatch.cpp:58-73 over the fp16 keys and values that
    src/kv_cache.cpp:292-365 would hand it).  At these lengths the context is cut into dozens of
    splits, the softmax reference moves lazily and the parts are merged in fixed order."""
    heads, dim, q_heads = 4, 128, 28
    k, v = kv_inputs(1000 + tokens, tokens, heads, dim)
    c = tq.TQKVCache(1, heads, dim)
    c.append(0, k, v)
    ex = c.export(0)
    q = np.random.default_rng(tokens).standard_normal((1, q_heads, dim)).astype(np.float16)
    for use_qjl in (False, True):
        want = oracle.attention(q[0].astype(np.float32), heads, ex["k_words"], ex["k_norms"], ex["v_words"], ex["v_norms"],
                                ex["qjl_words"], ex["qjl_norms"], layer=0, use_qjl=use_qjl)
        for kernel in (c.ATTENTION_PIPELINE, c.ATTENTION_LOADS, c.ATTENTION_TENSOR_MEMORY):
            c.set_attention_kernel(kernel)
            out = tq.compressed_attention([c], 0, q, use_qjl=use_qjl)
            c.check_attention_status()
            assert np.all(np.isfinite(out.astype(np.float32)))
            assert rel_l2(out[0], want) < ATTN_TOL, (tokens, use_qjl, kernel, rel_l2(out[0], want))
    c.close()


def test_attention_kernel_choice_is_automatic_for_long_batches(tq):
    """40 sequences x 8192 tokens fill every CTA slot with 512 tokens or more: the automatic choice is the
    pipeline kernel; it agrees with the load-based kernel, leaves the status clean, and the knob refuses
    unknown values."""
    heads, dim, q_heads, n, n_seqs = 4, 128, 28, 8192, 40
    rng = np.random.default_rng(21)
    k, v = kv_inputs(77, n, heads, dim)
    c = tq.TQKVCache(1, heads, dim)
    c.append(0, k, v)
    caches = [c] * n_seqs                      # the same storage read by every sequence of the batch
    q = rng.standard_normal((n_seqs, q_heads, dim)).astype(np.float16)
    auto = tq.compressed_attention(caches, 0, q)
    c.set_attention_kernel(c.ATTENTION_LOADS)
    loads = tq.compressed_attention(caches, 0, q)
    c.set_attention_kernel(c.ATTENTION_PIPELINE)
    pipe = tq.compressed_attention(caches, 0, q)
    c.check_attention_status()
    assert rel_l2(auto, loads.astype(np.float32)) < ATTN_TOL
    assert np.array_equal(auto.view(np.uint16), pipe.view(np.uint16))    # automatic == pipeline here
    with pytest.raises(tq.TQError):
        c.set_attention_kernel(7)
    c.close()


@pytest.mark.parametrize("case", KV_CASES, ids=[c[0] for c in KV_CASES])
def test_delta_is_byte_identical_and_applies(tq, golden, case):
    """tq_kv_delta writes the reference's serialized delta byte for byte; a cache holding the first
    tokens plus the delta of the rest equals the cache that appended everything."""
    name, layers, heads, dim, tokens, seed = case
    k, v = kv_inputs(seed, tokens, heads, dim)
    full = tq.TQKVCache(layers, heads, dim)
    full.append(layers - 1, k[: tokens // 2], v[: tokens // 2])
    full.append(layers - 1, k[tokens // 2:], v[tokens // 2:])
    assert bits_equal(full.delta(3, tokens - 2), golden[f"{name}_delta"])
    # ranges are clamped to each layer's length (the header keeps the positions as asked, as the
    # reference's does), an empty range is a valid stream
    assert bits_equal(full.delta(3, tokens + 50)[16:], full.delta(3, tokens)[16:])
    assert full.delta(tokens, tokens).size == 16 + layers * (4 + 4 + 6 * 4)
    # positions of 2^31 and above are narrowed to int as in the reference (src/kv_cache.cpp:571-572):
    # such an end position is negative, so every layer's range is empty
    assert full.delta(0, 0xFFFFFFFF).size == 16 + layers * (4 + 4 + 6 * 4)
    part = tq.TQKVCache(layers, heads, dim)
    part.append(layers - 1, k[:3], v[:3])
    part.apply_delta(golden[f"{name}_delta"])          # the reference's own stream
    part.apply_delta(full.delta(tokens - 2, tokens))
    assert part.seq_length() == tokens
    ea, eb = full.export(layers - 1), part.export(layers - 1)
    for key in ("k_words", "v_words", "k_norms", "v_norms", "qjl_words", "qjl_norms"):
        assert bits_equal(ea[key], eb[key]), key
    d = full.delta(0, tokens)
    for bad in (d[:20], d[:-3], np.zeros(40, np.uint8), full.snapshot()):
        with pytest.raises(ValueError):
            part.apply_delta(bad)
    assert part.seq_length() == tokens
    if layers > 1:
        other = tq.TQKVCache(layers + 1, heads, dim)
        with pytest.raises(ValueError):
            other.apply_delta(d)
        other.close()
    full.close()
    part.close()


def test_kv_edge_cases(tq):
    """Empty appends, empty layers and empty or reversed ranges: nothing changes, nothing faults,
    and the calls that cannot be served say so."""
    heads, dim = 2, 128
    c = tq.TQKVCache(2, heads, dim)
    assert c.seq_length() == 0 and c.export(0)["tokens"] == 0
    empty = np.zeros((0, heads, dim), np.float16)
    c.append(0, empty, empty)                              # zero tokens: a no-op
    assert c.seq_length() == 0
    q = np.ones((1, heads, dim), np.float16)
    with pytest.raises(tq.TQError):
        tq.compressed_attention([c], 0, q)                 # nothing to attend to
    assert c.snapshot().size == 32 + 2 * (4 + 4 + 6 * 4)   # a snapshot of an empty cache is just headers
    k, v = kv_inputs(3, 17, heads, dim)
    c.append(1, k, v)
    assert c.seq_length() == 17 and c.export(0)["tokens"] == 0
    for start, end in [(5, 5), (9, 4), (-1, 3), (0, 18)]:
        with pytest.raises((tq.TQError, ValueError, IndexError)):
            tq.compressed_attention([c], 1, q, start=start, end=end)
    with pytest.raises((tq.TQError, ValueError, IndexError)):
        tq.compressed_attention([c], 0, q)                 # layer 0 is still empty
    with pytest.raises((tq.TQError, ValueError, IndexError)):
        c.append(2, k, v)                                  # no such layer
    with pytest.raises(ValueError):
        c.append(1, k[:, :1], v[:, :1])                    # wrong head count
    c.reserve(1, 4)                                        # smaller than what is stored: a no-op
    c.append(1, empty, empty)
    assert c.seq_length() == 17
    one = tq.compressed_attention([c], 1, q, start=16, end=17)   # a single token: the output is that value vector
    vals = np.asarray(c.get_values_fp16(1, 16, 17)).astype(np.float32).reshape(heads, dim)
    assert np.all(np.isfinite(one.astype(np.float32)))
    assert rel_l2(one[0], vals) < 2e-3
    c.close()
