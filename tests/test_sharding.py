"""CPU tests of the multi-GPU host logic: the row partition of column-parallel linears and
the KV-head partition, plus a world_size-2 gloo run of the all-gather that follows them."""
import os
import socket

import numpy as np
import pytest

from turboquant_mlx_core_b200.sharding import head_range, row_range, shard_quantized_rows


def test_row_range_covers_everything_once():
    for out in (151936, 4096, 18944, 512, 7, 1):
        for world in (1, 2, 4, 8):
            spans = [row_range(out, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == out
            for a, b in zip(spans, spans[1:]):
                assert a[1] == b[0]
            sizes = [e - s for s, e in spans]
            assert max(sizes) - min(sizes) <= 16      # whole 16-row tiles except the tail
    assert row_range(151936, 3, 8) == (3 * 18992, 4 * 18992)


def test_head_range():
    assert [head_range(4, r, 2) for r in range(2)] == [(0, 2), (2, 4)]
    assert [head_range(8, r, 8) for r in range(8)] == [(r, r + 1) for r in range(8)]
    with pytest.raises(ValueError):
        head_range(4, 0, 8)          # more ranks than KV heads: callers split context instead


def test_shard_quantized_rows_slices_planes():
    pp = np.arange(64 * 8, dtype=np.uint8).reshape(64, 8)
    pr = pp[::-1].copy()
    norms = np.arange(64, dtype=np.float32)
    a, b, c = shard_quantized_rows(pp, pr, norms, 1, 2)
    s, e = row_range(64, 1, 2)
    assert np.array_equal(a, pp[s:e]) and np.array_equal(b, pr[s:e]) and np.array_equal(c, norms[s:e])


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_features, q):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from turboquant_mlx_core_b200.sharding import all_gather_rows, row_range
    s, e = row_range(out_features, rank, world)
    full = torch.arange(3 * out_features, dtype=torch.float32).reshape(3, out_features).to(torch.float16)
    local = full[:, s:e].contiguous()
    got = all_gather_rows(local, out_features, world)
    q.put((rank, bool(torch.equal(got, full))))
    dist.destroy_process_group()


def test_all_gather_of_row_shards_gloo():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, 1000, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(60)
    assert res == [(0, True), (1, True)]


def test_attention_grid_and_context_range():
    from turboquant_mlx_core_b200.sharding import attention_grid, context_range
    assert [attention_grid(4, r, 2) for r in range(2)] == [(0, 2, 0, 1), (2, 4, 0, 1)]
    assert [attention_grid(4, r, 8) for r in range(8)] == [(r % 4, r % 4 + 1, r // 4, 2) for r in range(8)]
    with pytest.raises(ValueError):
        attention_grid(4, 0, 6)
    spans = [context_range(5, 1005, p, 3) for p in range(3)]
    assert spans[0][0] == 5 and spans[-1][1] == 1005 and all(a[1] == b[0] for a, b in zip(spans, spans[1:]))


def _softmax_parts(rng, parts, rows, toks, dim):
    """Per-part attention outputs and log-sum-exps of one random problem, plus the full answer."""
    s = rng.standard_normal((rows, toks)).astype(np.float64) * 3
    v = rng.standard_normal((toks, dim)).astype(np.float64)
    w = np.exp(s - s.max(axis=1, keepdims=True))
    full = (w / w.sum(axis=1, keepdims=True)) @ v
    outs, lses = [], []
    for p in range(parts):
        a, b = toks * p // parts, toks * (p + 1) // parts
        sp = s[:, a:b]
        m = sp.max(axis=1, keepdims=True)
        e = np.exp(sp - m)
        outs.append((e / e.sum(axis=1, keepdims=True)) @ v[a:b])
        lses.append((m[:, 0] + np.log(e.sum(axis=1))))
    return np.stack(outs).astype(np.float32), np.stack(lses).astype(np.float32), full


def test_merge_attention_parts_is_exact():
    from turboquant_mlx_core_b200.sharding import merge_attention_parts
    rng = np.random.default_rng(4)
    outs, lses, full = _softmax_parts(rng, 3, 7, 50, 16)
    got = merge_attention_parts(outs, lses)
    assert np.allclose(got, full, rtol=1e-5, atol=1e-6)
    import torch
    got_t = merge_attention_parts(torch.tensor(outs), torch.tensor(lses)).numpy()
    assert np.allclose(got_t, full, rtol=1e-5, atol=1e-6)
    # a part with no tokens (lse = -inf) contributes nothing
    outs2 = np.concatenate([outs, np.zeros_like(outs[:1])])
    lses2 = np.concatenate([lses, np.full_like(lses[:1], -np.inf)])
    assert np.allclose(merge_attention_parts(outs2, lses2), full, rtol=1e-5, atol=1e-6)


def _worker_attn(rank, world, port, q):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from turboquant_mlx_core_b200.sharding import all_gather_attention_parts
    outs, lses, full = _softmax_parts(np.random.default_rng(9), world, 6, 40, 8)
    got = all_gather_attention_parts(torch.tensor(outs[rank]), torch.tensor(lses[rank]))
    q.put((rank, bool(np.allclose(got.numpy(), full, rtol=1e-5, atol=1e-6))))
    dist.destroy_process_group()


def test_context_split_merge_gloo():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_attn, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(60)
    assert res == [(0, True), (1, True)]


def test_row_parallel_column_shards_sum_to_the_full_layer(oracle):
    """Row-parallel split (input features in whole WHT blocks): the dequantised column shards,
    built with the rescaled norms, multiply the matching slices of x to partial outputs whose sum
    is the full layer's output."""
    from turboquant_mlx_core_b200.sharding import col_range, shard_quantized_cols
    rng = np.random.default_rng(2)
    rows, cols, bs, world = 24, 768, 128, 3
    cb = oracle.codebook(4)[0]
    w = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float16).astype(np.float32)
    pp, pr, norms, seeds = oracle.quantize_weight(w, cb, cb, 4, 4, bs, True)
    full = oracle.dequantize_weight(pp, pr, norms, seeds, cb, cb, bs)
    x = rng.standard_normal((2, cols)).astype(np.float16).astype(np.float32)
    want = x @ full.T
    got = np.zeros_like(want)
    spans = []
    for r in range(world):
        spp, spr, snorms, (c0, c1) = shard_quantized_cols(pp, pr, norms, cols, bs, r, world)
        spans.append((c0, c1))
        part = oracle.dequantize_weight(np.ascontiguousarray(spp), np.ascontiguousarray(spr), snorms, seeds, cb, cb, bs)
        assert part.shape == (rows, c1 - c0)
        # same weights up to fp32 rounding of the rescaled norm and inverse scale (a few 1e-8 on values of 0.08)
        assert np.max(np.abs(part - full[:, c0:c1])) < 1e-6 * np.max(np.abs(full))
        got += x[:, c0:c1] @ part.T
    assert spans[0][0] == 0 and spans[-1][1] == cols and all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    assert np.allclose(got, want, rtol=1e-4, atol=1e-6)
    assert col_range(27648, 128, 7, 8) == (7 * 3456, 8 * 3456)
