"""GPU tests of the rank-to-rank exchange kernels on ONE device: two "ranks" are two exchange handles
and two buffers in this process, and every broadcast is enqueued before the wait that consumes it (a
kernel never waits here for one that has not been launched).  The multi-process use over CUDA IPC is
exercised by bench.py's sharded legs on 2 or more GPUs; the partition rules and the merge formula are
covered on CPU in tests/test_sharding.py."""
import ctypes as C

import numpy as np
import pytest

from tests.conftest import rel_l2

pytestmark = pytest.mark.gpu


def _ptrs(items):
    return (C.c_void_p * len(items))(*items)


def test_broadcast_wait_sum_and_merge(tq):
    torch = pytest.importorskip("torch")
    from turboquant_mlx_core_b200.sharding import merge_attention_parts
    L = tq.load()
    world, batch, hidden = 2, 3, 1024
    slot = batch * hidden                                   # fp16 elements per rank's slot
    nbytes = world * slot * 2
    bufs = [torch.zeros(nbytes + 256, dtype=torch.uint8, device="cuda") for _ in range(world)]
    flags = [b.data_ptr() + nbytes for b in bufs]           # 32 words behind the payload
    ex = [L.tq_exchange_create(r, world) for r in range(world)]
    assert all(ex)
    g = torch.Generator(device="cuda").manual_seed(0)
    for step in range(3):                                   # epochs advance on both sides
        parts = [torch.randn((batch, hidden), generator=g, device="cuda").half() for _ in range(world)]
        for r in range(world):                              # rank r computes its partial into slot r of its own buffer
            bufs[r][r * slot * 2:(r + 1) * slot * 2].view(torch.float16).copy_(parts[r].reshape(-1))
        for r in range(world):                              # ... and sends it to slot r of the other rank
            other = 1 - r
            dst = _ptrs([bufs[other].data_ptr() + r * slot * 2])
            rc = L.tq_exchange_broadcast(ex[r], C.c_void_p(bufs[r].data_ptr() + r * slot * 2), dst, 1, batch, hidden * 2,
                                         hidden * 2, hidden * 2, _ptrs(flags), world, None)
            assert rc == 0, L.tq_last_error().decode()
        outs = []
        for r in range(world):
            assert L.tq_exchange_wait(ex[r], C.c_void_p(flags[r]), world, None) == 0
            out = torch.empty((batch, hidden), dtype=torch.float16, device="cuda")
            assert L.tq_exchange_sum_f16(C.c_void_p(bufs[r].data_ptr()), world, slot, slot, None, C.c_void_p(out.data_ptr()), None) == 0
            outs.append(out)
        torch.cuda.synchronize()
        want = (parts[0].float() + parts[1].float()).half()           # rank order, fp32 accumulate
        assert torch.equal(outs[0], want) and torch.equal(outs[1], want)
        for r in range(world):
            assert L.tq_exchange_status(ex[r]) == 0
            assert bufs[r][nbytes:nbytes + 8].view(torch.int32).tolist() == [step + 1, step + 1]

    # merge of softmax parts against the numpy rule
    rows, dim, nparts = 37, 128, 3
    o = torch.randn((nparts, rows, dim), generator=g, device="cuda").half()
    lse = torch.randn((nparts, rows), generator=g, device="cuda") * 3
    lse[1, 5] = float("-inf")                               # a part that saw no token
    merged = torch.empty((rows, dim), dtype=torch.float16, device="cuda")
    assert L.tq_exchange_merge_attention(C.c_void_p(o.data_ptr()), C.c_void_p(lse.data_ptr()), nparts, rows, dim, rows * dim, rows,
                                         C.c_void_p(merged.data_ptr()), None) == 0
    torch.cuda.synchronize()
    want = merge_attention_parts(o.float().cpu().numpy(), lse.cpu().numpy())
    assert rel_l2(merged.float().cpu().numpy(), want) < 1e-3
    for h in ex:
        L.tq_exchange_free(h)


def test_forward_fused_with_all_gather(tq, oracle):
    """tq_linear_forward_allgather with two ranks emulated on one stream: each rank's kernel computes its
    rows into its own buffer, its last CTA copies them into the other rank's buffer and raises the
    flags, and the next kernel's CTAs find the previous exchange complete when they wait for it."""
    torch = pytest.importorskip("torch")
    L = tq.load()
    rng = np.random.default_rng(21)
    cb = oracle.codebook(4)[0]
    world, rows, cols = 2, 208, 512           # per-rank rows; the gathered layer has world * rows
    total = world * rows
    lins = []
    for r in range(world):
        w = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float16).astype(np.float32)
        pp, pr, norms, seeds = oracle.quantize_weight(w, cb, cb, 4, 4, 128, True)
        lins.append(tq.TurboQuantLinear(cols, rows, tq.QuantizedWeight(pp, pr, norms, seeds), tq.codebook_from_centroids(cb),
                                        tq.codebook_from_centroids(cb), 128))
    for batch in (1, 3):
        nbytes = batch * total * 2
        bufs = [torch.zeros(nbytes + 256, dtype=torch.uint8, device="cuda") for _ in range(world)]
        flags = [b.data_ptr() + nbytes for b in bufs]
        ex = [L.tq_exchange_create(r, world) for r in range(world)]
        x = torch.from_numpy(rng.standard_normal((batch, cols)).astype(np.float16)).cuda()
        want = torch.cat([lin.forward(x) for lin in lins], dim=1)
        for step in range(3):
            for r in range(world):
                dst = _ptrs([bufs[r].data_ptr(), bufs[1 - r].data_ptr()])       # own buffer first
                wait = C.c_void_p(flags[r]) if step > 0 else None             # nothing to wait for before the first exchange
                rc = L.tq_linear_forward_allgather(lins[r].handle, ex[r], C.c_void_p(x.data_ptr()), batch, dst, world, total, r * rows,
                                                   _ptrs(flags), world, wait, world, None)
                assert rc == 0, L.tq_last_error().decode()
            torch.cuda.synchronize()
            for r in range(world):
                got = bufs[r][:nbytes].view(torch.float16).view(batch, total)
                assert torch.equal(got, want), (batch, step, r)
                assert bufs[r][nbytes:nbytes + 8].view(torch.int32).tolist() == [step + 1, step + 1]
            for b in bufs:
                b[:nbytes].zero_()
        for r in range(world):
            assert L.tq_exchange_wait(ex[r], C.c_void_p(flags[r]), world, None) == 0   # the last exchange
            assert L.tq_exchange_status(ex[r]) == 0
            lins[r].check_status()
            L.tq_exchange_free(ex[r])
    for lin in lins:
        lin.close()


def test_forward_fused_with_packet_all_gather(tq, oracle):
    """tq_linear_forward_allgather_packets with two ranks emulated on one stream: each rank's kernel stores its
    rows locally and its last CTA writes them to the other rank as {2 halves, epoch, 2 halves, epoch} packets
    (region [epoch parity][source rank]); the next step's kernels poll those packets before they start, and
    tq_exchange_unpack_packets gives the rows back."""
    torch = pytest.importorskip("torch")
    L = tq.load()
    rng = np.random.default_rng(22)
    cb = oracle.codebook(4)[0]
    world, rows, cols = 2, 208, 512
    lins = []
    for r in range(world):
        w = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float16).astype(np.float32)
        pp, pr, norms, seeds = oracle.quantize_weight(w, cb, cb, 4, 4, 128, True)
        lins.append(tq.TurboQuantLinear(cols, rows, tq.QuantizedWeight(pp, pr, norms, seeds), tq.codebook_from_centroids(cb),
                                        tq.codebook_from_centroids(cb), 128))
    for batch in (1, 3):
        n_pk = batch * rows // 4
        bufs = [torch.zeros(2 * world * n_pk * 16, dtype=torch.uint8, device="cuda") for _ in range(world)]
        ex = [L.tq_exchange_create(r, world) for r in range(world)]
        for step in range(4):
            x = torch.from_numpy(rng.standard_normal((batch, cols)).astype(np.float16)).cuda()
            want = [lin.forward(x) for lin in lins]
            ys = [torch.zeros((batch, rows), dtype=torch.float16, device="cuda") for _ in range(world)]
            for r in range(world):
                rc = L.tq_linear_forward_allgather_packets(lins[r].handle, ex[r], C.c_void_p(x.data_ptr()), batch,
                                                           C.c_void_p(ys[r].data_ptr()), rows, _ptrs([b.data_ptr() for b in bufs]),
                                                           1 if step > 0 else 0, None)
                assert rc == 0, L.tq_last_error().decode()
            torch.cuda.synchronize()
            parity = (step + 1) & 1
            for r in range(world):
                assert torch.equal(ys[r], want[r]), (batch, step, r)
                src = 1 - r
                region = bufs[r][(parity * world + src) * n_pk * 16:(parity * world + src + 1) * n_pk * 16]
                pk = region.view(torch.int32).view(n_pk, 4)
                assert bool((pk[:, 1] == step + 1).all()) and bool((pk[:, 3] == step + 1).all())
                got = torch.empty((batch, rows), dtype=torch.float16, device="cuda")
                assert L.tq_exchange_unpack_packets(C.c_void_p(region.data_ptr()), n_pk, C.c_void_p(got.data_ptr()), None) == 0
                torch.cuda.synchronize()
                assert torch.equal(got, want[src]), (batch, step, r)
        # the last exchange has not been waited for yet (each step's kernels waited for the one before): the waiting
        # kernel puts the other rank's rows beside this rank's own in the gathered result
        for r in range(world):
            gathered = torch.zeros((batch, world * rows), dtype=torch.float16, device="cuda")
            gathered[:, r * rows:(r + 1) * rows] = ys[r]
            assert L.tq_exchange_wait_packets(ex[r], C.c_void_p(bufs[r].data_ptr()), rows, batch, C.c_void_p(gathered.data_ptr()),
                                              world * rows, None) == 0
            torch.cuda.synchronize()
            assert torch.equal(gathered, torch.cat(want, dim=1)), (batch, r)
        # the same packets as the partial sums of an all-reduce: residual + the ranks' rows in rank order, fp32
        # (each rank's second waiting call of this exchange: the packets are still there, the epoch is the same)
        resid = torch.from_numpy(rng.standard_normal((batch, rows)).astype(np.float16)).cuda()
        for r in range(world):
            out = torch.empty((batch, rows), dtype=torch.float16, device="cuda")
            assert L.tq_exchange_sum_packets(ex[r], C.c_void_p(bufs[r].data_ptr()), C.c_void_p(ys[r].data_ptr()), batch * rows,
                                             C.c_void_p(resid.data_ptr()), C.c_void_p(out.data_ptr()), None) == 0
            torch.cuda.synchronize()
            acc = resid.float()
            for src in range(world):
                acc = acc + want[src].float()
            assert torch.equal(out, acc.half()), (batch, r)
            # the same sum followed in the same kernel by the RMSNorm of the summed rows (rows of 4-element groups)
            if rows % 4 == 0:
                wn = torch.from_numpy((1 + 0.1 * rng.standard_normal(rows)).astype(np.float16)).cuda()
                out2, normed2, normed = torch.empty_like(out), torch.empty_like(out), torch.empty_like(out)
                assert L.tq_exchange_sum_packets_rmsnorm(ex[r], C.c_void_p(bufs[r].data_ptr()), C.c_void_p(ys[r].data_ptr()), batch, rows,
                                                         C.c_void_p(resid.data_ptr()), C.c_void_p(out2.data_ptr()),
                                                         C.c_void_p(wn.data_ptr()), C.c_void_p(normed2.data_ptr()), 1e-6, None) == 0
                assert L.tq_rmsnorm_f16(C.c_void_p(out.data_ptr()), C.c_void_p(wn.data_ptr()), C.c_void_p(normed.data_ptr()), batch, rows,
                                        1e-6, None) == 0
                torch.cuda.synchronize()
                assert torch.equal(out2, out) and torch.equal(normed2, normed), (batch, r)
        for r in range(world):
            assert L.tq_exchange_status(ex[r]) == 0
            lins[r].check_status()
            L.tq_exchange_free(ex[r])
    for lin in lins:
        lin.close()


def test_wait_for_a_flag_nobody_raises_gives_up(tq):
    """A rank that never broadcasts: the wait runs out after its limit (about a second) and the
    status says so; the device stays usable."""
    torch = pytest.importorskip("torch")
    L = tq.load()
    flags = torch.zeros(32, dtype=torch.int32, device="cuda")
    ex = L.tq_exchange_create(0, 2)
    assert L.tq_exchange_wait(ex, C.c_void_p(flags.data_ptr()), 2, None) == 0
    assert L.tq_exchange_status(ex) != 0
    assert b"did not arrive" in L.tq_last_error()
    L.tq_exchange_free(ex)
    assert int(torch.ones(4, device="cuda").sum()) == 4
    # argument checks
    ex = L.tq_exchange_create(0, 1)
    buf = torch.zeros(1024, dtype=torch.uint8, device="cuda")
    bad = L.tq_exchange_broadcast(ex, C.c_void_p(buf.data_ptr()), _ptrs([buf.data_ptr()]), 1, 1, 24, 24, 24,
                                  _ptrs([flags.data_ptr()]), 1, None)
    assert bad != 0                                         # rows must be a multiple of 16 bytes
    assert L.tq_exchange_create(3, 2) is None
    L.tq_exchange_free(ex)
