#!/usr/bin/env python
"""Benchmark of the TurboQuant hot path on B200.

Headline workload: TQ8 fused dequant-GEMV, weight 4096x4096 drawn
N(0, 0.02^2) in fp16, row-normalised, blocked WHT (block 128) after a seeded sign
diagonal, 4-bit Lloyd-Max primary + 4-bit Lloyd-Max residual codebooks fitted to the
data, batch-1 fp16 activation ~ N(0,1).  A step is one pass over NBUF distinct weight
matrices (NBUF * 16.8 MB >> L2), one GEMV each, so every launch streams its codes from
HBM.  metric = layer-forwards ("tokens" through this layer) per second.

  python bench.py [--gpus N] [--steps K] [--warmup W]          the CUDA library
  python bench.py --impl reference [...]                       the reference's CPU path

Prints ONE JSON line (rank 0).  With N > 1 (torchrun, one rank per GPU) every rank runs
its own NBUF matrices (independent layers, no collective on this path: weak scaling).

Secondary measurements ride in the same line (--legs selects, --no-extras drops them):
  attention      decode attention over the compressed cache, 16 sequences, 4k / 32k / 128k context;
                 KV heads split over ranks, the context range as well beyond 4 ranks
  decoder_layer  the seven projections of a Qwen2.5-7B-shaped layer at batch 1 / 8 / 64
  prefill        2048 activation rows through the tcgen05 GEMM
  lm_head        151936 x 2048 at batch 1 / 32, rows sharded over the ranks: NCCL all-gather of the
                 logits, and the fused variant (peer stores from the GEMV + completion flags)
  side_kernels   dequantise, blocked WHT, KV append (bulk, one token x 16 sequences), KV decode
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

OUT_F, IN_F, BLOCK = 4096, 4096, 128
ALGO_BYTES = OUT_F * IN_F + 4 * OUT_F + 2 * IN_F + 2 * OUT_F   # codes + norms + x + y = 16 809 984
PUBLISHED_TOK_S = 671.0   # reference README: 1.49 ms/token, Apple GPU, same shape, block 512
# dram__bytes_read.sum + dram__bytes_write.sum of one tq8_gemv_kernel launch at this shape
# (from an ncu capture of that launch): reads only, no DRAM writes.
GEMV_DRAM_TRAFFIC = 16824704


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ---- clocks --------------------------------------------------------------------------------

class ClockSampler:
    """Samples SM clock and clock-event reasons of one GPU from a thread while the timed region
    runs (NVML reads only; nothing is set).  A timed region of a few milliseconds is shorter
    than one nvidia-smi start-up, hence NVML in-process with a ~1 ms period."""
    REASONS = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20),
               ("sw_power_cap", 0x4))

    def __init__(self, device):
        import threading
        self.samples, self.bits, self.max_mhz, self.err = [], 0, None, None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            import torch
            pynvml.nvmlInit()
            self.nv = pynvml
            uuid = str(torch.cuda.get_device_properties(device).uuid)
            try:
                self.h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(device.index or 0)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception as exc:  # no NVML: say so in the line instead of failing the bench
            self.nv, self.err = None, f"NVML unavailable: {type(exc).__name__}"

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                self.bits |= int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
            except Exception as exc:
                self.err = f"NVML read failed: {type(exc).__name__}"
                return
            time.sleep(0.001)

    def start(self):
        if self.nv is None:
            return
        import threading
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def stop(self):
        if self._thread is not None:
            self._stop.set()
            self._thread.join(timeout=2)
        reasons = [name for name, bit in self.REASONS if self.bits & bit]
        if self.err:
            reasons.append(self.err)
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": reasons, "samples": len(self.samples)}


# ---- synthetic inputs ------------------------------------------------------------------------

def build_codebooks(tq, w0):
    """Per-layer codebooks as the reference's converter fits them (src/converter.cpp:291-372): primary on
    the rotated, scaled weights; residual on what the shared primary codebook leaves; Lloyd-Max on the
    device through the library (tq_fit_layer_codebooks)."""
    return tq.fit_layer_codebooks(w0, BLOCK, 4, 4, 100)


def make_layer(tq, seed, device, cbs=None, out_f=OUT_F, in_f=IN_F):
    import torch
    g = torch.Generator(device=device).manual_seed(seed)
    w = (torch.randn((out_f, in_f), generator=g, device=device, dtype=torch.float32) * 0.02).half().float()
    if cbs is None:
        cbs = build_codebooks(tq, w)
    qw = tq.quantize_weight(w, cbs[0], cbs[1], tq.QuantizerConfig(4, 4, BLOCK, True))
    lin = tq.TurboQuantLinear(in_f, out_f, qw, cbs[0], cbs[1], BLOCK)
    return lin, qw, cbs


# ---- the CUDA arm ------------------------------------------------------------------------------

def run_cuda(args):
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)

    import turboquant_mlx_core_b200 as tq
    L = tq.load()
    if L.tq_set_device(local_rank) != 0:
        raise SystemExit("tq_set_device failed: " + L.tq_last_error().decode())

    nbuf = args.nbuf
    layers = []
    lin0, qw0, cbs = make_layer(tq, 1000 * rank, device)
    layers.append(lin0)
    for i in range(1, nbuf):
        layers.append(make_layer(tq, 1000 * rank + i, device, cbs)[0])
    g = torch.Generator(device=device).manual_seed(7 + rank)
    x_dev = torch.randn((nbuf, IN_F), generator=g, device=device, dtype=torch.float32).half()
    y_dev = torch.empty((nbuf, OUT_F), device=device, dtype=torch.float16)
    x_host = x_dev.cpu().pin_memory()
    y_host = torch.empty((nbuf, OUT_F), dtype=torch.float16).pin_memory()

    stream = torch.cuda.Stream(device=device)
    sp = C.c_void_p(stream.cuda_stream)

    # With more than one rank the headline is the row-sharded layer of the sharded paths: every rank
    # holds a 4096 x 4096 row shard of a (4096 * N) x 4096 layer, and after every layer-forward the
    # fp16 output shards are all-gathered (each rank stores its 8 KB into every rank's buffer over
    # NVLink and raises its flag; a one-warp kernel waits for all flags).  Two gather buffers
    # alternate.  If the shared buffers cannot be mapped on every rank, the ranks run independent
    # layers and the line says so.
    exchange, exchange_note = None, None
    if world > 1:
        from turboquant_mlx_core_b200.sharding import Exchange
        err = None
        try:
            # [2 gather buffers][world][OUT_F] fp16, then the packet area of the flag-in-data variant:
            # [2 epoch parities][world source ranks][OUT_F / 4 packets of 16 bytes]
            exchange = Exchange(2 * world * OUT_F * 2 + 2 * world * OUT_F * 4)
        except Exception as exc:
            err = str(exc)
        ok_t = torch.tensor([0.0 if err else 1.0], device=device)
        dist.all_reduce(ok_t, op=dist.ReduceOp.MIN)
        if ok_t.item() != 1.0:
            if exchange is not None:
                exchange.close()
            exchange, exchange_note = None, "shared buffers could not be mapped on every rank: independent layers, no exchange"

    gather_mode = os.environ.get("TQ_BENCH_GATHER", "packets")
    fused_gather = gather_mode != "split"
    packets_off = 2 * world * OUT_F * 2
    if exchange is not None:
        torch.cuda.synchronize()
        dist.barrier()
        # every fused call below waits for the exchange before it; this one is there for the first
        with torch.cuda.stream(stream):
            if gather_mode == "packets":
                exchange.forward_allgather_packets(layers[-1], x_dev[nbuf - 1:nbuf], y_dev[nbuf - 1:nbuf], packets_off, wait=False,
                                                   stream=stream)
            else:
                exchange.broadcast(0, 1, 16, 16, stream=stream)

    def one_pass():
        for i, lin in enumerate(layers):
            if exchange is None:
                rc = L.tq_linear_forward(lin.handle, C.c_void_p(x_dev[i].data_ptr()), tq.TQ_F16, 1,
                                         C.c_void_p(y_dev[i].data_ptr()), sp)
                if rc:
                    raise RuntimeError(L.tq_last_error().decode())
            elif gather_mode == "packets":
                # ONE kernel per layer: poll the packets of the previous layer's gather, GEMV into this rank's own rows,
                # then the last CTA writes them to the other ranks as {data, epoch} packets: no fence, no flag store
                exchange.forward_allgather_packets(lin, x_dev[i:i + 1], y_dev[i:i + 1], packets_off, wait=True, stream=stream)
            elif fused_gather:
                # ONE kernel per layer: wait for the previous layer's gather, GEMV into this rank's rows of
                # the gathered output, copy them to the peers, raise the flags
                exchange.forward_allgather(lin, x_dev[i:i + 1], world * OUT_F, rank * OUT_F,
                                           buffer_offset=(i & 1) * world * OUT_F * 2, wait=True, stream=stream)
            else:
                # three kernels per layer: wait for the previous gather, GEMV in place, copy + flags
                off = ((i & 1) * world + rank) * OUT_F * 2
                exchange.wait(stream=stream)
                rc = L.tq_linear_forward(lin.handle, C.c_void_p(x_dev[i].data_ptr()), tq.TQ_F16, 1,
                                         C.c_void_p(exchange.local + off), sp)
                if rc:
                    raise RuntimeError(L.tq_last_error().decode())
                exchange.broadcast(off, 1, OUT_F * 2, OUT_F * 2, stream=stream)

    # The exchange's waits give up after a second, so the ranks must be within a second of each other
    # when the first exchanging kernel starts: set-up times differ by more than that.
    if world > 1:
        torch.cuda.synchronize()
        dist.barrier()
    # the launch-bound inner loop is captured once and replayed
    with torch.cuda.stream(stream):
        one_pass()
    stream.synchronize()
    launch_mode = "CUDA graph of one GEMV per layer" + ("" if exchange is None else
                                                         " fused with the wait for the previous gather and the peer copy of its output as "
                                                         "flag-in-data packets" if gather_mode == "packets" else
                                                         " fused with the wait for the previous gather, the peer copy of its output and the flags"
                                                         if fused_gather else " + tq_exchange_wait before and tq_exchange_broadcast after it")
    try:
        if args.no_graph:
            raise RuntimeError("graph disabled by flag")
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            one_pass()
    except Exception as exc:  # capture refused: time plain launches and say so
        launch_mode = f"plain launches (graph capture failed: {type(exc).__name__})"
        torch.cuda.synchronize()

        class _Plain:
            @staticmethod
            def replay():
                one_pass()
        graph = _Plain()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(device)
    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            graph.replay()
    barrier()
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    with torch.cuda.stream(stream):
        e0.record(stream)
        for _ in range(args.steps):
            graph.replay()
        e1.record(stream)
    barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    t = torch.tensor([ms], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max = float(t.item())
    launches = args.steps * nbuf
    value = world * launches / (ms_max * 1e-3)

    # ---- end to end through the C-ABI with host buffers ----
    e2e_steps = max(3, args.steps // 20)

    def e2e_pass():
        for i, lin in enumerate(layers):
            rc = L.tq_linear_forward(lin.handle, C.c_void_p(x_host[i].data_ptr()), tq.TQ_F16, 1,
                                     C.c_void_p(y_host[i].data_ptr()), sp)
            if rc:
                raise RuntimeError(L.tq_last_error().decode())

    for _ in range(3):
        e2e_pass()
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record(stream)
    for _ in range(e2e_steps):
        e2e_pass()
    f1.record(stream)
    barrier()
    e2e_ms = torch.tensor([f0.elapsed_time(f1)], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    e2e_value = world * e2e_steps * nbuf / (float(e2e_ms.item()) * 1e-3)

    # parity guard on what was timed: the device and host paths must agree bit for bit
    torch.cuda.synchronize()
    gathered_ok = None
    if exchange is None:
        same = bool(torch.equal(y_dev.cpu(), y_host))
    elif gather_mode == "packets":
        # every rank has finished its kernels, so every packet has landed: the two epoch parities hold the last two
        # layers' rows of every OTHER rank; this rank's own rows are in y_dev
        dist.barrier()
        torch.cuda.synchronize()
        exchange.check_status()
        for lin in layers:
            lin.check_status()
        same = bool(torch.equal(y_dev.cpu(), y_host))
        n_pk = OUT_F // 4
        raw = exchange.buf.tensor((packets_off + 2 * world * n_pk * 16,), torch.uint8)[packets_off:].view(torch.int32).view(2, world, n_pk, 4)
        other = (rank + 1) % world
        newest = 0 if int(raw[0, other, 0, 1].item()) > int(raw[1, other, 0, 1].item()) else 1   # parity of the last layer's epoch
        gath = torch.empty((2, world, OUT_F), device=device, dtype=torch.float16)
        for k, parity in enumerate((1 - newest, newest)):            # k = 0: layer nbuf - 2, k = 1: layer nbuf - 1
            for src in range(world):
                if src == rank:
                    gath[k, src] = y_dev[nbuf - 2 + k]
                else:
                    exchange.unpack_packets(packets_off + ((parity * world + src) * n_pk) * 16, n_pk, gath[k, src], stream=None)
        torch.cuda.synchronize()
        ref = gath.clone()
        dist.broadcast(ref, src=0)
        ok = torch.tensor([1.0 if torch.equal(ref, gath) else 0.0], device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        gathered_ok = bool(ok.item() == 1.0)
    else:
        # the last two layers' gathered outputs sit in the two buffers: this rank's slots must equal
        # the host path's results, and every rank must hold the same gathered bytes
        with torch.cuda.stream(stream):
            exchange.wait(stream=stream)          # the last layer's gather
        exchange.check_status()
        for lin in layers:
            lin.check_status()
        gath = exchange.buf.tensor((2, world, OUT_F), torch.float16).clone()
        same = all(bool(torch.equal(gath[i & 1, rank].cpu(), y_host[i])) for i in (nbuf - 2, nbuf - 1))
        # layers differ per rank, so compare every rank's copy of the gathered block with rank 0's
        ref = gath.clone()
        dist.broadcast(ref, src=0)
        ok = torch.tensor([1.0 if torch.equal(ref, gath) else 0.0], device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        gathered_ok = bool(ok.item() == 1.0)

    peak, peak_kind = measured_peaks()
    per_launch_s = ms_max * 1e-3 / launches
    achieved = ALGO_BYTES / per_launch_s / 1e9
    line = {
        "metric": "tq8_dequant_gemv_4096x4096_b1_tok_per_s", "value": value, "unit": "tok/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_max / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": value / world / PUBLISHED_TOK_S if world == 1 else None,
        "dtype": "tf32 multiply, fp32 accumulate (fp16 activations in, fp16 out)", "data": "synthetic",
        "config": {"workload": "TQ8 4+4-bit fused dequant-GEMV, 4096x4096, block 128, shared rotation, "
                               "fitted Lloyd-Max codebooks, batch 1",
                   "layers_per_step": nbuf, "l2_policy": f"{nbuf} distinct weight matrices per step "
                                                         f"({nbuf * OUT_F * IN_F / 1e6:.0f} MB) "
                                                         + ("> L2" if nbuf * OUT_F * IN_F > 126e6 else "<= L2 (126 MB): not a valid HBM measurement"),
                   "launch": launch_mode,
                   "per_gpu": ("independent layers, no collective" if exchange is None else
                               "one 4096 x 4096 row shard of a (4096 N) x 4096 layer per launch; after every layer the fp16 output "
                               "shards are all-gathered over NVLink (peer stores" + (" of {data, epoch} packets" if gather_mode == "packets"
                                                                                    else " + flags") + ", no collective library)"),
                   "exchange_note": exchange_note,
                   "vs_baseline_note": "published 671 tok/s is the reference on an Apple GPU at block 512"},
        "gb_per_s": achieved * world,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "frac_of_nominal_8tbs": achieved / 8000.0, "peak_kind": peak_kind + " (burst copy)",
                     "algorithmic_bytes_per_launch": ALGO_BYTES, "us_per_launch": per_launch_s * 1e6,
                     "traffic": GEMV_DRAM_TRAFFIC},
        "e2e": {"value": e2e_value, "unit": "tok/s", "h2d_bytes_per_step": nbuf * IN_F * 2,
                "d2h_bytes_per_step": nbuf * OUT_F * 2, "steps": e2e_steps,
                "path": "tq_linear_forward with pinned host x and y, one call per layer"},
        "gpu_launches": launches,
        "clocks": clocks,
        "device_host_paths_bit_identical": same,
    }
    if gathered_ok is not None:
        line["gathered_outputs_identical_on_every_rank"] = gathered_ok
    if exchange is not None:
        exchange.close()

    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(qw0, cbs, x_host[0].numpy(), y_dev[0].cpu().numpy(), budget_s=12.0)
    legs = set(args.legs.split(",")) if args.legs else {"attention", "decoder_layer", "prefill", "lm_head", "side_kernels", "c4_decode_step"}
    if args.no_extras:
        legs = set()
    if "attention" in legs:
        try:
            line["attention"] = bench_attention(tq, L, device, stream, rank, world, args, args.attn_ctx)
            if world == 1 and args.attn_ctx == 32768:
                line["attention_ctx4k"] = bench_attention(tq, L, device, stream, rank, world, args, 4096)
                line["attention_ctx128k"] = bench_attention(tq, L, device, stream, rank, world, args, 131072)
        except Exception as e:  # secondary measurement: report, do not hide the headline
            line["attention"] = {"error": str(e)}
    if "decoder_layer" in legs and world == 1:
        try:
            line["decoder_layer"] = bench_decoder_layer(tq, L, device, stream, cbs, args)
        except Exception as e:
            line["decoder_layer"] = {"error": str(e)}
    if "side_kernels" in legs and world == 1:
        try:
            line["side_kernels"] = bench_side_kernels(tq, L, layers, device, stream, args)
        except Exception as e:
            line["side_kernels"] = {"error": str(e)}
    if "prefill" in legs:
        try:
            line["prefill"] = bench_prefill(tq, L, layers, device, stream, args)
        except Exception as e:
            line["prefill"] = {"error": str(e)}
        if world > 1:
            try:
                line["prefill_sharded"] = bench_prefill_sharded(tq, L, device, stream, rank, world, cbs, args)
            except Exception as e:
                line["prefill_sharded"] = {"error": str(e)}
    if "lm_head" in legs:
        try:
            line["lm_head"] = bench_lm_head(tq, L, device, stream, rank, world, cbs, args)
        except Exception as e:
            line["lm_head"] = {"error": str(e)}
    if "c4_decode_step" in legs:
        try:
            line["c4_decode_step"] = bench_c4_decode_step(tq, L, device, stream, rank, world, cbs, args)
        except Exception as e:
            line["c4_decode_step"] = {"error": str(e)}
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line))


# ---- secondary: compressed-cache decode attention (16 sequences, 4 KV / 28 query heads) ---------------------------

def bench_attention(tq, L, device, stream, rank, world, args, ctx):
    """16 sequences, 4 KV / 28 query heads, d 128, QJL on.  Up to 4 ranks split the KV heads (heads
    are independent).  With more ranks than KV heads the ranks sharing a head split the context
    range, each computes a partial result with its log-sum-exp, and an all-gather over the
    world followed by a merge gives every rank the full result (timed inside the region)."""
    import torch
    import torch.distributed as dist
    from turboquant_mlx_core_b200.sharding import attention_grid, context_range, merge_attention_parts
    kv_heads = args.attn_kv_heads
    n_seqs, q_heads, dim = 16, 7 * kv_heads, 128
    if world > kv_heads and world % kv_heads:
        return {"skipped": f"{world} ranks over {kv_heads} KV heads: rank count must be a multiple of the heads"}
    h0, h1, part, parts = attention_grid(kv_heads, rank, world)
    heads_local = h1 - h0
    qh_local = q_heads // kv_heads * heads_local
    c0, c1 = context_range(0, ctx, part, parts)
    ctx_local = c1 - c0
    g = torch.Generator(device=device).manual_seed(100 + rank)
    caches = []
    for s in range(n_seqs):
        c = tq.TQKVCache(1, heads_local, dim)
        for t0 in range(0, ctx_local, 8192):
            n = min(8192, ctx_local - t0)
            k = torch.randn((n, heads_local, dim), generator=g, device=device)
            v = torch.randn((n, heads_local, dim), generator=g, device=device)
            k[:, :, ::20] *= 8.0          # ~5 % outlier channels
            v[:, :, ::20] *= 8.0
            c.append(0, k.half(), v.half())
        caches.append(c)
    q = torch.randn((n_seqs, qh_local, dim), generator=g, device=device).half()
    out = torch.empty_like(q)
    lse = torch.empty((n_seqs, qh_local), device=device, dtype=torch.float32)
    arr = (C.c_void_p * n_seqs)(*[c.handle for c in caches])
    sp = C.c_void_p(stream.cuda_stream)
    # Ranks that share a KV head (more ranks than heads) exchange their (output | log-sum-exp) parts by
    # peer stores and merge them with one small kernel: slot `part` of the buffer of every rank that
    # shares the head; two buffers alternate.
    rows = n_seqs * qh_local
    out_bytes, slot_bytes = rows * dim * 2, rows * dim * 2 + rows * 4
    exchange, merge_path = None, None
    if parts > 1:
        from turboquant_mlx_core_b200.sharding import Exchange
        err = None
        try:
            exchange = Exchange(2 * parts * slot_bytes)
        except Exception as exc:
            err = str(exc)
        ok_t = torch.tensor([0.0 if err else 1.0], device=device)
        dist.all_reduce(ok_t, op=dist.ReduceOp.MIN)
        if ok_t.item() != 1.0:
            if exchange is not None:
                exchange.close()
            return {"skipped": "shared buffers could not be mapped on every rank", "local_error": err}
        sharing = [h0 + kv_heads * p for p in range(parts) if h0 + kv_heads * p != rank]
        peer_idx = [1 + (r if r < rank else r - 1) for r in sharing]
        merge_path = "parts exchanged by tq_exchange_broadcast (peer stores + flags), merged by tq_exchange_merge_attention"
    step = [0]

    def call():
        if exchange is None:
            o_ptr, l_ptr = out.data_ptr(), lse.data_ptr()
        else:
            base = (step[0] & 1) * parts * slot_bytes
            step[0] += 1
            o_ptr = exchange.local + base + part * slot_bytes
            l_ptr = o_ptr + out_bytes
        rc = L.tq_kv_attention_lse(arr, n_seqs, 0, C.c_void_p(q.data_ptr()), tq.TQ_F16, qh_local,
                                   C.c_void_p(o_ptr), C.c_void_p(l_ptr), 0, -1, 1, sp)
        if rc:
            raise RuntimeError(L.tq_last_error().decode())
        if exchange is not None:
            exchange.broadcast(base + part * slot_bytes, 1, slot_bytes, slot_bytes, stream=stream, peers=peer_idx)
            exchange.wait(stream=stream)
            exchange.merge_attention(base, base + out_bytes, parts, rows, dim, slot_bytes // 2, slot_bytes // 4, out.data_ptr(),
                                     stream=stream)
        return out

    # (launched eagerly: the attention entry point stages its per-sequence descriptors from host memory
    # on every call, so it cannot be captured in a CUDA graph)
    per_call = 1

    if world > 1:                          # exchanging kernels wait a second at most: start together
        torch.cuda.synchronize()
        dist.barrier()
    with torch.cuda.stream(stream):
        for _ in range(3):
            call()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    reps = 10
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        e0.record(stream)
        for _ in range(reps):
            call()
        e1.record(stream)
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) * 1e3 / (reps * per_call)], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    us = float(t.item())
    algo = n_seqs * heads_local * ctx_local * 118          # compact bytes per (token, KV head) with QJL
    peak, kind = measured_peaks()
    merged_ok = None
    if exchange is not None:
        # the merged result must equal what the torch-side rule gives on all-gathered parts
        exchange.check_status()
        mine = exchange.buf.tensor((2, parts, slot_bytes), torch.uint8)[0].clone()
        o_parts = mine[:, :out_bytes].contiguous().view(torch.float16).view(parts, rows, dim)
        l_parts = mine[:, out_bytes:].contiguous().view(torch.float32).view(parts, rows)
        want = merge_attention_parts(o_parts, l_parts)
        err = float((out.float().view(rows, dim) - want).norm() / want.norm().clamp_min(1e-30))
        ok = torch.tensor([1.0 if err < 1e-3 else 0.0], device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        merged_ok = bool(ok.item() == 1.0)
        exchange.close()
    for c in caches:
        c.close()
    return {"workload": f"{n_seqs} seqs x ctx {ctx}, {kv_heads} KV / {q_heads} query heads, d {dim}, QJL on",
            "merge_of_context_parts": merge_path, "merged_result_matches_rule_on_every_rank": merged_ok,
            "us_per_layer_step": us, "tok_per_s": n_seqs / (us * 1e-6), "gb_per_s_per_gpu": algo / (us * 1e-6) / 1e9,
            "frac_of_peak": algo / (us * 1e-6) / 1e9 / peak, "peak_kind": kind, "kv_heads_per_gpu": heads_local,
            "context_parts": parts,
            "l2_policy": f"cache {n_seqs * heads_local * ctx_local * 132 / 1e6:.0f} MB per GPU "
                         + ("> L2" if n_seqs * heads_local * ctx_local * 132 > 126e6 else "<= L2 (126 MB)")}


# ---- secondary: the memory-bound side kernels of the path (dequantise, rotation, KV encode / decode) ---

def bench_side_kernels(tq, L, layers, device, stream, args):
    """Device-resident inputs and outputs, CUDA events, inputs larger than L2 where the kernel
    streams (8 distinct layers / matrices per pass)."""
    import torch
    sp = C.c_void_p(stream.cuda_stream)
    peak, kind = measured_peaks()
    res = {"peak_kind": kind}

    def timed(fn, reps=5):
        with torch.cuda.stream(stream):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record(stream)
            for _ in range(reps):
                fn()
            e1.record(stream)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / reps

    n = min(len(layers), 8)
    # dequantise to fp16: 1 B read + 2 B written per weight
    outs = [torch.empty((OUT_F, IN_F), dtype=torch.float16, device=device) for _ in range(n)]

    def deq():
        for lin, o in zip(layers[:n], outs):
            if L.tq_linear_dequantize(lin.handle, C.c_void_p(o.data_ptr()), tq.TQ_F16, sp):
                raise RuntimeError(L.tq_last_error().decode())
    us = timed(deq) / n
    b = OUT_F * IN_F * 3
    res["dequantize_f16_4096x4096"] = {"us": us, "gb_per_s": b / (us * 1e-6) / 1e9, "frac_of_peak": b / (us * 1e-6) / 1e9 / peak}
    del outs
    # blocked WHT rotation of an fp32 matrix: 4 B read + 4 B written per element
    ms = [torch.randn((OUT_F, IN_F), device=device) for _ in range(n)]
    rot = torch.empty((OUT_F, IN_F), device=device)

    def wht():
        for m_ in ms:
            if L.tq_wht_rotate(C.c_void_p(m_.data_ptr()), C.c_void_p(rot.data_ptr()), OUT_F, IN_F, 1234, BLOCK, 0, sp):
                raise RuntimeError(L.tq_last_error().decode())
    us = timed(wht) / n
    b = OUT_F * IN_F * 8
    res["wht_rotate_f32_4096x4096"] = {"us": us, "gb_per_s": b / (us * 1e-6) / 1e9, "frac_of_peak": b / (us * 1e-6) / 1e9 / peak}
    del ms, rot
    # KV encode (append): bulk 8192 tokens x 4 heads x 128, and one token for 16 sequences
    heads, dim = 4, 128
    k = torch.randn((8192, heads, dim), device=device).half()
    v = torch.randn((8192, heads, dim), device=device).half()
    cache = tq.TQKVCache(1, heads, dim)
    cache.reserve(0, 16 * 8192)           # no growth (allocation + copy) inside the timed region
    with torch.cuda.stream(stream):
        for _ in range(8):
            cache.append(0, k, v, stream=stream)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        e0.record(stream)
        for _ in range(8):
            cache.append(0, k, v, stream=stream)
        e1.record(stream)
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / 8
    b = 8192 * heads * (2 * dim * 2 + 132)
    res["kv_append_8192_tokens"] = {"us": us, "tok_per_s": 8192 / (us * 1e-6), "gb_per_s": b / (us * 1e-6) / 1e9,
                                    "frac_of_peak": b / (us * 1e-6) / 1e9 / peak}
    # decode of the compressed keys back to fp16 (get_keys_fp16): 56 B read + 256 B written per vector
    out = torch.empty((65536, heads, dim), dtype=torch.float16, device=device)

    def dec():
        if L.tq_kv_get_fp16(cache.handle, 0, 0, 0, 65536, C.c_void_p(out.data_ptr()), sp):
            raise RuntimeError(L.tq_last_error().decode())
    us = timed(dec)
    b = 65536 * heads * (56 + 2 * dim)
    res["kv_get_keys_fp16_65536_tokens"] = {"us": us, "gb_per_s": b / (us * 1e-6) / 1e9, "frac_of_peak": b / (us * 1e-6) / 1e9 / peak}
    cache.close()
    seqs = [tq.TQKVCache(1, heads, dim) for _ in range(16)]
    for c in seqs:
        c.reserve(0, 4096)
    k1 = torch.randn((1, heads, dim), device=device).half()
    k16 = torch.randn((16, heads, dim), device=device).half()

    def step():
        for c in seqs:
            c.append(0, k1, k1, stream=stream)
    us = timed(step, reps=20)
    res["kv_append_1_token_x16_seqs"] = {"us_per_step_16_calls": us}
    us = timed(lambda: tq.append_batch(seqs, 0, k16, k16, stream=stream), reps=20)
    res["kv_append_1_token_x16_seqs"]["us_per_step_batched_call"] = us
    for c in seqs:
        c.close()

    # hybrid_attention's window branch: one query position over a 131 072-token fp16 decode window
    # (4 KV / 28 query heads, d 128): 4 * head_dim bytes per (token, KV head) = 268 MB > L2
    try:
        wtok, wheads, wq = 131072, 4, 28
        kfull = torch.randn((wtok, wheads, dim), device=device).half()
        wcache = tq.TQKVCache(1, wheads, dim)
        for t0 in range(0, wtok, 16384):
            wcache.append(0, kfull[t0:t0 + 16384], kfull[t0:t0 + 16384], stream=stream)
        buf = tq.DecodeBuffer(wtok, wheads, dim)
        buf.rebuild(kfull, kfull, stream=stream)
        qw = torch.randn((wq, dim), device=device).half()
        ow = torch.empty_like(qw)
        us = timed(lambda: tq.hybrid_attention(wcache, buf, 0, qw, out=ow, stream=stream), reps=10)
        b = wtok * wheads * 4 * dim
        res["window_attention_1seq_ctx131072"] = {"us": us, "gb_per_s": b / (us * 1e-6) / 1e9, "frac_of_peak": b / (us * 1e-6) / 1e9 / peak}
        wcache.close()
        buf.close()
        del kfull
    except Exception as exc:
        res["window_attention_1seq_ctx131072"] = {"error": str(exc)}

    # Lloyd-Max fit of a 16-entry codebook to the 16.8 M rotated samples of a 4096 x 4096 layer
    try:
        samples = torch.randn((OUT_F * IN_F,), device=device)
        t0 = time.perf_counter()
        cb, it_run = tq.generate_codebook_from_data(samples, 4, 100, return_iterations=True)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        res["codebook_fit_16M_samples"] = {"ms": dt * 1e3, "iterations": it_run, "us_per_iteration": dt * 1e6 / max(it_run, 1),
                                           "gb_per_s_per_iteration": samples.numel() * 4 / (dt / max(it_run, 1)) / 1e9}
        del samples
    except Exception as exc:
        res["codebook_fit_16M_samples"] = {"error": str(exc)}
    return res


# ---- secondary: prefill through the tensor-core GEMM (2048 activation rows) -------------

def bench_prefill(tq, L, layers, device, stream, args):
    """2048 activation rows through 4096x4096 TQ8 layers (distinct layers back to back, as in the
    headline loop): fused dequantise + tcgen05 GEMM, activation rotation included."""
    import torch
    m = 2048
    n_layers = min(len(layers), 8)
    g = torch.Generator(device=device).manual_seed(900)
    x = torch.randn((m, IN_F), generator=g, device=device).half()
    y = torch.empty((m, OUT_F), device=device, dtype=torch.float16)
    sp = C.c_void_p(stream.cuda_stream)

    def call(lin):
        rc = L.tq_linear_forward(lin.handle, C.c_void_p(x.data_ptr()), tq.TQ_F16, m, C.c_void_p(y.data_ptr()), sp)
        if rc:
            raise RuntimeError(L.tq_last_error().decode())

    with torch.cuda.stream(stream):
        for lin in layers[:n_layers]:
            call(lin)
    torch.cuda.synchronize()
    reps = 5
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        e0.record(stream)
        for _ in range(reps):
            for lin in layers[:n_layers]:
                call(lin)
        e1.record(stream)
    torch.cuda.synchronize()
    if L.tq_linear_status(layers[0].handle):
        raise RuntimeError(L.tq_last_error().decode())
    us = e0.elapsed_time(e1) * 1e3 / (reps * n_layers)
    flops = 2.0 * m * OUT_F * IN_F
    peak = None
    pth = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(pth):
        peak = float(json.load(open(pth)).get("bf16_tflops", 0)) or None
    peak_kind = "measured cuBLAS bf16 burst" if peak else "fallback"
    peak = peak or 1590.0
    tf = flops / (us * 1e-6) / 1e12
    return {"workload": f"{m} activation rows x 4096x4096 TQ8 layer (rotation + fused dequant GEMM, fp16 in, fp32 accumulate)",
            "us_per_layer": us, "tok_per_s": m / (us * 1e-6), "tflops": tf, "frac_of_tensor_peak": tf / peak,
            "peak_tflops": peak, "peak_kind": peak_kind}


def bench_prefill_sharded(tq, L, device, stream, rank, world, cbs, args):
    """The prefill GEMM with the layer's output rows split over the ranks: every rank multiplies the same 2048
    activation rows by its 4096 / world weight rows straight into its column block of a shared [2048, 4096]
    result (strided output), copies that block to every peer with 16-byte stores (one row piece per activation
    row) and waits for the peers' blocks.  Beside it: the same shard followed by an NCCL all-gather."""
    import torch
    import torch.distributed as dist
    from turboquant_mlx_core_b200.sharding import Exchange, all_gather_rows, row_range
    m = 2048
    s, e = row_range(OUT_F, rank, world)
    rows = e - s
    n_layers = 4
    lins = [make_layer(tq, 7000 + 10 * li + rank, device, cbs, out_f=rows)[0] for li in range(n_layers)]
    g = torch.Generator(device=device).manual_seed(901)        # the same activations on every rank
    x = torch.randn((m, IN_F), generator=g, device=device).half()
    y = torch.empty((m, rows), device=device, dtype=torch.float16)
    sp = C.c_void_p(stream.cuda_stream)
    res = {"workload": f"{m} activation rows x 4096x4096 TQ8 layer, output rows split over {world} ranks "
                       f"({rows} per rank), result gathered on every rank"}
    exchange, setup_error = None, None
    try:
        exchange = Exchange(2 * m * OUT_F * 2)
    except Exception as exc:
        setup_error = str(exc)
    ok_t = torch.tensor([0.0 if setup_error else 1.0], device=device)
    dist.all_reduce(ok_t, op=dist.ReduceOp.MIN)
    if ok_t.item() != 1.0:
        if exchange is not None:
            exchange.close()
        exchange = None
        res["exchange"] = {"skipped": "shared buffers could not be mapped on every rank", "local_error": setup_error}

    def timed(fn, reps=5):
        torch.cuda.synchronize()
        dist.barrier()
        with torch.cuda.stream(stream):
            for lin in lins:
                fn(lin)
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record(stream)
            for _ in range(reps):
                for lin in lins:
                    fn(lin)
            e1.record(stream)
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) * 1e3 / (reps * n_layers)], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def nccl(lin):
        rc = L.tq_linear_forward(lin.handle, C.c_void_p(x.data_ptr()), tq.TQ_F16, m, C.c_void_p(y.data_ptr()), sp)
        if rc:
            raise RuntimeError(L.tq_last_error().decode())
        return all_gather_rows(y, OUT_F, world)

    flops = 2.0 * m * OUT_F * IN_F
    us = timed(nccl)
    res["nccl_all_gather"] = {"us_per_layer": us, "tflops_aggregate": flops / (us * 1e-6) / 1e12, "tok_per_s": m / (us * 1e-6)}
    if exchange is not None:
        step = [0]

        def ex(lin):
            half = step[0] & 1
            step[0] += 1
            base = half * m * OUT_F * 2
            lin.forward_strided(x, exchange.local + base + s * 2, OUT_F, stream=stream)
            exchange.broadcast(base + s * 2, m, rows * 2, OUT_F * 2, stream=stream)
            exchange.wait(stream=stream)

        us_x = timed(ex)
        exchange.check_status()
        # the last layer's gathered result against the all-gather of the same shard
        with torch.cuda.stream(stream):
            full = nccl(lins[(step[0] - 1) % n_layers])
        torch.cuda.synchronize()
        got = exchange.buf.tensor((2, m, OUT_F), torch.float16)[(step[0] - 1) & 1]
        same = torch.tensor([1.0 if torch.equal(full, got) else 0.0], device=device)
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        res["exchange"] = {"us_per_layer": us_x, "tflops_aggregate": flops / (us_x * 1e-6) / 1e12, "tok_per_s": m / (us_x * 1e-6),
                           "bytes_to_each_peer": m * rows * 2,
                           "path": "strided-output GEMM into the shared result + tq_exchange_broadcast + tq_exchange_wait",
                           "identical_to_all_gather_on_every_rank": bool(same.item() == 1.0)}
        exchange.close()
    for lin in lins:
        lin.close()
    return res


# ---- secondary: decoder-layer projections at decode batch sizes (Qwen2.5-7B shapes) ----------------

def bench_decoder_layer(tq, L, device, stream, cbs, args):
    """The seven projections of a Qwen2.5-7B-shaped decoder layer (hidden 3584, intermediate 18944,
    28 query / 4 KV heads of 128), TQ8, at batch 1, 8, 16 and 64: one pass = q, k, v, o, gate, up, down
    back to back (233 MB of codes per pass > L2).  Only the linears are timed (no attention, norms
    or activations).  `fused` is the same layer with q/k/v stored as one 4608-row matrix and gate/up as
    one 37888-row matrix (four launches; possible when the projections that share x are quantised with
    the same rotation seeds).  Also: the widest projection's result against a matmul over its
    dequantised weights, and 2048-row prefill on these shapes."""
    import torch
    hidden, inter, q_out, kv_out = 3584, 18944, 28 * 128, 4 * 128
    shapes = [("q", q_out, hidden), ("k", kv_out, hidden), ("v", kv_out, hidden), ("o", hidden, q_out),
              ("gate", inter, hidden), ("up", inter, hidden), ("down", hidden, inter)]
    fused_shapes = [("qkv", q_out + 2 * kv_out, hidden), ("o", hidden, q_out), ("gate_up", 2 * inter, hidden), ("down", hidden, inter)]
    code_bytes = sum(o * i for _, o, i in shapes)
    sp = C.c_void_p(stream.cuda_stream)
    g = torch.Generator(device=device).manual_seed(77)
    res = {"workload": "q/k/v/o/gate/up/down of a Qwen2.5-7B-shaped layer, TQ8, block 128", "code_bytes_per_pass": code_bytes}
    peak_tf = None
    pth = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(pth):
        peak_tf = float(json.load(open(pth)).get("bf16_tflops", 0)) or None
    peak_tf = peak_tf or 1590.0

    def time_pass(lins, xs, ys, batch, reps, groups=None):
        """groups: lists of layer indices that share their input and go out as one tq_linear_forward_group launch."""
        calls = []
        for grp in (groups or [[i] for i in range(len(lins))]):
            if len(grp) == 1:
                calls.append((lins[grp[0]].handle, xs[grp[0]], ys[grp[0]]))
            else:
                calls.append(((C.c_void_p * len(grp))(*[lins[i].handle for i in grp]), xs[grp[0]],
                              (C.c_void_p * len(grp))(*[ys[i].data_ptr() for i in grp]), len(grp)))

        def one_pass():
            for c in calls:
                if len(c) == 3:
                    rc = L.tq_linear_forward(c[0], C.c_void_p(c[1].data_ptr()), tq.TQ_F16, batch, C.c_void_p(c[2].data_ptr()), sp)
                else:
                    rc = L.tq_linear_forward_group(c[0], c[3], C.c_void_p(c[1].data_ptr()), batch, c[2], sp)
                if rc:
                    raise RuntimeError(L.tq_last_error().decode())
        torch.cuda.synchronize()
        with torch.cuda.stream(stream):
            for _ in range(3):
                one_pass()
        torch.cuda.synchronize()
        # one pass = 7 (or 4) library calls of two or three kernels each: replayed as a CUDA graph, as a decode
        # step would be, so that the figure is the kernels' and not the host's launch rate
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            one_pass()
        with torch.cuda.stream(stream):
            graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record(stream)
            for _ in range(reps):
                graph.replay()
            e1.record(stream)
        torch.cuda.synchronize()
        del graph
        return e0.elapsed_time(e1) * 1e3 / reps

    for tag, shp in (("", shapes), ("fused_", fused_shapes)):
        lins = [make_layer(tq, 7000 + i, device, cbs, out_f=out_f, in_f=in_f)[0] for i, (_, out_f, in_f) in enumerate(shp)]
        for batch in (1, 8, 16, 64):
            xs = [torch.randn((batch, in_f), generator=g, device=device).half() for _, _, in_f in shp]
            ys = [torch.empty((batch, out_f), device=device, dtype=torch.float16) for _, out_f, _ in shp]
            us = time_pass(lins, xs, ys, batch, 10)
            res[f"{tag}b{batch}"] = {"us_per_layer": us, "tok_per_s": batch / (us * 1e-6), "code_gb_per_s": code_bytes / (us * 1e-6) / 1e9,
                                     "launches_per_layer": len(shp) if batch <= 8 else None}
            if tag == "":
                # the same seven separately quantised matrices, q / k / v and gate / up each as ONE grouped launch
                grouped = [[0, 1, 2], [3], [4, 5], [6]]
                us = time_pass(lins, xs, ys, batch, 10, groups=grouped)
                same = True
                for gi in (0, 1, 2, 4, 5):
                    want = lins[gi].forward(xs[0] if gi < 3 else xs[4])
                    same = same and bool(torch.equal(want, ys[gi]))
                res[f"grouped_b{batch}"] = {"us_per_layer": us, "tok_per_s": batch / (us * 1e-6), "code_gb_per_s": code_bytes / (us * 1e-6) / 1e9,
                                            "launches_per_layer": len(grouped), "bit_equal_to_separate_calls": same}
        if tag == "":
            # the widest dot products of the layer (down_proj, K = 18944): result against fp32 matmul over
            # this library's own dequantised weights (which the parity tests hold bit-equal to the reference's)
            down = lins[-1]
            wd = torch.empty((hidden, inter), device=device, dtype=torch.float16)
            down.dequantize(out=wd)
            for batch in (1, 8, 64):
                xb = torch.randn((batch, inter), generator=g, device=device).half()
                yb = down.forward(xb)
                torch.cuda.synchronize()
                ref = xb.float() @ wd.float().t()
                res[f"down_proj_rel_l2_b{batch}"] = float((yb.float() - ref).norm() / ref.norm())
            del wd
            # 2048-row prefill on this layer's shapes (rotation + GEMM), one projection at a time
            pf = {}
            for (name, out_f, in_f), lin in zip(shp, lins):
                if name in ("k", "v", "up"):
                    continue
                xp = torch.randn((2048, in_f), generator=g, device=device).half()
                yp = torch.empty((2048, out_f), device=device, dtype=torch.float16)
                us = time_pass([lin], [xp], [yp], 2048, 5)
                tf = 2.0 * 2048 * out_f * in_f / (us * 1e-6) / 1e12
                pf[name] = {"shape": f"{out_f}x{in_f}", "us": us, "tflops": tf, "frac_of_tensor_peak": tf / peak_tf}
                del xp, yp
            res["prefill_2048_rows"] = pf
        for lin in lins:
            lin.close()
        del lins
        torch.cuda.empty_cache()
    return res


# ---- secondary: row-sharded LM head (151936 x 2048) -------------------------------------------

def bench_lm_head(tq, L, device, stream, rank, world, cbs, args):
    """Rows sharded over the ranks (whole 16-row tiles).  Two ways to give every rank the full logits:
    (a) forward into a private shard, then an NCCL all-gather (torch.distributed); (b) forward straight
    into this rank's rows of the shared logits buffer, then tq_exchange_broadcast of that block to
    every rank (16-byte peer stores, flag) and tq_exchange_wait - no collective library.  (b) is
    captured in a CUDA graph (two alternating logits buffers) and compared bit for bit with (a)."""
    import torch
    import torch.distributed as dist
    from turboquant_mlx_core_b200.sharding import Exchange, all_gather_rows, row_range
    vocab, hidden = 151936, 2048
    s, e = row_range(vocab, rank, world)
    rows = e - s
    g = torch.Generator(device=device).manual_seed(500 + rank)
    w = (torch.randn((rows, hidden), generator=g, device=device) * 0.02).half().float()
    qw = tq.quantize_weight(w, cbs[0], cbs[1], tq.QuantizerConfig(4, 4, BLOCK, True))
    del w
    lin = tq.TurboQuantLinear(hidden, rows, qw, cbs[0], cbs[1], BLOCK)
    res = {"workload": f"LM head {vocab}x{hidden}, rows sharded over {world} GPU(s)"}
    sp = C.c_void_p(stream.cuda_stream)
    reps = 20

    def timed(fn, graph=False):
        """(device us per call, host us per call when issued eagerly)"""
        if world > 1:                      # exchanging kernels wait a second at most: start together
            torch.cuda.synchronize()
            dist.barrier()
        with torch.cuda.stream(stream):
            for _ in range(3):
                fn()
        torch.cuda.synchronize()
        run, per = fn, 1
        if graph:
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr, stream=stream):
                fn()
                fn()                      # both gather buffers
            run, per = gr.replay, 2
            with torch.cuda.stream(stream):
                run()
            torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        with torch.cuda.stream(stream):
            e0.record(stream)
            for _ in range(reps):
                run()
            e1.record(stream)
        host_us = (time.perf_counter() - t0) * 1e6 / (reps * per)
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) * 1e3 / (reps * per)], device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()), host_us

    exchange, setup_error = None, None
    lm_packets_off = 2 * 32 * vocab * 2        # packet area behind the two logits buffers: [2][world][8 * rows / 4] x 16 bytes
    if world > 1:
        try:
            exchange = Exchange(lm_packets_off + 2 * world * 8 * (rows // 4 + 1) * 16)
        except Exception as exc:
            setup_error = str(exc)
        ok_t = torch.tensor([0.0 if setup_error else 1.0], device=device)
        dist.all_reduce(ok_t, op=dist.ReduceOp.MIN)
        if ok_t.item() != 1.0:
            if exchange is not None:
                exchange.close()
            exchange = None
            res["exchange"] = {"skipped": "shared buffers could not be mapped on every rank", "local_error": setup_error}

    for batch in (1, 32):
        x = torch.randn((batch, hidden), generator=g, device=device).half()
        y = torch.empty((batch, rows), device=device, dtype=torch.float16)
        algo = vocab * hidden + 4 * vocab + 2 * batch * hidden + 2 * batch * vocab

        def call():
            rc = L.tq_linear_forward(lin.handle, C.c_void_p(x.data_ptr()), tq.TQ_F16, batch, C.c_void_p(y.data_ptr()), sp)
            if rc:
                raise RuntimeError(L.tq_last_error().decode())
            if world > 1:
                return all_gather_rows(y, vocab, world)
            return y

        us, host_us = timed(call, graph=(world == 1))
        key = f"b{batch}"
        res[key] = {"us": us, "tok_per_s": batch / (us * 1e-6), "gb_per_s_aggregate": algo / (us * 1e-6) / 1e9,
                    "host_us_per_call_eager": host_us,
                    "path": "forward" + (" + NCCL all-gather of the fp16 shards (eager launches)" if world > 1 else " (CUDA graph)")}
        if exchange is None:
            continue
        try:
            step = [0]

            def call_exchange():
                half = step[0] & 1
                step[0] += 1
                base = half * batch * vocab * 2                    # byte offset of this buffer's [batch, vocab] logits
                # rows [s, e) of every activation row, at the vocabulary's stride
                lin.forward_strided(x, exchange.local + base + s * 2, vocab, stream=stream)
                exchange.broadcast(base + s * 2, batch, rows * 2, vocab * 2, stream=stream)
                exchange.wait(stream=stream)

            us_f = None
            if batch <= 8:
                with torch.cuda.stream(stream):
                    exchange.broadcast(0, 1, 16, 16, stream=stream)      # something for the first fused call to wait for
                fstep = [0]

                def call_fused():
                    half = fstep[0] & 1
                    fstep[0] += 1
                    exchange.forward_allgather(lin, x, vocab, s, buffer_offset=half * batch * vocab * 2, wait=True, stream=stream)

                us_f, host_f = timed(call_fused, graph=True)
                with torch.cuda.stream(stream):
                    exchange.wait(stream=stream)
                torch.cuda.synchronize()
                exchange.check_status()
                lin.check_status()
                fused_logits = exchange.buf.tensor((2, batch, vocab), torch.float16).clone()
            us_p = None
            if batch <= 8 and rows % 4 == 0 and (vocab // world) == rows:
                pstep = [0]

                def call_packets():
                    half = pstep[0] & 1
                    pstep[0] += 1
                    base = exchange.local + half * batch * vocab * 2
                    # this rank's rows go straight to their place in the logits; every CTA sends its own rows to the other
                    # ranks as {data, epoch} packets while the rest of the grid is still computing; a second kernel waits
                    # for the other ranks' packets and writes their rows beside them
                    exchange.forward_allgather_packets(lin, x, None, lm_packets_off, wait=False, stream=stream, y_ptr=base + s * 2,
                                                       y_row_stride=vocab)
                    exchange.wait_packets(lm_packets_off, rows, batch, base, vocab, stream=stream)

                us_p, host_p = timed(call_packets, graph=True)
                exchange.check_status()
                lin.check_status()
                packet_logits = exchange.buf.tensor((2, batch, vocab), torch.float16).clone()
            us_x, host_x = timed(call_exchange, graph=True)
            exchange.check_status()
            with torch.cuda.stream(stream):
                full = call()
            torch.cuda.synchronize()
            logits = exchange.buf.tensor((2, batch, vocab), torch.float16)
            same = bool(torch.equal(full, logits[0])) and bool(torch.equal(full, logits[1]))
            same_t = torch.tensor([1.0 if same else 0.0], device=device)
            dist.all_reduce(same_t, op=dist.ReduceOp.MIN)
            if us_f is not None:
                same_f = bool(torch.equal(full, fused_logits[0])) and bool(torch.equal(full, fused_logits[1]))
                sf = torch.tensor([1.0 if same_f else 0.0], device=device)
                dist.all_reduce(sf, op=dist.ReduceOp.MIN)
                res[key + "_fused"] = {"us": us_f, "tok_per_s": batch / (us_f * 1e-6), "gb_per_s_aggregate": algo / (us_f * 1e-6) / 1e9,
                                       "host_us_per_call_eager": host_f,
                                       "path": "tq_linear_forward_allgather: one kernel waits for the previous gather, computes the "
                                               "shard, copies it to the peers and raises the flags (CUDA graph)",
                                       "identical_to_all_gather_on_every_rank": bool(sf.item() == 1.0)}
            if us_p is not None:
                same_p = bool(torch.equal(full, packet_logits[0])) and bool(torch.equal(full, packet_logits[1]))
                spk = torch.tensor([1.0 if same_p else 0.0], device=device)
                dist.all_reduce(spk, op=dist.ReduceOp.MIN)
                res[key + "_packets"] = {"us": us_p, "tok_per_s": batch / (us_p * 1e-6), "gb_per_s_aggregate": algo / (us_p * 1e-6) / 1e9,
                                         "host_us_per_call_eager": host_p,
                                         "path": "tq_linear_forward_allgather_packets (every CTA sends its own rows as {data, epoch} packets) "
                                                 "+ tq_exchange_wait_packets (CUDA graph)",
                                         "identical_to_all_gather_on_every_rank": bool(spk.item() == 1.0)}
            res[key + "_exchange"] = {"us": us_x, "tok_per_s": batch / (us_x * 1e-6), "gb_per_s_aggregate": algo / (us_x * 1e-6) / 1e9,
                                      "host_us_per_call_eager": host_x,
                                      "path": "forward into the shared logits + tq_exchange_broadcast + tq_exchange_wait (CUDA graph)",
                                      "identical_to_all_gather_on_every_rank": bool(same_t.item() == 1.0)}
        except Exception as exc:
            res[key + "_exchange"] = {"error": str(exc)}
    if exchange is not None:
        exchange.close()
    lin.close()
    return res


# ---- secondary: tensor-parallel decode step of a Qwen2.5-32B-shaped layer -------------------------------

def bench_c4_decode_step(tq, L, device, stream, rank, world, cbs, args):
    """One decoder layer per step, Qwen2.5-32B shapes (hidden 5120, intermediate 27648, 40 query / 8 KV
    heads of 128, context 8192), tensor-parallel over the ranks as the sharded paths prescribe:
    q / k / v / gate-up split by output rows (no exchange), o_proj and down_proj split by input columns
    on WHT-block boundaries, their partial outputs exchanged by peer stores and added in rank order
    (tq_exchange_broadcast / _wait / _sum_f16: the all-reduce), KV heads split for the compressed cache
    and the decode attention; RMSNorm, rotary embedding, SwiGLU and the residual adds run as this
    library's small kernels.  TQ8 (4+4 bit, block 128) weights with random codes for every layer (the
    model's first and last four layers would stay fp16), one token appended per sequence per step.  The
    whole step is one CUDA graph; enough distinct layers are cycled that the weights come from HBM.
    Also checks a small row-parallel linear against the unsharded layer (1e-3) and across ranks (bits)."""
    import torch
    import torch.distributed as dist
    from turboquant_mlx_core_b200.sharding import Exchange, col_range, shard_quantized_cols
    hidden, inter, q_heads, kv_heads, dim, ctx, n_model_layers = 5120, 27648, 40, 8, 128, 8192, 64
    if kv_heads % world:
        return {"skipped": f"{world} ranks do not divide {kv_heads} KV heads"}
    qh, kvh, il = q_heads // world, kv_heads // world, inter // world
    sp = C.c_void_p(stream.cuda_stream)
    res = {"workload": f"Qwen2.5-32B-shaped decoder layer, TQ8, tensor-parallel over {world} GPU(s), context {ctx}, 3.5-bit KV cache"}
    cp, cr = cbs[0].centroids.astype(np.float32), cbs[1].centroids.astype(np.float32)
    g = torch.Generator(device=device).manual_seed(900 + rank)
    handles = []

    def rand_linear(rows, cols, seed):
        pp = torch.randint(0, 256, (rows, cols // 2), generator=g, device=device, dtype=torch.uint8)
        pr = torch.randint(0, 256, (rows, cols // 2), generator=g, device=device, dtype=torch.uint8)
        norms = torch.ones(rows, device=device, dtype=torch.float32)
        seeds = np.array([seed, 0, BLOCK], np.uint32)
        h = L.tq_linear_create(cols, rows, C.c_void_p(pp.data_ptr()), cols // 2, C.c_void_p(pr.data_ptr()), C.c_void_p(norms.data_ptr()),
                               seeds.ctypes.data, cp.ctypes.data, cp.size, cr.ctypes.data, cr.size, BLOCK)
        if not h:
            raise RuntimeError(L.tq_last_error().decode())
        handles.append(h)
        return h

    def fwd(h, x, batch, y):
        if L.tq_linear_forward(h, C.c_void_p(x), tq.TQ_F16, batch, C.c_void_p(y), sp):
            raise RuntimeError(L.tq_last_error().decode())

    def chk(rc):
        if rc:
            raise RuntimeError(L.tq_last_error().decode())

    bytes_per_layer = ((qh + 2 * kvh) * dim * hidden + hidden * qh * dim + 2 * il * hidden + hidden * il)
    n_layers = max(2, -(-300_000_000 // bytes_per_layer))
    layers = []
    for li in range(n_layers):
        layers.append({"q": rand_linear(qh * dim, hidden, 10 * li + 1), "k": rand_linear(kvh * dim, hidden, 10 * li + 2),
                       "v": rand_linear(kvh * dim, hidden, 10 * li + 3), "o": rand_linear(hidden, qh * dim, 10 * li + 4),
                       "gu": rand_linear(2 * il, hidden, 10 * li + 5), "down": rand_linear(hidden, il, 10 * li + 6),
                       "n1": torch.ones(hidden, device=device, dtype=torch.float16),
                       "n2": torch.ones(hidden, device=device, dtype=torch.float16)})

    exchange = None
    if world > 1:
        err = None
        try:
            # two all-reduce buffers of [world][32 rows][hidden] fp16, then the packet area for batches up to 8:
            # [2 epoch parities][world][8 * hidden / 4 packets of 16 bytes]
            exchange = Exchange(2 * world * 32 * hidden * 2 + 2 * world * 8 * (hidden // 4) * 16)
        except Exception as exc:
            err = str(exc)
        ok_t = torch.tensor([0.0 if err else 1.0], device=device)
        dist.all_reduce(ok_t, op=dist.ReduceOp.MIN)
        if ok_t.item() != 1.0:
            if exchange is not None:
                exchange.close()
            for h in handles:
                L.tq_linear_free(h)
            return {"skipped": "shared buffers could not be mapped on every rank", "local_error": err}

    for batch in (1, 32):
        caches = [tq.TQKVCache(n_layers, kvh, dim) for _ in range(batch)]
        for c in caches:
            for li in range(n_layers):
                c.reserve(li, ctx + 16)
                kk = torch.randn((ctx, kvh, dim), generator=g, device=device).half()
                c.append(li, kk, kk)
        arr = (C.c_void_p * batch)(*[c.handle for c in caches])
        gx = torch.Generator(device=device).manual_seed(77 + batch)       # the residual stream is replicated: same on every rank
        x = torch.randn((batch, hidden), generator=gx, device=device).half() * 0.1
        x0 = x.clone()
        h1 = torch.empty_like(x)
        q = torch.empty((batch, qh, dim), device=device, dtype=torch.float16)
        k = torch.empty((batch, kvh, dim), device=device, dtype=torch.float16)
        v = torch.empty_like(k)
        attn = torch.empty_like(q)
        part = torch.empty((batch, hidden), device=device, dtype=torch.float16)   # world == 1: the "exchange" is local
        x1 = torch.empty_like(x)
        gu = torch.empty((batch, 2 * il), device=device, dtype=torch.float16)
        act = torch.empty((batch, il), device=device, dtype=torch.float16)
        pos = torch.full((batch,), ctx, device=device, dtype=torch.int32)
        count = batch * hidden
        toggle = [0]

        c4_packets_off = 2 * world * 32 * hidden * 2
        use_packets = exchange is not None and batch <= 8 and os.environ.get("TQ_BENCH_ALLREDUCE", "packets") == "packets"
        if use_packets:
            pk_bufs = (C.c_void_p * world)(*[p + c4_packets_off for p in exchange.rank_ptrs()])

        def all_reduce_add_packets(h, xin_ptr, residual, out, norm_w=None):
            """The column-sharded linear h writes its partial locally and sends it as packets from inside its kernel; one more
            kernel waits for the other ranks' packets and adds everything in rank order - and, with norm_w, writes the
            RMSNorm of the summed rows to h1 as well (the next projection's input)."""
            chk(L.tq_linear_forward_allgather_packets(h, exchange._h, C.c_void_p(xin_ptr), batch, C.c_void_p(part.data_ptr()), hidden,
                                                      pk_bufs, 0, sp))
            if norm_w is None:
                chk(L.tq_exchange_sum_packets(exchange._h, C.c_void_p(exchange.local + c4_packets_off), C.c_void_p(part.data_ptr()), count,
                                              C.c_void_p(residual.data_ptr()), C.c_void_p(out.data_ptr()), sp))
            else:
                chk(L.tq_exchange_sum_packets_rmsnorm(exchange._h, C.c_void_p(exchange.local + c4_packets_off), C.c_void_p(part.data_ptr()),
                                                      batch, hidden, C.c_void_p(residual.data_ptr()), C.c_void_p(out.data_ptr()),
                                                      C.c_void_p(norm_w.data_ptr()), C.c_void_p(h1.data_ptr()), 1e-6, sp))

        def all_reduce_add(partial_of, residual, out, norm_w=None):
            """partial_of(ptr) writes this rank's partial [batch, hidden] at ptr; out = residual + sum over ranks; with norm_w
            the summing kernel also writes the RMSNorm of the summed rows to h1."""
            if exchange is None:
                partial_of(part.data_ptr())
                slots_ptr, n_slots = part.data_ptr(), 1
            else:
                base = (toggle[0] & 1) * world * count * 2
                toggle[0] += 1
                partial_of(exchange.local + base + rank * count * 2)
                exchange.broadcast(base + rank * count * 2, 1, count * 2, count * 2, stream=stream)
                exchange.wait(stream=stream)
                slots_ptr, n_slots = exchange.local + base, world
            if norm_w is None:
                chk(L.tq_exchange_sum_f16(C.c_void_p(slots_ptr), n_slots, count, count, C.c_void_p(residual.data_ptr()),
                                          C.c_void_p(out.data_ptr()), sp))
            else:
                chk(L.tq_exchange_sum_f16_rmsnorm(C.c_void_p(slots_ptr), n_slots, count, batch, hidden, C.c_void_p(residual.data_ptr()),
                                                  C.c_void_p(out.data_ptr()), C.c_void_p(norm_w.data_ptr()), C.c_void_p(h1.data_ptr()),
                                                  1e-6, sp))

        marks = None                       # set to a list: layer_step then records an event after every group of kernels

        def mark(name):
            if marks is not None:
                e = torch.cuda.Event(enable_timing=True)
                e.record(stream)
                marks.append((name, e))

        def layer_step(li):
            w = layers[li]
            mark("start")
            if li == 0:      # later layers' input norm comes out of the previous layer's last all-reduce kernel
                chk(L.tq_rmsnorm_f16(C.c_void_p(x.data_ptr()), C.c_void_p(w["n1"].data_ptr()), C.c_void_p(h1.data_ptr()), batch, hidden, 1e-6, sp))
            mark("rmsnorm_1")
            # q, k and v read the same activation: one grouped launch per kernel of the path (bit-equal to the three calls)
            chk(L.tq_linear_forward_group((C.c_void_p * 3)(w["q"], w["k"], w["v"]), 3, C.c_void_p(h1.data_ptr()), batch,
                                          (C.c_void_p * 3)(q.data_ptr(), k.data_ptr(), v.data_ptr()), sp))
            mark("q_k_v")
            chk(L.tq_rope_qk_f16(C.c_void_p(q.data_ptr()), C.c_void_p(k.data_ptr()), C.c_void_p(pos.data_ptr()), batch, qh, kvh, dim, 1e6, sp))
            mark("rope_q_k")
            chk(L.tq_kv_append_batch(arr, batch, li, C.c_void_p(k.data_ptr()), C.c_void_p(v.data_ptr()), tq.TQ_F16, sp))
            mark("kv_append")
            chk(L.tq_kv_attention(arr, batch, li, C.c_void_p(q.data_ptr()), tq.TQ_F16, qh, C.c_void_p(attn.data_ptr()), 0, ctx, 1, sp))
            mark("attention")
            if use_packets:
                all_reduce_add_packets(w["o"], attn.data_ptr(), x, x1, norm_w=w["n2"])
            else:
                all_reduce_add(lambda ptr: fwd(w["o"], attn.data_ptr(), batch, ptr), x, x1, norm_w=w["n2"])
            mark("o_proj_sum_residual_rmsnorm")
            fwd(w["gu"], h1.data_ptr(), batch, gu.data_ptr())
            mark("gate_up")
            chk(L.tq_swiglu_f16(C.c_void_p(gu.data_ptr()), C.c_void_p(act.data_ptr()), batch, il, sp))
            mark("swiglu")
            nxt = layers[li + 1]["n1"] if li + 1 < n_layers else None
            if use_packets:
                all_reduce_add_packets(w["down"], act.data_ptr(), x1, x, norm_w=nxt)
            else:
                all_reduce_add(lambda ptr: fwd(w["down"], act.data_ptr(), batch, ptr), x1, x, norm_w=nxt)
            mark("down_proj_sum_residual_rmsnorm")

        def one_pass():
            for li in range(n_layers):
                layer_step(li)

        torch.cuda.synchronize()           # the inputs were made on the default stream
        if world > 1:
            dist.barrier()                 # exchanging kernels wait a second at most: start together
        with torch.cuda.stream(stream):
            one_pass()                     # allocates scratch, uploads attention descriptors per layer
            x.copy_(x0)
            one_pass()
        torch.cuda.synchronize()
        # the cache grew by two tokens per layer during the eager passes; the captured step re-appends
        # at a fixed position and attends to [0, ctx), so its descriptors repeat the eager call's
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            x.copy_(x0)
        with torch.cuda.graph(graph, stream=stream):
            one_pass()
        with torch.cuda.stream(stream):
            for _ in range(2):
                graph.replay()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        reps = 5
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record(stream)
            for _ in range(reps):
                graph.replay()
            e1.record(stream)
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) * 1e3 / (reps * n_layers)], device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        us = float(t.item())
        # the residual stream must be finite and identical on every rank (fixed-order sums)
        finite = bool(torch.isfinite(x.float()).all())
        same = True
        if world > 1:
            ref = x.clone()
            dist.broadcast(ref, src=0)
            ok = torch.tensor([1.0 if torch.equal(ref, x) else 0.0], device=device)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            same = bool(ok.item() == 1.0)
            exchange.check_status()
        # where the step's time goes: one eager pass with an event after every group of kernels (median over the
        # layers; eager launches, so each group also carries its launch gaps - the graph figure above is the step)
        breakdown = None
        if True:                           # every rank runs the passes (the exchanges need all of them); rank 0 reports
            marks = []
            if world > 1:
                dist.barrier()
            with torch.cuda.stream(stream):
                for _ in range(3):
                    one_pass()
            torch.cuda.synchronize()
            groups = {}
            for (n0, ev0), (n1, ev1) in zip(marks, marks[1:]):
                if n1 != "start":
                    groups.setdefault(n1, []).append(ev0.elapsed_time(ev1) * 1e3)
            breakdown = {n: round(float(np.median(v)), 2) for n, v in groups.items()}
            marks = None
        weight_bytes = bytes_per_layer
        kv_bytes = batch * kvh * ctx * 118
        res[f"b{batch}"] = {"us_per_layer": us, "tok_per_s_64_layers": batch / (us * 1e-6 * n_model_layers),
                            "gb_per_s_per_gpu": (weight_bytes + kv_bytes) / (us * 1e-6) / 1e9,
                            "bytes_per_layer_per_gpu": weight_bytes + kv_bytes, "distinct_layers_cycled": n_layers,
                            "kernels_per_layer": "q + k + v (one grouped launch), rope of q and k, kv append x2, attention, o_proj, "
                                                 "[copy to peers, wait,] sum + residual + rmsnorm, gate-up, swiglu, down, [copy to peers, wait,] "
                                                 "sum + residual + the next layer's rmsnorm",
                            "all_reduce": ("none (one rank)" if exchange is None else
                                           "partials sent as packets from inside o_proj / down_proj, one kernel waits and adds" if use_packets
                                           else "tq_exchange_broadcast + tq_exchange_wait + tq_exchange_sum_f16"),
                            "residual_stream_finite": finite, "identical_on_every_rank": same}
        if breakdown is not None:
            res[f"b{batch}"]["eager_us_by_kernel_group"] = breakdown
        for c in caches:
            c.close()

    # ---- row-parallel linear against the unsharded layer (small, real quantised weights) ----
    try:
        rows, cols, batch = 512, 2048, 3
        gq = torch.Generator(device=device).manual_seed(4242)            # the same on every rank
        wfull = (torch.randn((rows, cols), generator=gq, device=device) * 0.02).half().float()
        cbc = tq.generate_codebook(4)       # analytic: the same on every rank (the fitted ones come from rank-seeded weights)
        qwf = tq.quantize_weight(wfull, cbc, cbc, tq.QuantizerConfig(4, 4, BLOCK, True))
        full = tq.TurboQuantLinear(cols, rows, qwf, cbc, cbc, BLOCK)
        xs = torch.randn((batch, cols), generator=gq, device=device).half()
        want = full.forward(xs)
        pp, pr, nrm, (c0, c1) = shard_quantized_cols(qwf.packed_primary, qwf.packed_residual, qwf.norms, cols, BLOCK, rank, world)
        shard = tq.TurboQuantLinear(c1 - c0, rows, tq.QuantizedWeight(np.ascontiguousarray(pp), np.ascontiguousarray(pr), nrm, qwf.seeds),
                                    cbc, cbc, BLOCK)
        xl = xs[:, c0:c1].contiguous()
        got = torch.empty((batch, rows), device=device, dtype=torch.float16)
        cnt = batch * rows
        torch.cuda.synchronize()           # the inputs were made on the default stream
        if world > 1:
            dist.barrier()
        with torch.cuda.stream(stream):
            if exchange is None:
                tmp = shard.forward(xl, stream=stream)
                chk(L.tq_exchange_sum_f16(C.c_void_p(tmp.data_ptr()), 1, cnt, cnt, None, C.c_void_p(got.data_ptr()), sp))
            else:
                base = (toggle[0] & 1) * world * 32 * hidden * 2
                toggle[0] += 1
                off = base + rank * cnt * 2
                fwd(shard.handle, xl.data_ptr(), batch, exchange.local + off)
                exchange.broadcast(off, 1, cnt * 2, cnt * 2, stream=stream)
                exchange.wait(stream=stream)
                exchange.sum_f16(base, world, cnt, cnt, got.data_ptr(), stream=stream)
        torch.cuda.synchronize()
        rel = float((got.float() - want.float()).norm() / want.float().norm())
        same = True
        if world > 1:
            ref = got.clone()
            dist.broadcast(ref, src=0)
            ok = torch.tensor([1.0 if torch.equal(ref, got) else 0.0], device=device)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            same = bool(ok.item() == 1.0)
        res["row_parallel_check"] = {"shape": f"{rows}x{cols}, batch {batch}, columns split over {world} rank(s) on WHT-block boundaries",
                                     "rel_l2_vs_unsharded_layer": rel, "within_1e-3": rel < 1e-3, "identical_on_every_rank": same}
        full.close()
        shard.close()
    except Exception as exc:
        res["row_parallel_check"] = {"error": str(exc)}
    if exchange is not None:
        exchange.close()
    for h in handles:
        L.tq_linear_free(h)
    return res


# ---- CPU legs ---------------------------------------------------------------------------------------

def cpu_threads():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_linear_once(ref, ora, qw, cbs, x, threads):
    """The reference's CPU linear: dequantize_weight_cpu, then an fp32 matmul over the
    fp16-rounded activation (src/dequantizer.cpp:52-256, tests/integration/test_linear.cpp:98-107)."""
    cp, cr = cbs[0].centroids, cbs[1].centroids
    if ref is not None:
        w = ref.dequantize_weight_mt(qw.packed_primary, qw.packed_residual, qw.norms, qw.seeds, cp, cr, BLOCK, threads)
    else:
        w = ora.dequantize_weight(qw.packed_primary, qw.packed_residual, qw.norms, qw.seeds, cp, cr, BLOCK)
    xh = x.astype(np.float16).astype(np.float32)
    return xh @ w.T


def load_cpu_libs():
    from oracle import build as obuild
    from oracle.pyoracle import Oracle, Ref, have_ref
    obuild.build_oracle()
    ora = Oracle()
    ref = Ref() if have_ref() else None
    return ref, ora


def cpu_baseline(qw, cbs, x, y_gpu, budget_s):
    ref, ora = load_cpu_libs()
    threads = cpu_threads() if ref is not None else 1
    t0 = time.perf_counter()
    y = cpu_linear_once(ref, ora, qw, cbs, x[None], threads)
    first = time.perf_counter() - t0
    n = max(1, min(20, int(budget_s / max(first, 1e-3)) - 1))
    times = [first]
    for _ in range(n):
        t0 = time.perf_counter()
        cpu_linear_once(ref, ora, qw, cbs, x[None], threads)
        times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    rel = float(np.linalg.norm(y_gpu.astype(np.float64) - y[0]) / np.linalg.norm(y[0]))
    return {"value": 1.0 / med, "unit": "tok/s", "cores": threads, "kind": "reference" if ref is not None else "port",
            "sample": f"{len(times)} forwards of one 4096x4096 layer (dequantize_weight_cpu + fp32 GEMV), median",
            "gpu_vs_cpu_rel_l2": rel}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    ref, ora = load_cpu_libs()
    threads = cpu_threads() if ref is not None else 1
    rng = np.random.default_rng(0)
    w = (rng.standard_normal((OUT_F, IN_F)) * 0.02).astype(np.float16).astype(np.float32)
    cb4 = ora.codebook(4)[0]
    src = ref if ref is not None else ora
    pp, pr, norms, seeds = src.quantize_weight(w, cb4, cb4, 4, 4, BLOCK, True)

    class QW:
        pass
    qw = QW()
    qw.packed_primary, qw.packed_residual, qw.norms, qw.seeds = pp, pr, norms, seeds

    class CB:
        def __init__(self, c):
            self.centroids = c
    cbs = (CB(cb4), CB(cb4))
    x = rng.standard_normal((1, IN_F)).astype(np.float16).astype(np.float32)
    for _ in range(args.warmup):
        cpu_linear_once(ref, ora, qw, cbs, x, threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_linear_once(ref, ora, qw, cbs, x, threads)
    dt = time.perf_counter() - t0
    value = args.steps / dt
    kind = "reference" if ref is not None else "port"
    print(json.dumps({
        "impl": "reference", "metric": "tq8_dequant_gemv_4096x4096_b1_tok_per_s", "value": value, "unit": "tok/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
        "config": {"workload": "TQ8 4+4-bit linear, 4096x4096, block 128, shared rotation, batch 1; "
                               "each step = one layer forward on the host cores"},
        "cpu_baseline": {"value": value, "unit": "tok/s", "cores": threads, "kind": kind,
                         "sample": "one 4096x4096 layer forward per step: the reference's dequantize_weight_cpu "
                                   "(row-sliced over all host threads) + fp32 GEMV"},
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", default="cuda", choices=["cuda", "reference"])
    ap.add_argument("--nbuf", type=int, default=64, help="distinct 4096x4096 layers per step")
    ap.add_argument("--attn-ctx", type=int, default=32768)
    ap.add_argument("--attn-kv-heads", type=int, default=4, help="KV heads of the attention leg (7 query heads each)")
    ap.add_argument("--no-extras", action="store_true", help="skip the secondary measurements")
    ap.add_argument("--legs", default="", help="comma list of secondary measurements to run "
                                               "(attention, decoder_layer, prefill, lm_head, side_kernels); default all")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="time plain stream launches instead of a CUDA graph")
    a = ap.parse_args()
    if a.impl == "reference":
        a.steps = a.steps if a.steps is not None else 5
        a.warmup = a.warmup if a.warmup is not None else 1
        run_reference(a)
    else:
        a.steps = a.steps if a.steps is not None else 2000
        a.warmup = max(3, a.warmup if a.warmup is not None else 50)
        run_cuda(a)


if __name__ == "__main__":
    main()
