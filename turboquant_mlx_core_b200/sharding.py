"""Host-side partition rules for the multi-GPU paths (one process per GPU).

Column-parallel linears (LM head, q/k/v/gate/up) shard by OUTPUT ROWS: every row has its
own codes and norm, while codebooks, seeds and the activation are replicated, so a rank
builds an ordinary TurboQuantLinear over its row range and the only exchange is an
all-gather of the fp16 outputs.  Attention shards by KV HEADS (heads are independent);
query heads follow their KV head.  Nothing here touches device memory.
"""
from __future__ import annotations


def row_range(out_features: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous row range of `rank`, in whole 16-row tiles (the GEMV kernel's tile) except
    at the tail, as even as possible."""
    tiles = (out_features + 15) // 16
    t0 = tiles * rank // world
    t1 = tiles * (rank + 1) // world
    return min(t0 * 16, out_features), min(t1 * 16, out_features)


def head_range(kv_heads: int, rank: int, world: int) -> tuple[int, int]:
    if world > kv_heads or kv_heads % world:
        raise ValueError("KV heads must divide evenly over the ranks; split the context range for extra ranks")
    per = kv_heads // world
    return rank * per, (rank + 1) * per


def shard_quantized_rows(packed_primary, packed_residual, norms, rank: int, world: int):
    """Row slice of a QuantizedWeight's planes and norms for `rank`."""
    s, e = row_range(packed_primary.shape[0], rank, world)
    return packed_primary[s:e], packed_residual[s:e], norms[s:e]


def all_gather_rows(local, out_features: int, world: int):
    """All-gather [batch, rows_of_rank] shards into [batch, out_features] (torch.distributed).
    Shards may differ in width by one tile, so each is padded to the widest before the
    collective and trimmed after."""
    import torch
    import torch.distributed as dist
    spans = [row_range(out_features, r, world) for r in range(world)]
    width = max(e - s for s, e in spans)
    batch = local.shape[0]
    if all(e - s == width for s, e in spans):
        # equal shards need no padding: one collective straight into the result (one activation
        # row), or into [world, batch, width] followed by a single permuting copy
        out = torch.empty((batch, out_features), dtype=local.dtype, device=local.device)
        if batch == 1:
            dist.all_gather_into_tensor(out.view(world, width), local.contiguous().view(1, width))
            return out
        flat = torch.empty((world, batch, width), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(flat.view(world * batch, width), local.contiguous())
        out.view(batch, world, width).copy_(flat.permute(1, 0, 2))
        return out
    padded = torch.zeros((batch, width), dtype=local.dtype, device=local.device)
    padded[:, : local.shape[1]] = local
    flat = torch.empty((world * batch, width), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(flat, padded)
    gathered = flat.view(world, batch, width)
    out = torch.empty((batch, out_features), dtype=local.dtype, device=local.device)
    for r, (s, e) in enumerate(spans):
        out[:, s:e] = gathered[r, :, : e - s]
    return out


def attention_grid(kv_heads: int, rank: int, world: int) -> tuple[int, int, int, int]:
    """Placement of `rank` for decode attention: (first KV head, one-past-last KV head, context
    part, number of context parts).  Up to kv_heads ranks split the heads; beyond that each head
    is shared by world / kv_heads ranks which split the context range in equal parts and merge
    their partial results (merge_attention_parts)."""
    if world <= kv_heads:
        s, e = head_range(kv_heads, rank, world)
        return s, e, 0, 1
    if world % kv_heads:
        raise ValueError("more ranks than KV heads: the rank count must be a multiple of the KV heads")
    parts = world // kv_heads
    head = rank % kv_heads
    return head, head + 1, rank // kv_heads, parts


def context_range(start: int, end: int, part: int, parts: int) -> tuple[int, int]:
    """Token range of context part `part` of [start, end)."""
    n = end - start
    return start + n * part // parts, start + n * (part + 1) // parts


def merge_attention_parts(outs, lses):
    """Merge attention results computed over disjoint token ranges of the same sequences.
    outs: [parts, ..., head_dim], lses: [parts, ...] (log of each part's softmax denominator).
    Returns the attention over the union, fp32.  Works on numpy arrays and torch tensors."""
    if hasattr(outs, "detach"):
        import torch
        m = lses.max(dim=0, keepdim=True).values
        m = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
        w = torch.exp(lses - m)
        den = w.sum(dim=0)
        num = (outs.float() * w.unsqueeze(-1)).sum(dim=0)
        return num / den.clamp_min(1e-38).unsqueeze(-1)
    import numpy as np
    outs = np.asarray(outs, np.float32)
    lses = np.asarray(lses, np.float32)
    m = lses.max(axis=0, keepdims=True)
    m = np.where(np.isfinite(m), m, 0.0)
    w = np.exp(lses - m)
    den = w.sum(axis=0)
    num = (outs * w[..., None]).sum(axis=0)
    return num / np.maximum(den, 1e-38)[..., None]


def all_gather_attention_parts(out_local, lse_local, group=None):
    """All-gather (out, lse) over the ranks that share a KV head and merge them."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    outs = torch.empty((world,) + tuple(out_local.shape), dtype=out_local.dtype, device=out_local.device)
    lses = torch.empty((world,) + tuple(lse_local.shape), dtype=lse_local.dtype, device=lse_local.device)
    dist.all_gather_into_tensor(outs.view(world * out_local.shape[0], *out_local.shape[1:]), out_local.contiguous(), group=group)
    dist.all_gather_into_tensor(lses.view(world * lse_local.shape[0], *lse_local.shape[1:]), lse_local.contiguous(), group=group)
    return merge_attention_parts(outs, lses)


class SharedBuffer:
    """One device buffer per rank that every rank of the job (one node) can write with plain
    stores: allocated by the library (cudaMalloc), its CUDA IPC handle exchanged through
    torch.distributed, mapped on the peers.  ptrs[0] is this rank's own buffer, the others follow
    in rank order (skipping this rank) - the order TurboQuantLinear.forward_scatter wants.  No
    multicast object is created anywhere."""

    def __init__(self, nbytes: int, group=None):
        import ctypes as C
        import torch.distributed as dist
        from . import _lib
        self._L = _lib.load()
        self.nbytes = int(nbytes)
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        # 32 completion flags (one per rank) live behind the payload, 256-byte aligned
        self.flag_offset = (self.nbytes + 255) // 256 * 256
        # A rank whose allocation fails still takes part in the exchange (with None), so that all
        # ranks raise together instead of leaving the others inside the collective.
        self.local = self._L.tq_shared_alloc(self.flag_offset + 256)
        mine, err = None, None
        if not self.local:
            err = "tq_shared_alloc: " + _lib.last_error()
        else:
            handle = C.create_string_buffer(64)
            if self._L.tq_shared_export(C.c_void_p(self.local), handle, 64) != 0:
                err = "tq_shared_export: " + _lib.last_error()
            else:
                mine = bytes(handle.raw)
        handles = [None] * self.world
        dist.all_gather_object(handles, mine, group=group)
        if any(h is None for h in handles):
            if self.local:
                self._L.tq_shared_free(C.c_void_p(self.local))
            self.local = None
            raise _lib.TQError(err or "a peer could not allocate or export its shared buffer")
        self._peers = []
        self.ptrs = [self.local]
        for r in range(self.world):
            if r == self.rank:
                continue
            h = C.create_string_buffer(handles[r], 64)
            p = self._L.tq_shared_open(h, 64)
            if not p:
                raise _lib.TQError("tq_shared_open: " + _lib.last_error())
            self._peers.append(p)
            self.ptrs.append(p)
        self._group = group
        self.flag_ptrs = [p + self.flag_offset for p in self.ptrs]   # same order as ptrs
        self.local_flags = self.local + self.flag_offset

    def tensor(self, shape, dtype):
        """A torch view of this rank's own buffer (zero-copy)."""
        import torch
        typestr = {torch.float16: "<f2", torch.float32: "<f4", torch.uint8: "|u1"}[dtype]

        class _View:
            pass
        v = _View()
        v.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(self.local), False),
                                      "version": 2, "strides": None}
        return torch.as_tensor(v, device="cuda")

    def close(self):
        import ctypes as C
        import torch
        import torch.distributed as dist
        if getattr(self, "local", None) is None:
            return
        torch.cuda.synchronize()
        dist.barrier(group=self._group)        # nobody may still be writing into a buffer about to go
        for p in self._peers:
            self._L.tq_shared_close(C.c_void_p(p))
        self._L.tq_shared_free(C.c_void_p(self.local))
        self.local, self._peers, self.ptrs = None, [], []


class Exchange:
    """The data plane of the sharded paths for one rank: a SharedBuffer every rank can write, plus the
    library's exchange handle (tq_exchange_*: broadcast a block to all ranks with plain 16-byte
    peer stores and raise this rank's flag; wait for every rank's flag; epochs live in device
    memory, so the sequence can be captured in a CUDA graph).  Every rank must issue the same
    sequence of broadcast() and wait() calls.

      all-gather of row shards   : compute the shard in place in self.buf, broadcast(offset, ...); wait()
      all-reduce of partial sums : compute the partial into slot `rank`, broadcast; wait(); sum_f16()
      merge of attention parts   : compute (out | lse) into slot `part`, broadcast; wait(); merge_attention()
    """

    def __init__(self, nbytes: int, group=None):
        import ctypes as C
        from . import _lib
        self._L = _lib.load()
        self.buf = SharedBuffer(nbytes, group)
        self.rank, self.world = self.buf.rank, self.buf.world
        self._h = self._L.tq_exchange_create(self.rank, self.world)
        if not self._h:
            raise _lib.TQError("tq_exchange_create: " + _lib.last_error())
        n_peers = self.world - 1
        self._flags = (C.c_void_p * self.world)(*self.buf.flag_ptrs)
        self._n_peers = n_peers

    @property
    def local(self) -> int:
        return self.buf.local

    def broadcast(self, offset: int, rows: int, row_bytes: int, stride_bytes: int, stream=None, peers=None):
        """Copy the block at byte `offset` of this rank's buffer (rows x row_bytes, rows stride_bytes
        apart) to the same place of the buffers of `peers` (indices into buf.ptrs; default: all other
        ranks) and raise this rank's flag on every rank."""
        import ctypes as C
        from . import _lib
        idx = list(range(1, self.world)) if peers is None else list(peers)
        if not idx:                       # a single rank: only the flag is raised (copy onto itself)
            idx = [0]
        dst = (C.c_void_p * len(idx))(*[self.buf.ptrs[i] + offset for i in idx])
        _lib.check(self._L.tq_exchange_broadcast(self._h, C.c_void_p(self.buf.local + offset), dst, len(idx), rows, row_bytes,
                                                  stride_bytes, stride_bytes, self._flags, self.world, _stream_ptr(stream)),
                   "tq_exchange_broadcast")

    def forward_allgather(self, lin, x, dst_row_stride: int, row_offset: int, buffer_offset: int = 0, wait: bool = True,
                          stream=None):
        """A row-sharded layer's decode forward fused with the all-gather of its result
        (tq_linear_forward_allgather): this rank's rows go to its own buffer at byte `buffer_offset`
        (+ row_offset elements), the kernel's last CTA copies them to the same place of every other
        rank's buffer and raises this rank's flag; with wait=True every CTA first waits for the
        previous exchange (counts as one wait())."""
        import ctypes as C
        import numpy as np
        from . import _lib
        from .api import _ptr
        batch = int(np.prod(x.shape[:-1])) if len(x.shape) > 1 else 1
        dst = (C.c_void_p * self.world)(*[p + buffer_offset for p in self.buf.ptrs])
        _lib.check(self._L.tq_linear_forward_allgather(lin.handle, self._h, _ptr(x), batch, dst, self.world, int(dst_row_stride),
                                                        int(row_offset), self._flags, self.world,
                                                        C.c_void_p(self.buf.local_flags) if wait else None, self.world,
                                                        _stream_ptr(stream)), "tq_linear_forward_allgather")

    def rank_ptrs(self):
        """Every rank's buffer address in RANK order (this rank's own at index rank)."""
        others = iter(self.buf.ptrs[1:])
        return [self.buf.local if r == self.rank else next(others) for r in range(self.world)]

    def wait_packets(self, packets_offset: int, rows_per_rank: int, batch: int, out_ptr: int, out_row_stride: int, stream=None):
        """tq_exchange_wait_packets: after forward_allgather_packets on the same stream, wait for the other ranks' packets and
        write their rows into the gathered result at raw device address out_ptr ([batch][out_row_stride] fp16)."""
        import ctypes as C
        from . import _lib
        _lib.check(self._L.tq_exchange_wait_packets(self._h, C.c_void_p(self.buf.local + packets_offset), int(rows_per_rank), int(batch),
                                                     C.c_void_p(int(out_ptr)), int(out_row_stride), _stream_ptr(stream)),
                   "tq_exchange_wait_packets")

    def forward_allgather_packets(self, lin, x, y, packets_offset: int = 0, wait: bool = True, stream=None, y_ptr=None, y_row_stride=None):
        """tq_linear_forward_allgather_packets: y (device fp16 [batch, out]) gets this rank's rows; the other ranks
        get them as flag-in-data packets in their buffers at byte `packets_offset`
        ([epoch parity][source rank][batch * out / 4 packets of 16 bytes]); with wait=True every CTA first polls
        the packets of the previous call.  The packet region must be zero before the first call."""
        import ctypes as C
        import numpy as np
        from . import _lib
        from .api import _ptr
        batch = int(np.prod(x.shape[:-1])) if len(x.shape) > 1 else 1
        bufs = (C.c_void_p * self.world)(*[p + packets_offset for p in self.rank_ptrs()])
        yp = C.c_void_p(int(y_ptr)) if y_ptr is not None else _ptr(y)
        ys = int(y_row_stride) if y_row_stride is not None else int(y.shape[-1])
        _lib.check(self._L.tq_linear_forward_allgather_packets(lin.handle, self._h, _ptr(x), batch, yp, ys, bufs,
                                                                1 if wait else 0, _stream_ptr(stream)),
                   "tq_linear_forward_allgather_packets")

    def unpack_packets(self, packets_offset: int, n_packets: int, out, stream=None):
        """Packets at byte `packets_offset` of this rank's buffer -> contiguous fp16 in `out` (4 values per packet)."""
        import ctypes as C
        from . import _lib
        from .api import _ptr
        _lib.check(self._L.tq_exchange_unpack_packets(C.c_void_p(self.buf.local + packets_offset), int(n_packets), _ptr(out),
                                                       _stream_ptr(stream)), "tq_exchange_unpack_packets")

    def wait(self, stream=None):
        import ctypes as C
        from . import _lib
        _lib.check(self._L.tq_exchange_wait(self._h, C.c_void_p(self.buf.local_flags), self.world, _stream_ptr(stream)),
                   "tq_exchange_wait")

    def sum_f16(self, slots_offset: int, n_slots: int, slot_stride_elems: int, count: int, out_ptr: int, residual_ptr: int = 0,
                stream=None):
        import ctypes as C
        from . import _lib
        _lib.check(self._L.tq_exchange_sum_f16(C.c_void_p(self.buf.local + slots_offset), n_slots, slot_stride_elems, count,
                                                C.c_void_p(residual_ptr) if residual_ptr else None, C.c_void_p(out_ptr),
                                                _stream_ptr(stream)), "tq_exchange_sum_f16")

    def merge_attention(self, outs_offset: int, lses_offset: int, parts: int, rows: int, head_dim: int, part_stride_out: int,
                        part_stride_lse: int, out_ptr: int, stream=None):
        import ctypes as C
        from . import _lib
        _lib.check(self._L.tq_exchange_merge_attention(C.c_void_p(self.buf.local + outs_offset), C.c_void_p(self.buf.local + lses_offset),
                                                        parts, rows, head_dim, part_stride_out, part_stride_lse, C.c_void_p(out_ptr),
                                                        _stream_ptr(stream)), "tq_exchange_merge_attention")

    def check_status(self):
        from . import _lib
        _lib.check(self._L.tq_exchange_status(self._h), "tq_exchange_status")

    def close(self):
        if getattr(self, "_h", None):
            self._L.tq_exchange_free(self._h)
            self._h = None
        self.buf.close()


def _stream_ptr(stream):
    import ctypes as C
    if stream is None:
        return None
    return C.c_void_p(stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream))


def col_range(in_features: int, block_size: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous input-feature range of `rank` for a ROW-parallel linear (o_proj, down_proj):
    whole WHT blocks, as even as possible, so every rank rotates only its own slice of x."""
    blocks = in_features // block_size
    b0 = blocks * rank // world
    b1 = blocks * (rank + 1) // world
    return b0 * block_size, b1 * block_size


def shard_quantized_cols(packed_primary, packed_residual, norms, in_features: int, block_size: int, rank: int,
                         world: int):
    """Column slice of a QuantizedWeight for a row-parallel linear.  The codes of columns
    [c0, c1) are cut out of both planes (two codes per byte; 5-bit primaries one per byte); the
    per-row norm is a plain factor of the row, so every rank keeps it - multiplied by
    sqrt((c1 - c0) / in_features), because a TurboQuantLinear over the slice divides by the
    square root of ITS in_features.  Each rank then runs an ordinary forward on x[:, c0:c1] and the
    partial outputs are summed (all-reduce).  Seeds and codebooks are unchanged: the sign pattern
    repeats per WHT block, so whole blocks carry over."""
    import numpy as np
    c0, c1 = col_range(in_features, block_size, rank, world)
    primary_per_byte = 2 if packed_primary.shape[1] == in_features // 2 else 1
    pp = packed_primary[:, c0 // primary_per_byte: c1 // primary_per_byte]
    pr = packed_residual[:, c0 // 2: c1 // 2]
    scale = np.float32(np.sqrt(np.float32(c1 - c0) / np.float32(in_features)))
    return pp, pr, (norms * scale).astype(np.float32), (c0, c1)
