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
    padded = torch.zeros((batch, width), dtype=local.dtype, device=local.device)
    padded[:, : local.shape[1]] = local
    flat = torch.empty((world * batch, width), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(flat, padded)
    gathered = flat.view(world, batch, width)
    out = torch.empty((batch, out_features), dtype=local.dtype, device=local.device)
    for r, (s, e) in enumerate(spans):
        out[:, s:e] = gathered[r, :, : e - s]
    return out
