"""Host-side sharding of the NVFP4 linear path across the GPUs of one node.

GEMM: column-parallel.  A weight `[N, K/2]` is row-major over N, and its
swizzled scales are grouped by 128 output columns first, so with
`N % (world * 128) == 0` a rank's shard of both is one contiguous range: no
repacking, no copy.  Activations are replicated, each rank writes
`out[M, N/world]`; an all-gather of the outputs is optional and separate.
Producer: row-parallel on 128-row boundaries (scales again contiguous).
The reference has no multi-GPU code; this is new design."""
from __future__ import annotations


def sf_bytes(rows: int, dim: int) -> int:
    return ((rows + 127) // 128) * ((dim // 16 + 3) // 4) * 512


def column_shard_bounds(n: int, world: int, rank: int):
    if n % (world * 128) != 0:
        raise ValueError(f"N={n} must be a multiple of world*128={world * 128} to shard on scale-group boundaries")
    per = n // world
    return rank * per, (rank + 1) * per


def shard_weight(packed, sf_swizzled, n: int, k: int, world: int, rank: int):
    """Views of rank's columns of a packed weight [n, k/2] and its swizzled scales."""
    lo, hi = column_shard_bounds(n, world, rank)
    per_group = ((k // 16 + 3) // 4) * 512
    return packed[lo:hi], sf_swizzled[(lo // 128) * per_group:(hi // 128) * per_group]


def row_shard_bounds(m: int, world: int, rank: int):
    """Rows of the producer owned by `rank`: whole 128-row scale groups, remainder to the last ranks' left."""
    groups = (m + 127) // 128
    base, extra = divmod(groups, world)
    g_lo = rank * base + min(rank, extra)
    g_hi = g_lo + base + (1 if rank < extra else 0)
    return min(g_lo * 128, m), min(g_hi * 128, m)


def gather_columns(dist, out_local, world: int):
    """all-gather `[M, N/world]` shards into `[M, N]` (one collective + a local permute)."""
    import torch
    m, n_loc = out_local.shape
    gathered = torch.empty((world * m, n_loc), dtype=out_local.dtype, device=out_local.device)
    dist.all_gather_into_tensor(gathered, out_local.contiguous())
    return gathered.view(world, m, n_loc).permute(1, 0, 2).reshape(m, world * n_loc)
