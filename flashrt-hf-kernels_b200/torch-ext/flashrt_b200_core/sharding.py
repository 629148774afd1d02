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


class SharedActivations:
    """NVFP4 activation buffers that every rank of a process group holds a copy of and every rank fills a row
    shard of: `produce` runs the fused residual-add + RMSNorm -> NVFP4 producer on this rank's rows and stores the
    result into ALL ranks' copies from inside the kernel (NVSwitch multicast stores when the allocation has a
    multicast mapping, peer stores otherwise); `wait` enqueues the bounded wait for every rank's rows.  Two buffers
    (default) used alternately cover a producer -> GEMMs -> producer -> GEMMs chain: a buffer is refilled only
    after every rank has passed the wait on the other one.

    The memory is one torch symmetric-memory allocation, made once here; `produce` and `wait` allocate nothing."""

    def __init__(self, rows: int, dim: int, device, group=None, buffers: int = 2, multicast: bool = True):
        import ctypes as C
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        from . import capi
        self.capi, self.C = capi, C
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if rows % (128 * self.world) != 0:
            raise ValueError(f"rows={rows} must be a multiple of 128 * world ({128 * self.world}): row shards keep "
                             "whole 128-row scale groups")
        self.rows, self.dim, self.buffers = rows, dim, buffers
        self.rows_local = rows // self.world
        self.row0 = self.rank * self.rows_local
        al = lambda n: (n + 255) // 256 * 256
        pk, sf = al(rows * dim // 2), al(sf_bytes(rows, dim))
        self._per = pk + sf
        ctrl = al(buffers * 64)                            # per buffer: 8 flags (uint32), then a counter word
        self.mem = symm.empty(buffers * self._per + ctrl, dtype=torch.uint8, device=device)
        self.handle = symm.rendezvous(self.mem, self.group)
        self.mem.zero_()
        torch.cuda.synchronize(device)
        self.handle.barrier()                              # nobody publishes a flag before everybody has zeroed
        self.packed = [self.mem[b * self._per:b * self._per + rows * dim // 2].view(rows, dim // 2) for b in range(buffers)]
        self.sf = [self.mem[b * self._per + pk:b * self._per + pk + sf_bytes(rows, dim)] for b in range(buffers)]
        self._pk_off = [b * self._per for b in range(buffers)]
        self._sf_off = [b * self._per + pk for b in range(buffers)]
        self._ctrl_off = [buffers * self._per + b * 64 for b in range(buffers)]
        self._bases = [int(p) for p in self.handle.buffer_ptrs]
        mc = int(self.handle.multicast_ptr or 0) if multicast else 0
        self._mc = mc
        self.epoch = [0] * buffers
        arr = lambda vals: (C.c_void_p * 8)(*(list(vals) + [None] * (8 - len(vals))))
        self._dst_pk = [arr([base + self._pk_off[b] for base in self._bases]) for b in range(buffers)]
        self._dst_sf = [arr([base + self._sf_off[b] for base in self._bases]) for b in range(buffers)]
        self._flags = [arr([base + self._ctrl_off[b] for base in self._bases]) for b in range(buffers)]

    @property
    def uses_multicast(self) -> bool:
        return bool(self._mc)

    WAIT_PEERS = 0x100                                    # FRT_PRODUCER_WAIT_PEERS

    def produce(self, b: int, residual, x, weight, eps: float, stream, inv_global_scale: float = 1.0, flags: int = 0,
                wait: bool = True):
        """residual / x: THIS rank's rows (rows_local, dim) bf16; fills rows [row0, row0 + rows_local) of buffer b on
        every rank and publishes the new epoch of the buffer.  With `wait` (default) the call also waits, on the
        stream, until every rank's rows have landed in this rank's copy: the buffer may be consumed by the next
        kernel of the stream.  With wait=False enqueue `wait(b, stream)` before the first consumer."""
        capi, C = self.capi, self.C
        self.epoch[b] += 1
        if wait:
            flags |= self.WAIT_PEERS
        mc_pk = C.c_void_p(self._mc + self._pk_off[b]) if self._mc else None
        mc_sf = C.c_void_p(self._mc + self._sf_off[b]) if self._mc else None
        local = self._bases[self.rank]
        rc = capi.lib().frt_norm_quant_nvfp4_bcast(
            capi.ptr(residual), capi.ptr(x), capi.ptr(weight), eps, inv_global_scale, mc_pk, mc_sf,
            self._dst_pk[b], self._dst_sf[b], self.world, self.row0, self.rows_local, self.dim, flags,
            C.c_void_p(local + self._ctrl_off[b] + 32), self._flags[b], self.world, self.rank, self.epoch[b], stream)
        capi.check(rc, "frt_norm_quant_nvfp4_bcast")

    def wait(self, b: int, stream):
        capi, C = self.capi, self.C
        rc = capi.lib().frt_peer_wait(C.c_void_p(self._bases[self.rank] + self._ctrl_off[b]), self.world,
                                      self.epoch[b], stream)
        capi.check(rc, "frt_peer_wait")
