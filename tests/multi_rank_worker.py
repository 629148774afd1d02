"""Worker of tests/test_gpu_multi_rank.py, one process per GPU (launched by torch.distributed.run).

Every rank runs the fused producer on its row shard with the in-kernel exchange (NVSwitch multicast stores, then
plain peer stores) and must end up with exactly the bytes the one-GPU producer writes for the whole tensor, on
both buffers and over several epochs; a column-sharded GEMM on the shared buffer must equal the same columns of
the unsharded GEMM."""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "flashrt-hf-kernels_b200" / "torch-ext"))

from flashrt_b200_core import alloc_fp4, capi, load  # noqa: E402
from flashrt_b200_core.sharding import SharedActivations, shard_weight  # noqa: E402


def main():
    rank, world, lr = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(lr)
    dev = torch.device("cuda", lr)
    dist.init_process_group("nccl", device_id=dev)
    load()
    L, P = capi.lib(), capi.ptr
    st = capi.stream_ptr()
    M, H, N = 128 * world * 3, 1024, 256 * world
    g = torch.Generator(device=dev).manual_seed(5)                  # the same tensors on every rank
    hidden = torch.randn(M, H, generator=g, device=dev).to(torch.bfloat16)
    residual0 = torch.randn(M, H, generator=g, device=dev).to(torch.bfloat16)
    norm_w = (1 + 0.1 * torch.randn(H, generator=g, device=dev)).to(torch.bfloat16)
    w = (torch.randn(N, H, generator=g, device=dev) * 0.05).to(torch.bfloat16)
    wp, wsf = alloc_fp4(N, H, dev)
    capi.check(L.frt_nvfp4_quantize(P(w), 0, P(wp), P(wsf), N, H, st))
    # one-GPU result on the whole tensor
    want_res = residual0.clone()
    want_p, want_sf = alloc_fp4(M, H, dev)
    capi.check(L.frt_norm_quant_nvfp4(P(want_res), P(hidden), P(norm_w), 1e-6, 1.0, None, P(want_p), P(want_sf), M, H, 0, st))
    want_out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    capi.check(L.frt_nvfp4_gemm_bf16(P(want_p), P(want_sf), P(wp), P(wsf), None, None, P(want_out), M, N, H, 1.0, 0.0, st))
    torch.cuda.synchronize()
    for multicast in (True, False):
        sh = SharedActivations(M, H, dev, multicast=multicast)
        if multicast and not sh.uses_multicast and rank == 0:
            print("note: no multicast mapping on this system, peer stores only", flush=True)
        r0, r1 = sh.row0, sh.row0 + sh.rows_local
        for epoch in range(3):
            for b in range(sh.buffers):
                res = residual0.clone()
                sh.packed[b].fill_(0xEE)
                sh.sf[b].fill_(0xEE)
                torch.cuda.synchronize()
                dist.barrier()                                       # nobody's poison lands after a peer's rows
                if epoch == 1:                                       # separate wait kernel
                    sh.produce(b, res[r0:r1], hidden[r0:r1], norm_w, 1e-6, st, wait=False)
                    sh.wait(b, st)
                else:                                                # wait inside the finishing kernel
                    sh.produce(b, res[r0:r1], hidden[r0:r1], norm_w, 1e-6, st)
                n_loc = N // world
                wp_loc, wsf_loc = shard_weight(wp, wsf, N, H, world, rank)
                out = torch.empty(M, n_loc, device=dev, dtype=torch.bfloat16)
                capi.check(L.frt_nvfp4_gemm_bf16(P(sh.packed[b]), P(sh.sf[b]), P(wp_loc), P(wsf_loc), None, None, P(out),
                                                 M, n_loc, H, 1.0, 0.0, st))
                torch.cuda.synchronize()
                assert torch.equal(sh.packed[b], want_p), (rank, multicast, epoch, b, "packed")
                assert torch.equal(sh.sf[b], want_sf), (rank, multicast, epoch, b, "scales")
                assert torch.equal(res[r0:r1], want_res[r0:r1]), (rank, "residual rows of this rank")
                assert torch.equal(res[:r0], residual0[:r0]) and torch.equal(res[r1:], residual0[r1:])
                assert torch.equal(out, want_out[:, rank * n_loc:(rank + 1) * n_loc]), (rank, "gemm shard")
                status = torch.zeros(1, dtype=torch.int32)
                import ctypes as C
                v = C.c_uint(0)
                capi.check(L.frt_device_status(st, C.byref(v)))
                assert v.value == 0, hex(v.value)
                dist.barrier()
        del sh
    if rank == 0:
        print("MULTI_RANK_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
