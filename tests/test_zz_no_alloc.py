"""The grouped GEMM entry point that allocates nothing.

Some callers cannot hand the library a scratch buffer: they run inside a host
runtime that owns all device memory and forbids allocation on its worker
threads, or in a process whose free device memory already belongs to another
pool, so that an allocation would fail.  For them
frt_nvfp4_grouped_gemm_bf16_noalloc keeps the work list in a fixed array inside
the library.  This file is collected last so that a run stopping at the first
failure has already exercised every other test; it must also pass on its own
in a fresh process.

Checked here, through the C ABI: two calls in a row give exactly the output of
the caller-workspace entry point (the array is shared and keeps the previous
call's contents, so the second call proves the reset), and sizes beyond the
fixed maximum are refused with a clear error."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from tests.gpu_common import DEV, O, capi  # noqa: E402


def make_case(rows_per_expert, n, k, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    experts = len(rows_per_expert)
    offs = torch.zeros(experts + 1, dtype=torch.int32)
    offs[1:] = torch.cumsum(torch.tensor(rows_per_expert), 0)
    rows = int(offs[-1])
    L = capi.lib()
    ap = torch.randint(0, 256, (rows, k // 2), generator=g, dtype=torch.uint8, device=DEV)
    wp = torch.randint(0, 256, (experts, n, k // 2), generator=g, dtype=torch.uint8, device=DEV)
    asw = torch.randint(32, 80, (int(L.frt_nvfp4_sf_swizzled_bytes(rows, k)),), generator=g, dtype=torch.uint8,
                        device=DEV)
    wsw = torch.randint(32, 80, (experts, int(L.frt_nvfp4_sf_swizzled_bytes(n, k))), generator=g,
                        dtype=torch.uint8, device=DEV)
    alpha = torch.rand(experts, generator=g, device=DEV) + 0.5
    return rows, experts, offs.to(DEV), ap, wp, asw, wsw, alpha


def call(noalloc, case, n, k, out):
    rows, experts, offs, ap, wp, asw, wsw, alpha = case
    L, P = capi.lib(), capi.ptr
    common = (P(ap), P(asw), P(wp), P(wsw), P(alpha), P(offs), None, 0, P(out), rows, n, k, experts,
              n * (k // 2), int(wsw.shape[1]))
    if noalloc:
        rc = L.frt_nvfp4_grouped_gemm_bf16_noalloc(*common, capi.stream_ptr())
    else:
        work = torch.empty(int(L.frt_nvfp4_grouped_gemm_workspace_bytes(rows, experts)), dtype=torch.uint8, device=DEV)
        rc = L.frt_nvfp4_grouped_gemm_bf16(*common, P(work), capi.stream_ptr())
    torch.cuda.synchronize()
    return rc


def test_noalloc_matches_workspace_entry_point_twice_in_a_row():
    n, k = 384, 512
    # a large first problem leaves a long stale work list behind for the small second one
    first = make_case([300, 0, 129, 64, 1000, 7, 513], n, k, seed=101)
    second = make_case([33, 95], n, k, seed=202)
    for case in (first, second):
        rows = case[0]
        want = torch.zeros(rows, n, dtype=torch.bfloat16, device=DEV)
        got = torch.zeros(rows, n, dtype=torch.bfloat16, device=DEV)
        assert call(False, case, n, k, want) == 0
        assert call(True, case, n, k, got) == 0
        assert torch.equal(got, want)
        rel, cos = O.gemm_error_metrics(got.cpu(), want.cpu())     # the suite's GEMM tolerance, trivially met
        assert rel <= 1e-2 and cos >= 0.999
    # and once more on the first problem: same answer after the small one ran
    want = torch.zeros(first[0], n, dtype=torch.bfloat16, device=DEV)
    got = torch.zeros(first[0], n, dtype=torch.bfloat16, device=DEV)
    assert call(False, first, n, k, want) == 0 and call(True, first, n, k, got) == 0
    assert torch.equal(got, want)


def test_noalloc_refuses_sizes_beyond_its_fixed_array():
    L, P = capi.lib(), capi.ptr
    dummy = torch.zeros(64, dtype=torch.uint8, device=DEV)
    too_many_rows = L.frt_nvfp4_grouped_gemm_bf16_noalloc(
        P(dummy), P(dummy), P(dummy), P(dummy), P(dummy), P(dummy), None, 0, P(dummy), 131072 + 64, 64, 64, 4,
        64 * 32, 512, capi.stream_ptr())
    too_many_experts = L.frt_nvfp4_grouped_gemm_bf16_noalloc(
        P(dummy), P(dummy), P(dummy), P(dummy), P(dummy), P(dummy), None, 0, P(dummy), 64, 64, 64, 2049,
        64 * 32, 512, capi.stream_ptr())
    assert too_many_rows == -8 and too_many_experts == -8
    assert b"fixed maximum" in L.frt_error_string(-8)
