"""The weight-compressed kernel's entry point that allocates nothing.

Who needs it: callers that hold device pointers but may not call cudaMalloc --
a plugin living inside a runtime that owns all device memory, or a decode loop
in a section of a serving engine where touching the allocator is forbidden.
b200_matmul_wc_noalloc_launch runs the same kernels as b200_matmul_wc_launch,
with the partial-sum scratch in a fixed array inside the library instead of a
caller-allocated buffer.

The test drives both entry points directly through the C ABI on the same
inputs and requires identical destinations (same kernels, same order of
operations apart from the order of the atomic additions, hence the tolerance
the other weight-compression tests use), twice in a row: the second call finds
the array as the first one left it.  It also checks the size limit.
"""
import ctypes as C

import numpy as np
import pytest

from onednn_b200 import api, dtypes as dt, kernels_abi as K, workloads as W

pytestmark = pytest.mark.gpu


def _params(case, x, wpacked, scales, zps, dst, scratch):
    p = K.MatmulParams()
    p.M, p.N, p.K = case.M, case.N, case.K
    p.src, p.src_dt, p.src_sm, p.src_sk = x.data_ptr(), dt.BF16, case.K, 1
    p.wei, p.wei_dt, p.wei_layout = wpacked.data_ptr(), dt.U4, K.WEI_WC4_TILED
    p.dst, p.dst_dt, p.dst_sm, p.dst_sn = dst.data_ptr(), dt.BF16, case.N, 1
    g = case.wei_scale.groups[0]
    p.wei_scale = K.quant(scales.data_ptr(), dt.BF16, s0=case.N, s1=1, g0=g, g1=1)
    p.wei_zp = K.quant(zps.data_ptr(), dt.U4, s0=case.N, s1=1, g0=g, g1=1)
    for q in (p.src_scale, p.dst_scale, p.src_zp, p.dst_zp):
        q.g0 = q.g1 = 1
    p.apply_to_int = 1
    if scratch is not None:
        p.scratch, p.scratch_bytes = scratch.data_ptr(), scratch.numel()
    return p


@pytest.mark.parametrize("M", [1, 5])
def test_no_alloc_entry_point_matches_the_allocating_one(M):
    import torch
    L = K.lib()
    case = W.config2(M, N=512, K=1024)
    dev = torch.device("cuda", 0)
    stream = torch.cuda.current_stream().cuda_stream

    def up(a):
        return torch.from_numpy(np.ascontiguousarray(a).view(np.uint8).reshape(-1)).to(dev)

    x, wplain, scales, zps = up(case.src), up(case.wei), up(case.wei_scale.data), up(case.wei_zp.data)
    wpacked = torch.empty_like(wplain)
    assert L.b200_wc_pack_launch(wplain.data_ptr(), wpacked.data_ptr(), case.K, case.N, dt.U4, stream) == 0

    # reference: the existing entry point with a caller-allocated scratch
    dst_ref = torch.zeros(case.M * case.N * 2, dtype=torch.uint8, device=dev)
    p = _params(case, x, wpacked, scales, zps, dst_ref, None)
    scratch = torch.zeros(L.b200_matmul_scratch_bytes(C.byref(p), 2), dtype=torch.uint8, device=dev)
    p = _params(case, x, wpacked, scales, zps, dst_ref, scratch)
    assert L.b200_matmul_wc_launch(C.byref(p), stream) == 0
    torch.cuda.synchronize()
    want = dt.bf16_to_f32(dst_ref.cpu().numpy().view(np.uint16)).astype(np.float64)

    before = torch.cuda.memory_allocated()
    for call in range(2):
        dst = torch.full_like(dst_ref, 0x7F)
        q = _params(case, x, wpacked, scales, zps, dst, None)   # no scratch passed at all
        assert L.b200_matmul_wc_noalloc_launch(C.byref(q), stream) == 0
        torch.cuda.synchronize()
        got = dt.bf16_to_f32(dst.cpu().numpy().view(np.uint16)).astype(np.float64)
        assert np.all(np.abs(got - want) <= case.atol + case.rtol * np.abs(want)), "call %d" % call
        del dst
    assert torch.cuda.memory_allocated() == before


def test_no_alloc_entry_point_rejects_what_does_not_fit():
    import torch
    L = K.lib()
    limit = L.b200_matmul_wc_noalloc_max_bytes()
    assert limit == 2 << 20
    case = W.config2(1, N=64, K=128)
    dev = torch.device("cuda", 0)
    buf = torch.zeros(1 << 16, dtype=torch.uint8, device=dev)
    p = _params(case, buf, buf, buf, buf, buf, None)
    p.M, p.N = 64, limit // 4 // 64 + 16          # M * N * 4 bytes just over the array
    assert L.b200_matmul_wc_noalloc_launch(C.byref(p), None) == K.ERR_TOO_LARGE
    # exactly at the boundary: the partial sums (rounded up to 256 bytes) and the strip counters
    # (N / 16 words, rounded up to 256 bytes) share the array
    N = 1024
    counters = (N // 16 * 4 + 255) // 256 * 256
    rows_fit = (limit - counters) // (N * 4)
    x = torch.zeros(rows_fit + 1, 128, dtype=torch.bfloat16, device=dev)
    w = torch.zeros(128 * N // 2, dtype=torch.uint8, device=dev)
    sz = torch.zeros(N, dtype=torch.bfloat16, device=dev)
    out = torch.zeros((rows_fit + 1) * N, dtype=torch.bfloat16, device=dev)
    edge = W.config2(1, N=N, K=128)
    for rows, want in ((rows_fit, 0), (rows_fit + 1, K.ERR_TOO_LARGE)):
        p = _params(edge, x, w, sz, w, out, None)
        p.M = rows
        assert (rows * N * 4 + 255) // 256 * 256 + counters <= limit or want != 0
        assert L.b200_matmul_wc_noalloc_launch(C.byref(p), torch.cuda.current_stream().cuda_stream) == want
    torch.cuda.synchronize()
    p = _params(case, buf, buf, buf, buf, buf, None)
    p.wei_layout = K.WEI_PLAIN                    # would need a packing scratch
    assert L.b200_matmul_wc_noalloc_launch(C.byref(p), None) == K.ERR_UNSUPPORTED
    p = _params(case, buf, buf, buf, buf, buf, None)
    p.src_dt = dt.F32                             # would need a conversion scratch
    assert L.b200_matmul_wc_noalloc_launch(C.byref(p), None) == K.ERR_UNSUPPORTED
