"""Sharded matmul (M-split, N-split): host logic with gloo ranks on CPU, CUDA path on GPUs."""
import os
import socket

import numpy as np
import pytest

import cases
from onednn_b200 import dtypes as dt, multi_gpu, workloads as W
from oracle import binding as ob


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _int8_case(M=24, N=64, K=96):
    c = W.config1(M, N, K, seed=5)
    return c


def _gloo_rank(rank, world, port, how, q):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        case = _int8_case()
        part = W.shard(case, rank, world, how)
        mine = ob.run_oracle(part, tanh_mode=1)                     # this rank's slice of dst
        got = [torch.empty_like(torch.from_numpy(mine)) for _ in range(world)]
        dist.all_gather(got, torch.from_numpy(mine.copy()))
        if how == "n":
            full = multi_gpu.gather_columns_host(np.stack([g.numpy() for g in got]))
        else:
            full = multi_gpu.assemble_rows_host([g.numpy() for g in got])
        want = ob.run_oracle(case, tanh_mode=1)
        q.put((rank, bool((full == want).all()), full.shape))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("how", ["m", "n"])
def test_split_matches_unsharded_gloo_world2(how):
    """Two CPU ranks: each computes its shard with the oracle, the shards are all-gathered
    over gloo and assembled; the result equals the unsharded problem bit for bit."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_gloo_rank, args=(r, 2, port, how, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    case = _int8_case()
    for rank, same, shape in out:
        assert same, "rank %d: sharded result differs" % rank
        assert shape == (case.M, case.N)


def test_shard_shapes():
    case = W.config4(32, 128, 64)
    for world in (1, 2, 4):
        for r in range(world):
            m = W.shard(case, r, world, "m")
            n = W.shard(case, r, world, "n")
            assert (m.M, m.N, m.K) == (case.M // world, case.N, case.K)
            assert (n.M, n.N, n.K) == (case.M, case.N // world, case.K)
            assert n.wei.shape == (case.K, case.N // world) and n.bias.shape == (1, case.N // world)
            assert n.wei_scale.data.size == case.N // world


def test_gather_columns_host():
    st = np.arange(3 * 4 * 5).reshape(3, 4, 5)
    full = multi_gpu.gather_columns_host(st)
    assert full.shape == (4, 15)
    for r in range(3):
        assert (full[:, r * 5:(r + 1) * 5] == st[r]).all()


@pytest.mark.gpu
def test_gather_columns_kernel():
    import torch
    from onednn_b200 import kernels_abi
    g, M, ns = 4, 37, 48
    st = torch.randint(-128, 127, (g, M, ns), dtype=torch.int8, device="cuda")
    dst = torch.zeros((M, g * ns), dtype=torch.int8, device="cuda")
    rc = kernels_abi.lib().b200_gather_columns_launch(st.data_ptr(), dst.data_ptr(), M, g * ns, g, 1,
                                                      torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert (dst.cpu().numpy() == multi_gpu.gather_columns_host(st.cpu().numpy())).all()
    # a slice that is not a multiple of 16 bytes is refused, not mangled
    assert kernels_abi.lib().b200_gather_columns_launch(st.data_ptr(), dst.data_ptr(), M, 4 * 10, 4, 1, 0) == -1


def _nccl_rank(rank, world, port, q, mode="nccl"):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        case = W.config4(256, 512, 128, seed=9)
        op = multi_gpu.NSplitMatmul(case, rank, world, rank, mode=mode)
        for _ in range(2):   # twice: the second run overwrites a destination that is already full
            op.execute()
        got = op.result()
        want = ob.run_oracle(case, tanh_mode=1, exact_acc=1)
        a, b = dt.to_f32(got, case.dst_dt), dt.to_f32(want, case.dst_dt)
        q.put((rank, op.impl, float(np.abs(a - b).max()), float(np.abs(b).max())))
    except Exception as ex:  # the parent must hear about it instead of waiting
        q.put((rank, "error: %r" % (ex,), float("inf"), 0.0))
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["nccl", "p2p"])
def test_n_split_cuda(mode):
    """N-split through the library: on two GPUs when the box has them (NCCL all-gather, or
    slices stored into the peers' copies by the matmul's epilogue), else the same code path
    with a single rank."""
    import torch
    world = 2 if torch.cuda.device_count() >= 2 else 1
    if world == 1:
        case = W.config4(256, 512, 128, seed=9)
        op = multi_gpu.NSplitMatmul(case, 0, 1, 0, mode=mode)
        op.execute()
        got = op.result()
        want = ob.run_oracle(case, tanh_mode=1, exact_acc=1)
        assert np.allclose(dt.to_f32(got, case.dst_dt), dt.to_f32(want, case.dst_dt), rtol=1e-2, atol=1e-2)
        return
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_nccl_rank, args=(r, world, port, q, mode)) for r in range(world)]
    for p in procs:
        p.start()
    out = [q.get(timeout=150) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, impl, err, mag in out:
        assert err <= 1e-2 * max(1.0, mag), (rank, impl, err, mag)
