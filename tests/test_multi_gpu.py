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


def _checked_n_split(op, case, want_full, dist=None):
    """Run ``op`` once on a destination filled with a sentinel and count the elements that differ
    from the unsharded primitive's result on the same GPU; then once more on the already full
    destination (a store that is skipped the second time would otherwise hide behind the first)."""
    import torch
    bad = []
    for _ in range(2):
        op.dst.fill_(multi_gpu.SENTINEL)
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()   # nobody's kernel stores into a copy that its owner is still filling
        op.execute()
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        bad.append(multi_gpu.count_mismatched_elements(op.dst, want_full, op.elem))
    return bad


def _nccl_rank(rank, world, port, q, mode="nccl"):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        case = W.config4(256, 512, 128, seed=9)
        want_full = multi_gpu.unsharded_on_this_gpu(case, rank)
        op = multi_gpu.NSplitMatmul(case, rank, world, rank, mode=mode)
        bad = _checked_n_split(op, case, want_full, dist)
        oracle = ob.run_oracle(case, tanh_mode=1, exact_acc=1)
        vs_oracle = int((op.result().view(np.uint16) != oracle.view(np.uint16)).sum())
        q.put((rank, op.impl, op.mode, bad, vs_oracle))
    except Exception as ex:  # the parent must hear about it instead of waiting
        q.put((rank, "error: %r" % (ex,), mode, [-1], -1))
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["nccl", "p2p"])
def test_n_split_cuda(mode):
    """N-split through the library on two GPUs (NCCL all-gather, or slices stored into the peers'
    copies by the matmul's epilogue): the assembled dst on every rank equals, byte for byte, what
    the unsharded primitive gives on that GPU and what the CPU oracle gives.  With one GPU the
    all-gather path runs with a single rank; the peer-store kernel has its own one-GPU test below."""
    import torch
    world = 2 if torch.cuda.device_count() >= 2 else 1
    if world == 1:
        if mode == "p2p":
            pytest.skip("needs two GPUs; test_peer_store_kernel_with_local_mirrors covers the kernel on one")
        case = W.config4(256, 512, 128, seed=9)
        op = multi_gpu.NSplitMatmul(case, 0, 1, 0, mode=mode)
        bad = _checked_n_split(op, case, multi_gpu.unsharded_on_this_gpu(case, 0))
        assert bad == [0, 0]
        want = ob.run_oracle(case, tanh_mode=1, exact_acc=1)
        assert np.array_equal(op.result().view(np.uint16), want.view(np.uint16))
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
    for rank, impl, ran_as, bad, vs_oracle in out:
        assert ran_as == mode, (rank, impl, ran_as)
        assert bad == [0, 0] and vs_oracle == 0, (rank, impl, bad, vs_oracle)


@pytest.mark.gpu
@pytest.mark.parametrize("parts", [2, 4])
def test_peer_store_kernel_with_local_mirrors(parts):
    """The kernel variant that also stores every finished block into the other ranks' copies of
    dst, on ONE GPU: the copies are further buffers on the same device and the ranks' column
    slices run one after the other.  Every copy must end up equal, byte for byte, to the
    unsharded primitive's result -- the same check the two-GPU test makes, so the kernel has
    correctness evidence wherever the tests run."""
    import torch
    from onednn_b200 import api
    case = W.config4(300, 128 * parts, 128, seed=10)   # ragged rows, several tiles per slice
    eng = api.Engine()
    ts = torch.cuda.current_stream()
    strm = api.Stream(eng, cuda_stream=ts.cuda_stream)
    want = multi_gpu.unsharded_on_this_gpu(case, 0)
    elem = 2
    copies = [torch.full((case.M, case.N * elem), multi_gpu.SENTINEL, dtype=torch.uint8, device="cuda") for _ in range(parts)]
    ns = case.N // parts
    keep = []
    for r in range(parts):
        plan = api.CasePlan(W.shard(case, r, parts, "n"), eng, strm, weights="any", dst_strides=(case.N, 1))
        assert "tcgen05_i8" in plan.impl
        off = r * ns * elem
        args = dict(plan.args)
        args[api.ARG_DST] = api.Memory(plan.mds["dst"], eng, handle=copies[r].data_ptr() + off)
        i = 0
        for o in range(parts):
            if o != r:
                args[api.ARG_B200_DST_PEER0 + i] = api.Memory(plan.mds["dst"], eng, handle=copies[o].data_ptr() + off)
                i += 1
        plan.prim.execute(strm, args)
        keep.append((plan, args))
    strm.wait()
    for r in range(parts):
        assert multi_gpu.count_mismatched_elements(copies[r], want, elem) == 0, "copy %d" % r
