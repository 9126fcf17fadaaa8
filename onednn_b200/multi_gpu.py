"""One matmul over the GPUs of a node: one process per GPU, ``torch.distributed`` for the plumbing.

The reference library has no multi-device matmul.  The two splits below follow from
its arithmetic (``src/cpu/matmul/ref_matmul_int8.cpp:154-261``: every dst element is
computed on its own from a full K reduction), so any partition of dst rows or columns
gives results identical to the unsharded primitive:

* M-split: rank r owns rows ``[r*M/g, (r+1)*M/g)`` of src and dst; weights, scales and
  bias are replicated.  No data moves between GPUs.
* N-split: rank r owns columns ``[r*N/g, (r+1)*N/g)`` of the weights, per-N scales, bias
  and dst; src is replicated.  One exchange assembles the full dst on every rank: an
  all-gather of the column slices.

``NSplitMatmul`` runs the N-split with the library's own primitive for the slice, in one
of two ways:

* ``mode="p2p"`` (fused): the full ``(M, N)`` destination lives in symmetric memory (the same
  allocation on every GPU, each mapped into every process); the slice primitive is given
  the other GPUs' mirrors as extra destinations (``DNNL_ARG_B200_DST_PEER``) and its
  epilogue stores every finished tile into all of them over NVLink while the tensor cores
  work on the next tile.  One stream-ordered barrier afterwards tells every rank that all
  slices have landed.  Nothing is ever loaded from another GPU.
* ``mode="nccl"`` (the baseline): slices go to a ``[g][M][N/g]`` staging buffer, one NCCL
  all-gather exchanges them and ``b200_gather_columns_launch`` lays them out as the
  row-major ``(M, N)``.

``gather_columns_host`` is that layout step in numpy, for tests without a GPU.
"""
import numpy as np

from . import dtypes as dt
from .workloads import MatmulCase, shard


def m_split(case: MatmulCase, rank: int, world: int) -> MatmulCase:
    return shard(case, rank, world, "m")


def n_split(case: MatmulCase, rank: int, world: int) -> MatmulCase:
    return shard(case, rank, world, "n")


def gather_columns_host(staged: np.ndarray) -> np.ndarray:
    """``[g][M][N/g]`` (slices in rank order) -> row-major ``(M, N)``."""
    g, m, ns = staged.shape
    return np.ascontiguousarray(np.transpose(staged, (1, 0, 2)).reshape(m, g * ns))


def assemble_rows_host(parts) -> np.ndarray:
    """M-split results in rank order -> the full dst."""
    return np.concatenate(list(parts), axis=0)


SENTINEL = 0xA5  # byte pattern a destination is filled with before a checked execution


class MSplitMatmul:
    """dst rows ``[r*M/g, (r+1)*M/g)`` on rank r: the row shard of ``case`` through the
    library's primitive, weights replicated, nothing exchanged.  ``self.dst`` is a torch byte
    tensor ``(M/g, N * elem)`` holding this rank's rows."""

    def __init__(self, case: MatmulCase, rank: int, world: int, device_index: int):
        import torch
        from . import api
        if case.M % world != 0:
            raise ValueError("M must be a multiple of the number of ranks")
        self.torch, self.api = torch, api
        self.rank, self.world, self.case = rank, world, case
        self.local = m_split(case, rank, world)
        self.eng = api.Engine(index=device_index)
        self.tstream = torch.cuda.current_stream()
        self.strm = api.Stream(self.eng, cuda_stream=self.tstream.cuda_stream)
        self.elem = np.dtype(dt.RAW[case.dst_dt]).itemsize
        self.plan = api.CasePlan(self.local, self.eng, self.strm, weights="any")
        self.dst = torch.empty((self.local.M, case.N * self.elem), dtype=torch.uint8, device="cuda")
        self.args = dict(self.plan.args)
        self.args[api.ARG_DST] = api.Memory(self.plan.mds["dst"], self.eng, handle=self.dst.data_ptr())
        self.rows = slice(rank * self.local.M, (rank + 1) * self.local.M)

    @property
    def impl(self):
        return self.plan.impl

    def execute(self):
        self.plan.prim.execute(self.strm, self.args)


def unsharded_on_this_gpu(case: MatmulCase, device_index: int):
    """The whole problem through the ordinary primitive on this GPU: the yardstick a sharded run
    must equal byte for byte (every dst element is a function of its own row of src and column
    of the weights only).  Returns a torch byte tensor ``(M, N * elem)``."""
    import torch
    from . import api
    eng = api.Engine(index=device_index)
    tstream = torch.cuda.current_stream()
    strm = api.Stream(eng, cuda_stream=tstream.cuda_stream)
    elem = np.dtype(dt.RAW[case.dst_dt]).itemsize
    plan = api.CasePlan(case, eng, strm, weights="any")
    out = torch.empty((case.M, case.N * elem), dtype=torch.uint8, device="cuda")
    if case.dst_init is not None:
        out.copy_(torch.from_numpy(np.ascontiguousarray(case.dst_init).view(np.uint8).reshape(case.M, -1)))
    args = dict(plan.args)
    args[api.ARG_DST] = api.Memory(plan.mds["dst"], eng, handle=out.data_ptr())
    plan.prim.execute(strm, args)
    strm.wait()
    return out


def count_mismatched_elements(got, want, elem: int) -> int:
    """Number of dst elements (of ``elem`` bytes) whose bytes differ between two byte tensors."""
    ne = (got != want)
    if elem > 1:
        ne = ne.view(ne.shape[0], -1, elem).any(dim=2)
    return int(ne.sum().item())


class NSplitMatmul:
    """dst = matmul(src, W) with W's columns split over the ranks of ``group``; after
    ``execute()`` every rank holds the full row-major dst in ``self.dst`` (a torch byte
    tensor ``(M, N * elem)``).  Everything is enqueued on torch's current stream."""

    def __init__(self, case: MatmulCase, rank: int, world: int, device_index: int, group=None, mode="nccl"):
        import torch
        from . import api
        if case.N % world != 0:
            raise ValueError("N must be a multiple of the number of ranks")
        if mode not in ("nccl", "p2p"):
            raise ValueError("mode is 'nccl' or 'p2p'")
        if world - 1 > 7 and mode == "p2p":
            raise ValueError("at most eight ranks")
        self.torch = torch
        self.api = api
        self.rank, self.world, self.group, self.mode = rank, world, group, mode
        self.case = case
        self.local = n_split(case, rank, world)
        self.eng = api.Engine(index=device_index)
        self.tstream = torch.cuda.current_stream()
        self.strm = api.Stream(self.eng, cuda_stream=self.tstream.cuda_stream)
        self.elem = np.dtype(dt.RAW[case.dst_dt]).itemsize
        ns = case.N // world
        if (ns * self.elem) % 16 != 0:
            raise ValueError("a column slice must be a multiple of 16 bytes per row")
        if mode == "nccl" or world == 1:
            self.plan = api.CasePlan(self.local, self.eng, self.strm, weights="any")
            # raw bytes: the collective and the layout kernel move them without looking inside
            self.staged = torch.empty((world, case.M, ns * self.elem), dtype=torch.uint8, device="cuda")
            self.dst = torch.empty((case.M, case.N * self.elem), dtype=torch.uint8, device="cuda")
            # the slice primitive writes straight into this rank's part of the staging buffer
            self.args = dict(self.plan.args)
            self.args[api.ARG_DST] = api.Memory(self.plan.mds["dst"], self.eng, handle=self.staged[rank].data_ptr())
            self.mode = "nccl"
            return
        import os
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        # plain peer mappings are all that is needed here: no NVLink multicast binding
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        self.plan = api.CasePlan(self.local, self.eng, self.strm, weights="any", dst_strides=(case.N, 1))
        self.buf = symm_mem.empty(case.M * case.N * self.elem, dtype=torch.uint8, device=torch.device("cuda", device_index))
        self.hdl = symm_mem.rendezvous(self.buf, group if group is not None else dist.group.WORLD)
        self.dst = self.buf.view(case.M, case.N * self.elem)
        off = rank * ns * self.elem          # this rank's columns, in every copy of dst
        md = self.plan.mds["dst"]
        self.args = dict(self.plan.args)
        self.args[api.ARG_DST] = api.Memory(md, self.eng, handle=self.buf.data_ptr() + off)
        i = 0
        for r in range(world):
            if r != rank:
                self.args[api.ARG_B200_DST_PEER0 + i] = api.Memory(md, self.eng, handle=int(self.hdl.buffer_ptrs[r]) + off)
                i += 1
        self.flag = torch.zeros(1, dtype=torch.int32, device="cuda")

    @property
    def impl(self):
        return self.plan.impl

    def execute(self):
        self.plan.prim.execute(self.strm, self.args)
        if self.mode == "p2p":
            import torch.distributed as dist
            # stream-ordered: when it completes here, every rank's kernel before it has completed,
            # so every slice has been stored into this GPU's copy
            dist.all_reduce(self.flag, group=self.group)
            return
        if self.world > 1:
            import torch.distributed as dist
            dist.all_gather_into_tensor(self.staged.view(-1), self.staged[self.rank].view(-1), group=self.group)
        from . import kernels_abi
        rc = kernels_abi.lib().b200_gather_columns_launch(
            self.staged.data_ptr(), self.dst.data_ptr(), self.case.M, self.case.N, self.world, self.elem,
            self.tstream.cuda_stream)
        if rc != 0:
            raise RuntimeError("b200_gather_columns_launch failed: %d" % rc)

    def result(self) -> np.ndarray:
        self.torch.cuda.synchronize()
        return self.dst.cpu().numpy().view(dt.RAW[self.case.dst_dt]).reshape(self.case.M, self.case.N)
