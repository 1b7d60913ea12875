"""Data-parallel use of the contraction path on one multi-GPU box.

One process per GPU (torch.distributed; NCCL over NVLink on GPUs, gloo in the
CPU tests).  The path shards without communication except in one place:

* convolution forward / backward: each rank owns a contiguous slice of the
  batch; weights are replicated; outputs stay sharded.
* matMul: each rank owns a contiguous slice of the rows of A (and of C); B is
  replicated.
* convolution weight update: each rank reduces its batch slice to a full-size
  fp32 weight gradient; ONE all-reduce (sum) makes it the gradient of the whole
  batch, which is then cast to the weights' type.  This is the only collective.

The reference has no counterpart: it spreads one convolution over the tiles of
several IPUs inside a single graph (lib/poplin/ConvPlan.hpp:28-77).
"""
from __future__ import annotations

from typing import Optional, Tuple

from . import capi


def shard_range(total: int, rank: int, world: int) -> Tuple[int, int]:
    """[begin, end) of the slice `rank` owns when `total` units are dealt out as
    evenly as possible, in order, to `world` ranks."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    base, extra = divmod(total, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def local_conv_params(make_kwargs: dict, rank: int, world: int) -> Tuple[capi.ConvParams, int, int]:
    """ConvParams of this rank's batch slice of the convolution described by
    `make_kwargs` (the keyword arguments of capi.ConvParams.make, global batch)."""
    begin, end = shard_range(int(make_kwargs["batch"]), rank, world)
    kw = dict(make_kwargs)
    kw["batch"] = end - begin
    return capi.ConvParams.make(**kw), begin, end


def allreduce_weight_grads(dw_f32, group=None):
    """Sums the per-rank fp32 weight gradients in place across the process
    group (a no-op for a single process)."""
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(dw_f32, op=dist.ReduceOp.SUM, group=group)
    return dw_f32


class ShardedConv:
    """One rank's part of a batch-sharded convolution layer."""

    def __init__(self, ctx: capi.Context, make_kwargs: dict, rank: int = 0, world: int = 1,
                 group=None, opt: Optional[capi.ConvOptions] = None):
        self.ctx, self.rank, self.world, self.group, self.opt = ctx, rank, world, group, opt
        self.params, self.begin, self.end = local_conv_params(make_kwargs, rank, world)
        self.global_batch = int(make_kwargs["batch"])

    def fwd(self, x_local, w, y_local, bias=None):
        if self.params.batch:
            self.ctx.conv_fwd(self.params, x_local, w, y_local, bias=bias, opt=self.opt)

    def bwd(self, dy_local, w, dx_local):
        if self.params.batch:
            self.ctx.conv_bwd(self.params, dy_local, w, dx_local, opt=self.opt)

    def wu(self, x_local, dy_local, dw, dw_f32):
        """dw (weights' type) and dw_f32 receive the gradient of the WHOLE batch
        on every rank.  dw_f32 is a torch tensor on the context's device."""
        import torch
        if self.params.batch:
            self.ctx.conv_wu(self.params, x_local, dy_local, None, dw_f32, opt=self.opt)
        else:
            dw_f32.zero_()
        if self.world > 1:
            # The kernels ran on the context's stream; the collective is enqueued
            # on torch's current stream.  If they are the same stream everything
            # is already ordered, otherwise fence on both sides.
            shared = self.ctx.stream == torch.cuda.current_stream().cuda_stream
            if not shared:
                self.ctx.synchronize()
            allreduce_weight_grads(dw_f32, self.group)
            if not shared:
                torch.cuda.current_stream().synchronize()
        self.ctx.cast_from_f32(self.params.input_type, dw, dw_f32, dw_f32.numel())


class ShardedMatMul:
    """One rank's rows of A and C of a row-sharded matrix product."""

    def __init__(self, ctx: capi.Context, m: int, k: int, n: int, rank: int = 0, world: int = 1, **desc_kwargs):
        self.ctx = ctx
        self.begin, self.end = shard_range(m, rank, world)
        self.desc = capi.MatmulDesc.make(self.end - self.begin, k, n, **desc_kwargs)

    def run(self, a_local, b, c_local, d_local):
        if self.end > self.begin:
            self.ctx.matmul(self.desc, a_local, b, c_local, d_local)
