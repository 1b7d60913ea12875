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
  On GPUs it is a kernel of this library over NVLink peer memory
  (PeerAllReduce: flags + peer loads + the cast in one launch per rank); the
  process group's all_reduce (NCCL / gloo) is the fallback and the checker.

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


class PeerAllReduce:
    """Sum of one fp32 vector per rank over NVLink peer memory
    (plb_allreduce_f32_p2p): every rank writes its vector into its half of a
    symmetric buffer, one kernel per rank exchanges flags with the peers, adds
    all ranks' vectors in rank order and writes the fp32 sum and its half cast.

    The symmetric buffer comes from torch.distributed's symmetric memory (one
    process per GPU, peers mapped through CUDA IPC / fabric handles)."""

    #: inbound bytes per rank ((world - 1) x the vector) from which the
    #: reduce-scatter + all-gather kernel is used.  Below it every rank simply
    #: reads all peers' vectors: the second flag round and the fenced peer stores
    #: cost more than the traffic they save (measured on a 590 KB gradient: 60.2
    #: against 72.2 us per step on 2 GPUs, 69.0 against 76.1 us on 8)
    RS_MIN_BYTES = 8 << 20

    def __init__(self, ctx: capi.Context, count: int, group=None, overlap: bool = False,
                 mode: str = "auto"):
        """mode: "oneshot" (plb_allreduce_f32_p2p: one flag round, every rank
        reads all N vectors), "rs" (plb_allreduce_f32_p2p_rs: each rank sums one
        slice and stores it to all, two flag rounds, 1/N of the traffic) or
        "auto" (rs from RS_MIN_BYTES of inbound traffic on).

        With overlap=True the all-reduce kernel runs on a stream (and library
        context) of its own: it is ordered after the kernels that fill input()
        by an event, and the next step's kernels on the main stream do not wait
        for it -- the exchange over NVLink then hides behind the next layer's
        (or step's) compute.  Consumers of the outputs call wait() first."""
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        if count % 4:
            raise ValueError("element count must be a multiple of 4")
        self.ctx, self.count = ctx, count
        group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        device = torch.device("cuda", torch.cuda.current_device())
        if mode not in ("auto", "oneshot", "rs"):
            raise ValueError(f"unknown all-reduce mode {mode!r}")
        big = (self.world - 1) * count * 4 >= self.RS_MIN_BYTES
        self.mode = ("rs" if big else "oneshot") if mode == "auto" else mode
        # rows 0, 1: input halves, used on alternate steps (in the one-shot form a
        # peer may still read the last one); row 2: the result buffer of the
        # reduce-scatter form, written by the peers
        self.buf = symm_mem.empty((3, count), dtype=torch.float32, device=device)
        self.handle = symm_mem.rendezvous(self.buf, group)
        need = capi.lib().plb_allreduce_p2p_signal_bytes(self.world)
        if self.handle.signal_pad_size < need:
            raise RuntimeError(f"signal pad of {self.handle.signal_pad_size} bytes is smaller than {need}")
        self.buffer_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.signal_ptrs = [int(p) for p in self.handle.signal_pad_ptrs]
        self.epoch = 0
        self.overlap = overlap
        # per half: the view to fill and every rank's address of that half
        self.halves = [self.buf[0], self.buf[1]]
        self.half_ptrs = [[p + h * count * 4 for p in self.buffer_ptrs] for h in (0, 1)]
        self.result_ptrs = [p + 2 * count * 4 for p in self.buffer_ptrs]
        if overlap:
            self.main_stream = torch.cuda.ExternalStream(ctx.stream, device=device)
            self.comm_stream = torch.cuda.Stream(device=device)
            self.comm_ctx = capi.Context(device.index, stream=self.comm_stream.cuda_stream)
            self.filled = [torch.cuda.Event(), torch.cuda.Event()]   # input half written (main stream)
            self.done = [None, None]                                  # all-reduce that read a half (comm stream)

    def input(self):
        """The buffer (a torch view, `count` floats) this rank must fill for the next call."""
        half = (self.epoch + 1) & 1
        if self.overlap:
            # This rank's all-reduce of step e completing only proves that the
            # peers have STARTED theirs.  That a peer has finished reading the
            # half of step e - 1 is known once its flag of step e has arrived,
            # i.e. when this rank's all-reduce of step e (the latest) is done; in
            # the reduce-scatter form the second flag round says it directly.
            # So the main stream waits for the latest all-reduce before it may
            # overwrite the other half.
            for ev in self.done:
                if ev is not None:
                    self.main_stream.wait_event(ev)
        return self.halves[half]

    def run(self, out_f32=None, out_half=None):
        """All ranks call this after filling input(); enqueued on the context's
        stream, or with overlap on the communication stream behind an event."""
        import torch
        self.epoch += 1
        half = self.epoch & 1
        ptrs = self.half_ptrs[half]

        def launch(c):
            if self.mode == "rs":
                c.allreduce_f32_p2p_rs(self.rank, self.world, ptrs, self.result_ptrs, self.signal_ptrs,
                                       self.epoch, self.count, out_f32, out_half)
            else:
                c.allreduce_f32_p2p(self.rank, self.world, ptrs, self.signal_ptrs, self.epoch, self.count,
                                    out_f32, out_half)
        if not self.overlap:
            launch(self.ctx)
            return
        self.filled[half].record(self.main_stream)
        self.comm_stream.wait_event(self.filled[half])
        launch(self.comm_ctx)
        if self.done[half] is None:
            self.done[half] = torch.cuda.Event()
        self.done[half].record(self.comm_stream)

    def wait(self):
        """Orders the main stream after the latest all-reduce (overlap mode)."""
        if self.overlap and self.epoch and self.done[self.epoch & 1] is not None:
            self.main_stream.wait_event(self.done[self.epoch & 1])

    def synchronize(self):
        """Host-side wait for the communication stream; raises if a peer's flag timed out."""
        if self.overlap:
            self.comm_ctx.synchronize()


class FusedPeerWeightUpdate:
    """Buffers of plb_conv_wu_allreduce: the weight-update pass whose split-K
    reduction kernel also adds the peers' gradients, chunk by chunk, over
    NVLink peer memory.  Holds two peer-addressable gradient buffers (used on
    alternate steps: a peer may still be reading the previous step's) and the
    per-chunk flag area, all in torch.distributed's symmetric memory.

    owners=True: every chunk of the gradient is added by one rank and fetched
    by the others from a third peer-addressable buffer
    (plb_conv_wu_allreduce_owners): less NVLink traffic per rank, one more flag
    per chunk.  None picks it from OWNERS_MIN_WORLD ranks on."""

    #: ranks from which the sum is shared out by default.  Measured on one box
    #: of B200s (590 KB gradient): 59.5 against 56.6 us per step on 2 GPUs, 62.1
    #: against 62.3 us on 8, so up to 8 ranks every rank adds everything
    OWNERS_MIN_WORLD = 9

    def __init__(self, ctx: capi.Context, params: capi.ConvParams, count: int, group=None, owners=None):
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        group = group if group is not None else dist.group.WORLD
        self.ctx, self.params, self.count = ctx, params, count
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        flag_bytes = int(capi.lib().plb_conv_wu_allreduce_flag_bytes(params))
        if flag_bytes == 0 or count % 4:
            raise ValueError("this layer has no fused weight update (see plb_conv_wu_allreduce)")
        device = torch.device("cuda", torch.cuda.current_device())
        self.owners = self.world >= self.OWNERS_MIN_WORLD if owners is None else bool(owners)
        self.grads = symm_mem.empty((3 if self.owners else 2, count), dtype=torch.float32, device=device)
        grads_handle = symm_mem.rendezvous(self.grads, group)
        self.flags = symm_mem.empty((flag_bytes // 4,), dtype=torch.int32, device=device)
        self.flags.zero_()
        flags_handle = symm_mem.rendezvous(self.flags, group)
        torch.cuda.synchronize()
        dist.barrier(group)          # every rank's flags are zero before anyone's first step
        self._handles = (grads_handle, flags_handle)
        base = [int(v) for v in grads_handle.buffer_ptrs]
        self.grad_ptrs = [[v + h * count * 4 for v in base] for h in (0, 1)]
        self.result_ptrs = [v + 2 * count * 4 for v in base] if self.owners else None
        self.flag_ptrs = [int(v) for v in flags_handle.buffer_ptrs]
        self.epoch = 0
        self.mode, self.overlap = "fused", False

    def wu(self, x_local, dy_local, dw, dw_f32, opt=None):
        self.epoch += 1
        self.ctx.conv_wu_allreduce(self.params, x_local, dy_local, self.rank, self.world,
                                   self.grad_ptrs[self.epoch & 1], self.flag_ptrs, self.epoch, dw, dw_f32,
                                   opt=opt, result_ptrs=self.result_ptrs)

    def wait(self):
        pass

    def synchronize(self):
        pass


class ShardedConv:
    """One rank's part of a batch-sharded convolution layer."""

    def __init__(self, ctx: capi.Context, make_kwargs: dict, rank: int = 0, world: int = 1,
                 group=None, opt: Optional[capi.ConvOptions] = None, peer_allreduce: bool = False,
                 overlap_allreduce: bool = False, allreduce_mode: str = "auto"):
        self.ctx, self.rank, self.world, self.group, self.opt = ctx, rank, world, group, opt
        self.params, self.begin, self.end = local_conv_params(make_kwargs, rank, world)
        self.global_batch = int(make_kwargs["batch"])
        # the all-reduce over peer memory needs GPUs that can address one another
        self.peer = None
        if peer_allreduce and world > 1:
            p = self.params
            count = int(p.groups) * int(p.out_chans_per_group) * int(p.in_chans_per_group)
            for i in range(p.num_field_dims):
                count *= int(p.kernel[i])
            # "fused" (and "auto" where the layer allows it): the sum over ranks
            # happens inside the weight update's own reduction kernel
            self.fused = None
            if allreduce_mode in ("auto", "fused", "fused_all", "fused_owners") and not overlap_allreduce:
                owners = {"fused_all": False, "fused_owners": True}.get(allreduce_mode)
                try:
                    self.fused = FusedPeerWeightUpdate(ctx, p, count, group, owners=owners)
                except ValueError:
                    if allreduce_mode != "auto":
                        raise
            if self.fused is not None:
                self.peer = self.fused
            else:
                self.peer = PeerAllReduce(ctx, count, group, overlap=overlap_allreduce,
                                          mode="auto" if allreduce_mode.startswith("fused") else allreduce_mode)

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
        if self.peer is not None and self.peer.mode == "fused":
            self.peer.wu(x_local, dy_local, dw, dw_f32, opt=self.opt)
            return
        if self.peer is not None:
            # local gradient straight into this step's half of the symmetric
            # buffer; one kernel then sums all ranks' halves and casts
            mine = self.peer.input()
            if self.params.batch:
                self.ctx.conv_wu(self.params, x_local, dy_local, None, mine, opt=self.opt)
            else:
                self.ctx.memset(mine, 0, mine.numel() * 4)
            self.peer.run(dw_f32, dw)
            return
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
