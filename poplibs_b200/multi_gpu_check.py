"""Self-check of the sharded path on several GPUs of one box.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N \\
        --master-addr 127.0.0.1 --master-port P -m poplibs_b200.multi_gpu_check

Every rank draws the same global problem (seeded +-1 data, so all sums are
exact), runs its batch shard of the forward, backward and weight-update
passes and its row shard of a matrix product through the library, and the
pieces are compared with the same passes run unsharded on rank 0:

* forward / backward / matMul: the shards, gathered, must equal the
  unsharded result bit for bit (no communication is involved);
* weight update: the gradient summed over the ranks by the library's
  all-reduce kernel over NVLink peer memory must be identical on all ranks,
  equal to the unsharded gradient, and equal to what the process group's own
  all-reduce (NCCL) gives.

Rank 0 prints one line per check and exits non-zero on a mismatch.
"""
from __future__ import annotations

import os
import sys

import torch
import torch.distributed as dist

from . import capi, parallel


def main() -> int:
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=device)
    stream = torch.cuda.Stream(device=device)
    ctx = capi.Context(local_rank, stream=stream.cuda_stream)
    ok = True

    def report(name, good):
        nonlocal ok
        flag = torch.tensor([1 if good else 0], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        good = bool(flag.item())
        ok &= good
        if rank == 0:
            print(f"{name}: {'ok' if good else 'MISMATCH'}", flush=True)

    g = torch.Generator().manual_seed(7)   # same data on every rank
    pm1 = lambda *shape: (torch.randint(0, 2, shape, generator=g) * 2 - 1).half()  # noqa: E731
    batch = 4 * world + 1                  # an uneven split
    kw = dict(batch=batch, field=[12, 12], kernel=[3, 3], in_chans=64, out_chans=72, padding=1)
    x, w = pm1(batch, 12, 12, 64).to(device), pm1(3, 3, 72, 64).to(device)
    dy = pm1(batch, 12, 12, 72).to(device)
    full = capi.ConvParams.make(**kw)
    sh = parallel.ShardedConv(ctx, kw, rank, world, peer_allreduce=True, allreduce_mode="oneshot")
    sh_rs = parallel.ShardedConv(ctx, kw, rank, world, peer_allreduce=True, allreduce_mode="rs")
    sh_fu = parallel.ShardedConv(ctx, kw, rank, world, peer_allreduce=True, allreduce_mode="fused_all")
    sh_ow = parallel.ShardedConv(ctx, kw, rank, world, peer_allreduce=True, allreduce_mode="fused_owners")
    b, e = sh.begin, sh.end
    with torch.cuda.stream(stream):
        # unsharded reference (every rank computes it; cheap)
        y_ref = torch.empty(batch, 12, 12, 72, dtype=torch.float16, device=device)
        dx_ref = torch.empty(batch, 12, 12, 64, dtype=torch.float16, device=device)
        dw_ref = torch.empty(3, 3, 72, 64, dtype=torch.float32, device=device)
        ctx.conv_fwd(full, x, w, y_ref)
        ctx.conv_bwd(full, dy, w, dx_ref)
        ctx.conv_wu(full, x, dy, None, dw_ref)
        # this rank's shard
        y = torch.empty(e - b, 12, 12, 72, dtype=torch.float16, device=device)
        dx = torch.empty(e - b, 12, 12, 64, dtype=torch.float16, device=device)
        sh.fwd(x[b:e].contiguous(), w, y)
        sh.bwd(dy[b:e].contiguous(), w, dx)
        dw16 = torch.empty(3, 3, 72, 64, dtype=torch.float16, device=device)
        dw32 = torch.empty(3, 3, 72, 64, dtype=torch.float32, device=device)
        rs16, rs32 = torch.empty_like(dw16), torch.empty_like(dw32)
        fu16, fu32 = torch.empty_like(dw16), torch.empty_like(dw32)
        ow16, ow32 = torch.empty_like(dw16), torch.empty_like(dw32)
        for _ in range(20):                # many steps: both buffer halves, growing epochs
            sh.wu(x[b:e].contiguous(), dy[b:e].contiguous(), dw16, dw32)
            sh_rs.wu(x[b:e].contiguous(), dy[b:e].contiguous(), rs16, rs32)
            sh_fu.wu(x[b:e].contiguous(), dy[b:e].contiguous(), fu16, fu32)
            sh_ow.wu(x[b:e].contiguous(), dy[b:e].contiguous(), ow16, ow32)
        # the same sum by the process group's all-reduce
        local = torch.empty_like(dw32)
        ctx.conv_wu(sh.params, x[b:e].contiguous(), dy[b:e].contiguous(), None, local)
    ctx.synchronize()
    torch.cuda.synchronize()
    dist.all_reduce(local)
    report("forward shards equal the unsharded rows", torch.equal(y, y_ref[b:e]))
    report("backward shards equal the unsharded rows", torch.equal(dx, dx_ref[b:e]))
    report("weight gradient over peer memory equals the unsharded gradient", torch.equal(dw32, dw_ref))
    report("weight gradient over peer memory equals the NCCL sum", torch.equal(dw32, local))
    report("half cast of the gradient", torch.equal(dw16, dw_ref.half()))
    report("reduce-scatter + all-gather form: same bits, fp32 and half",
           torch.equal(rs32, dw32) and torch.equal(rs16, dw16))
    first = dw32.clone()
    dist.broadcast(first, 0)
    report("all ranks hold identical bits", torch.equal(first, dw32))

    # the same with the all-reduce on a stream of its own, several steps in flight
    report("sum over ranks fused into the split-K reduction: same bits, fp32 and half",
           torch.equal(fu32, dw32) and torch.equal(fu16, dw16))
    report("the same with every chunk added by one owner rank: same bits, fp32 and half",
           torch.equal(ow32, dw32) and torch.equal(ow16, dw16))
    # different, non-integer data on every rank: the order of additions now matters,
    # and all three forms must give the per-rank gradients added in rank order
    gr = torch.Generator().manual_seed(100 + rank)
    xr = (torch.rand(e - b, 12, 12, 64, generator=gr) * 2 - 1).half().to(device)
    dyr = (torch.rand(e - b, 12, 12, 72, generator=gr) * 2 - 1).half().to(device)
    with torch.cuda.stream(stream):
        mine = torch.empty_like(dw32)
        ctx.conv_wu(sh.params, xr, dyr, None, mine)
        outs3 = []
        for s3 in (sh, sh_rs, sh_fu, sh_ow):
            o16, o32 = torch.empty_like(dw16), torch.empty_like(dw32)
            s3.wu(xr, dyr, o16, o32)
            outs3.append((o16, o32))
    ctx.synchronize()
    torch.cuda.synchronize()
    parts = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(parts, mine)
    ordered = parts[0].clone()
    for part in parts[1:]:
        ordered += part
    report("uniform data: one-shot, reduce-scatter and both fused sums equal the rank-order sum, fp32 and half",
           all(torch.equal(o32, ordered) and torch.equal(o16, ordered.half()) for o16, o32 in outs3))
    for mode in ("oneshot", "rs"):
        sho = parallel.ShardedConv(ctx, kw, rank, world, peer_allreduce=True, overlap_allreduce=True,
                                   allreduce_mode=mode)
        outs = [(torch.empty_like(dw16), torch.empty_like(dw32)) for _ in range(5)]
        with torch.cuda.stream(stream):
            for o16, o32 in outs:
                sho.wu(x[b:e].contiguous(), dy[b:e].contiguous(), o16, o32)
            sho.peer.wait()
        ctx.synchronize()
        sho.peer.synchronize()
        torch.cuda.synchronize()
        report(f"all-reduce ({mode}) on a stream of its own, five steps enqueued",
               all(torch.equal(o32, dw_ref) and torch.equal(o16, dw_ref.half()) for o16, o32 in outs))

    m, k, n = 64 * world + 32, 256, 192
    a, bm = pm1(m, k).to(device), pm1(k, n).to(device)
    mm = parallel.ShardedMatMul(ctx, m, k, n, rank, world)
    with torch.cuda.stream(stream):
        c_ref = torch.empty(m, n, dtype=torch.float16, device=device)
        ctx.matmul(capi.MatmulDesc.make(m, k, n), a, bm, None, c_ref)
        c = torch.empty(mm.end - mm.begin, n, dtype=torch.float16, device=device)
        mm.run(a[mm.begin:mm.end].contiguous(), bm, None, c)
    ctx.synchronize()
    torch.cuda.synchronize()
    report("matMul row shards equal the unsharded rows", torch.equal(c, c_ref[mm.begin:mm.end]))
    dist.barrier()
    dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
