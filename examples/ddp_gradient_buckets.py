"""Data-parallel training step with gradient buckets: the use of an allreduce
library that the reference's README names (README.md:3-9) and leaves to the
framework on top.

Every rank holds a copy of a small MLP, computes gradients on its own shard of
a synthetic batch, averages them over the ranks through
`allreduce_proto_b200.GradientBuckets` (gradients live in flat buckets,
`param.grad` are views, the 1/N scale is fused into the reduction) and takes an
SGD step.  With `--sharded` the averaging is a reduce-scatter, every rank
updates only its block of the flat parameters, and an all-gather puts the
parameters together again (the ZeRO-1 pattern).  With `--overlap` the allreduce
of a bucket starts from an autograd hook while backward is still running.  At the end the ranks compare
a checksum of their parameters: they must agree.

    python -m torch.distributed.run --nproc-per-node 8 examples/ddp_gradient_buckets.py
    python -m torch.distributed.run --nproc-per-node 2 examples/ddp_gradient_buckets.py --device cpu --sharded

On `--device cpu` the tensors live on the host and travel over the library's
shared-memory transport (torch.distributed is only used for the rendezvous).
"""
from __future__ import annotations

import argparse
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

import allreduce_proto_b200 as ar  # noqa: E402


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu", choices=["cpu", "cuda"])
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--sharded", action="store_true", help="reduce-scatter + sharded update + all-gather")
    ap.add_argument("--overlap", action="store_true",
                    help="start a bucket's allreduce from an autograd hook as soon as its gradients are complete")
    ap.add_argument("--hidden", type=int, default=256)
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    if args.device == "cuda":
        torch.cuda.set_device(local_rank)
        device = torch.device("cuda", local_rank)
        dist.init_process_group("nccl", device_id=device)
    else:
        device = torch.device("cpu")
        dist.init_process_group("gloo")
    comm = ar.Communicator.from_torch_distributed()

    torch.manual_seed(0)  # the same initial weights everywhere
    model = torch.nn.Sequential(torch.nn.Linear(64, args.hidden), torch.nn.ReLU(), torch.nn.Linear(args.hidden, args.hidden),
                                torch.nn.ReLU(), torch.nn.Linear(args.hidden, 10)).to(device)
    params = list(model.parameters())
    lr = 0.05

    # Gradients: views into flat buckets (symmetric memory on GPUs, so the collectives run in place).
    grads = ar.GradientBuckets([p.shape for p in params], device=device, comm=comm, bucket_bytes=256 << 10,
                               symmetric=args.device == "cuda", shardable=args.sharded)
    if args.overlap and not args.sharded:
        grads.overlap_with_backward(params, average=True)
    else:
        grads.attach(params)
    weights = None
    if args.sharded:
        # Parameters in the same flat layout, so that block r of a bucket is rank r's share of the weights.
        weights = ar.GradientBuckets([p.shape for p in params], device=device, comm=comm, bucket_bytes=256 << 10,
                                     symmetric=args.device == "cuda", shardable=True)
        weights.load([p.data for p in params])
        for p, v in zip(params, weights.views):
            p.data = v

    gen = torch.Generator(device="cpu").manual_seed(1000 + rank)  # every rank its own shard of the batch
    for step in range(args.steps):
        x = torch.randn(32, 64, generator=gen).to(device)
        y = torch.randint(0, 10, (32,), generator=gen).to(device)
        grads.zero_()
        loss = torch.nn.functional.cross_entropy(model(x), y)
        loss.backward()
        if args.sharded:
            my_grads = grads.reduce_scatter(average=True, sync=True)
            for w, g in zip(weights.shards(), my_grads):
                w.add_(g, alpha=-lr)          # this rank's block of the weights only
            weights.all_gather(sync=True)
        else:
            if args.overlap:
                grads.finish()                # the collectives were started during backward
            else:
                grads.allreduce(average=True, sync=True)
            with torch.no_grad():
                for p in params:
                    p.add_(p.grad, alpha=-lr)
        if rank == 0:
            print(f"step {step}: loss of rank 0 = {loss.item():.4f}")

    # The ranks must hold the same weights: the sum of a checksum equals N times the local one.  (An
    # allreduce needs at least as many elements as ranks, a rule kept from the reference: one value per tensor.)
    checksum = torch.stack([p.detach().double().sum() for p in params]).cpu()
    checksum = torch.cat([checksum, torch.zeros(max(0, world - checksum.numel()), dtype=torch.float64)])
    total = checksum.clone()
    comm.allreduce(total)
    ok = bool(torch.allclose(total, checksum * world, rtol=1e-9, atol=1e-9))
    print(f"rank {rank}: {'OK' if ok else 'FAIL'} (checksum {checksum.sum().item():.6f})")
    comm.close()
    dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
