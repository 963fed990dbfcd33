"""Data-parallel training step of one of the benchmark models (default
ResNet-50: synthetic 224x224x3 images, bf16 autocast, SGD, 161 f32 gradients
averaged over the ranks; also vgg16, bert-base, bert-large on synthetic token
ids of length --seq).

    torchrun --nproc-per-node N -m stdml_collective_experimental_b200.benchmarks.resnet50_dp \
        [--model resnet50] [--batch 256] [--seq 128] [--steps 10] [--warmup 3] \
        [--mode ours|nccl|local|all]

modes: `ours` = DataParallel of this package (gradients live in the symmetric
heap, fused in-place all-reduce with the 1/N scale, launched from autograd hooks
and overlapped with backward); `nccl` = torch DistributedDataParallel over NCCL;
`local` = no communication (the compute floor).  Prints one JSON line per mode
with the step time (CUDA events, max over ranks) and images/s of the whole job.
"""
import argparse
import json
import os

import torch
import torch.distributed as dist

from .. import DeviceSession
from ..models.resnet import ResNet50
from ..parallel.ddp import DataParallel


def make_workload(args, rank, dev):
    """(model, inputs, targets, loss(model_output, targets)) for --model."""
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    if args.model in ("resnet50", "vgg16"):
        if args.model == "resnet50":
            model = ResNet50()
        else:
            from ..models.vgg import VGG16
            model = VGG16()
        model = model.to(dev).to(memory_format=torch.channels_last)
        x = torch.randn(args.batch, 3, 224, 224, device=dev, generator=g).to(
            memory_format=torch.channels_last)
        y = torch.randint(0, 1000, (args.batch,), device=dev, generator=g)
        return model, x, y, torch.nn.CrossEntropyLoss()
    if args.model in ("bert-base", "bert-large"):
        from ..models.bert import bert_base, bert_large
        model = (bert_base() if args.model == "bert-base" else bert_large()).to(dev)
        x = torch.randint(0, 30522, (args.batch, args.seq), device=dev, generator=g)
        y = torch.randint(0, 2, (args.batch,), device=dev, generator=g)

        def loss(out, target):  # every parameter takes part: sequence output and pooler
            seq, pooled = out
            return torch.nn.functional.cross_entropy(pooled[:, :2].float(), target) + \
                seq.float().pow(2).mean()
        return model, x, y, loss
    raise SystemExit(f"unknown --model {args.model}")


def run_mode(mode, args, sess, rank, world, dev):
    torch.manual_seed(0)
    model, x, y, loss_fn = make_workload(args, rank, dev)
    opt_target = model
    ddp = None
    if mode == "ours":
        ddp = DataParallel(model, sess, buckets=args.buckets)
        opt_target = ddp
    elif mode == "nccl" and world > 1:
        model = torch.nn.parallel.DistributedDataParallel(model, device_ids=[dev.index],
                                                          gradient_as_bucket_view=True)
        opt_target = model
    opt = torch.optim.SGD(opt_target.parameters(), lr=0.01, momentum=0.9)

    def step():
        if ddp is not None:
            ddp.zero_grad()
        else:
            opt.zero_grad(set_to_none=False)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = loss_fn(opt_target(x), y)
        loss.backward()
        opt.step()
        return loss

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        loss = step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    if ddp is not None:
        sess.check()
    out = {"mode": mode, "model": args.model, "n_gpus": world, "batch_per_gpu": args.batch,
           "ms_per_step": ms, "images_per_s": world * args.batch / (ms * 1e-3), "loss": float(loss)}
    if args.model.startswith("bert"):
        out["seq_len"] = args.seq
        out["tokens_per_s"] = world * args.batch * args.seq / (ms * 1e-3)
        del out["images_per_s"]
    if ddp is not None:
        ddp.close()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="resnet50",
                    choices=["resnet50", "vgg16", "bert-base", "bert-large"])
    ap.add_argument("--seq", type=int, default=128)
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--buckets", type=int, default=4)
    ap.add_argument("--mode", default="all")
    args = ap.parse_args()
    rank, world, local = (int(os.environ.get(k, d)) for k, d in
                          (("RANK", 0), ("WORLD_SIZE", 1), ("LOCAL_RANK", 0)))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    # the gradients of the model live in the symmetric heap (f32), plus slack
    from ..models.gradsets import gradset_sizes
    heap = max(256 << 20, 4 * sum(gradset_sizes(args.model)) + (128 << 20))
    sess = DeviceSession.from_env(heap_bytes=heap, rank=rank, world=world, device=local)
    modes = ["local", "nccl", "ours"] if args.mode == "all" else [args.mode]
    for mode in modes:
        res = run_mode(mode, args, sess, rank, world, dev)
        if rank == 0:
            print(json.dumps(res), flush=True)
    sess.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
