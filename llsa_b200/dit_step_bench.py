"""One training step of the rope-DiT-S with llsa_l2 attention, timed -- BASELINE config "full pixel-space rope-DiT-S
training step": 12 blocks, hidden 384, 6 x 64 heads, MLP 1536, 128 x 128 x 3 synthetic images ~ U(-1, 1), timesteps
~ U{0..999}, noise-prediction MSE loss, bf16 autocast over fp32 parameters, AdamW, 8 images per GPU, data-parallel
(DistributedDataParallel over NCCL, gradient all-reduce) when launched with torchrun.

    python -m llsa_b200.dit_step_bench [--steps 10 --warmup 3 --batch 8 --layers 12 --attn sparse_l2]
    torchrun --nproc-per-node 8 -m llsa_b200.dit_step_bench --gpus 8

Prints one JSON line: images/s over all ranks (CUDA events around K steps, max over ranks), ms per step, and the share of
the step spent inside the llsa operators (CUDA events around every attention call of one extra, untimed step).
"""
import argparse
import json
import os

import torch
import torch.distributed as dist
import torch.nn.functional as F

from .dit import RopeDiT


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=12)
    ap.add_argument("--size", type=int, default=128)
    ap.add_argument("--attn", default="sparse_l2", choices=["pixel", "sparse_l1", "sparse_l2"])
    ap.add_argument("--unfused-rope", action="store_true")
    args = ap.parse_args()
    rank, world, local = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(1234)
    model = RopeDiT(layers=args.layers, sample_size=args.size, attn_type=args.attn, fused_rope=not args.unfused_rope).to(dev)
    net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local]) if world > 1 else model
    opt = torch.optim.AdamW(net.parameters(), lr=1e-4, fused=True)
    g = torch.Generator(device=dev).manual_seed(100 + rank)

    def step():
        x0 = torch.rand(args.batch, 3, args.size, args.size, device=dev, generator=g) * 2 - 1
        noise = torch.randn(x0.shape, device=dev, generator=g)
        t = torch.randint(0, 1000, (args.batch,), device=dev, generator=g)
        a = torch.cos(t.float() * (3.14159265 / 2000.0))[:, None, None, None]          # a simple variance-preserving schedule
        xt = a * x0 + torch.sqrt(1 - a * a) * noise
        with torch.autocast("cuda", dtype=torch.bfloat16):
            pred = net(xt, t)
        loss = F.mse_loss(pred.float(), noise)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        return loss

    for _ in range(max(args.warmup, 3)):
        loss = step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        loss = step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t_ = torch.tensor([ms], device=dev)
        dist.all_reduce(t_, op=dist.ReduceOp.MAX)
        ms = float(t_.item())
    ms_step = ms / args.steps

    # share of one step inside the llsa operators (forward + backward kernels between the stage marks)
    share = None
    if args.attn != "pixel":
        from . import ops
        marks = []

        def hook(name):
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            marks.append((name, ev))

        ops.set_stage_hook(hook)
        step()
        ops.set_stage_hook(None)
        torch.cuda.synchronize()
        inside = sum(ev.elapsed_time(nxt) for (name, ev), (_, nxt) in zip(marks[:-1], marks[1:]) if name != "end")
        share = inside / ms_step
    if rank == 0:
        print(json.dumps(dict(metric="rope-DiT-S training step, images/s", value=world * args.batch / (ms_step * 1e-3), unit="images/s",
                              n_gpus=world, steps=args.steps, warmup=max(args.warmup, 3), ms_per_step=ms_step, higher_is_better=True,
                              scaling="weak", dtype="bf16 autocast, fp32 parameters", data="synthetic", loss=float(loss),
                              llsa_share_of_step=share,
                              config=dict(model="rope-DiT-S", layers=args.layers, hidden=384, heads=6, tokens=args.size * args.size,
                                          attention=args.attn, fused_rope=not args.unfused_rope, images_per_gpu=args.batch,
                                          parallelism="ddp%d" % world))), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
