"""Data-parallel data-plane benchmark: the wgrad GEMM whose epilogue is the gradient reduce-scatter.

Launch with torchrun, one rank per GPU.  For the four weight shapes of a 1B layer it times, on every rank at once,
  local    dW += dy^T x with the accumulate epilogue into local memory (no communication),
  scatter  the same GEMM with the reduce-scatter epilogue: each element is added with ``red.global.add.v4.f32`` into
           the flat gradient buffer of the rank that owns it ((W-1)/W of the tile crosses NVLink),
  remote   the reduce-scatter epilogue with every element owned by the next rank (all of it crosses NVLink),
and reports TFLOP/s, the bytes each rank sends per launch and the roofline fraction: the target time is the slower
of FLOPs / measured sustained cuBLAS rate and bytes / measured peer-copy bandwidth (770 GB/s per direction).

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m gruboros_b200.tools.bench_dp_ops
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ..ops import _lib as L
from ..ops import kernels as K
from ..parallel.comm import PeerGroup
from .bench_ops import peaks

NVLINK_GBS = 770.0
SHAPES = {"gate": (6144, 2048), "out": (2048, 3072), "ff1": (8192, 2048), "ff2": (2048, 8192)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=16376)
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    group = PeerGroup(rank, world, dev)
    _, _, sustained, src = peaks()
    M = a.rows
    res = {}
    for name, (n, k) in SHAPES.items():
        numel = n * k
        buf = group.alloc(f"grad_{name}", numel * 4)
        g = buf.tensor(torch.float32, numel)
        g.zero_()
        ptrs = group.ptrs(f"grad_{name}")
        nxt = [ptrs[(rank + 1) % world]] * world
        dy = torch.randn(M, n, device=dev).bfloat16()
        x = torch.randn(M, k, device=dev).bfloat16()
        sk = 1
        variants = {
            "local": (lambda: K.linear_wgrad(dy, x, g.view(n, k), splitk=sk), 0.0),
            "scatter": (lambda: K.linear_wgrad(dy, x, None, splitk=sk, scatter=(ptrs, numel // world, 0)),
                        numel * 4.0 * sk * (world - 1) / world),
            "remote": (lambda: K.linear_wgrad(dy, x, None, splitk=sk, scatter=(nxt, numel // world, 0)), numel * 4.0 * sk),
        }
        flops = 2.0 * M * n * k
        res[name] = {}
        for vname, (fn, nbytes) in variants.items():
            for _ in range(3):
                fn()
            group.device_barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(a.iters):
                fn()
            e1.record()
            group.device_barrier()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / a.iters
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = t.item()
            target_ms = max(flops / (sustained * 1e9), nbytes / (NVLINK_GBS * 1e6))
            res[name][vname] = {"ms": round(ms, 4), "TFLOPs": round(flops / ms / 1e9, 1), "sent_MB": round(nbytes / 1e6, 1),
                                "nvlink_GBs": round(nbytes / ms / 1e6, 1), f"frac_of_{src}_roofline": round(target_ms / ms, 3)}
        L.check_device_status()
    if rank == 0:
        print(json.dumps({"world": world, "rows": M, "shapes": res}, indent=1))
    dist.barrier()
    group.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
