"""Multi-GPU check of the ring and shard launchers, one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \\
        --master-port 29511 tests/multi_gpu_ring_check.py [--seq-len 16384]

Every rank builds the same seeded full tensors, keeps its zig-zag shard, runs the NCCL ring and
compares its rows with the single-launch kernel on the full sequence (and rank 0 additionally with
the CPU oracle on sampled rows).  Shard mode: every rank computes its (batch x KV-head) units and
the all-gathered result is compared with the full computation.  Prints one line per rank and exits
non-zero on a mismatch.  tests/test_parallel_gpu.py launches it when the box has two GPUs or more.
"""
import argparse
import os
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "mini-attention_b200"))

import torch
import torch.distributed as dist

import miniattn
from miniattn import parallel as par


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--seq-len", type=int, default=16384)
    args = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    ok = True
    hp_group = par.ring_process_group()   # the launcher's high-priority group; the default group is used too
    for dtype, tol in ((torch.float16, 2e-3), (torch.bfloat16, 1e-2)):
        g = torch.Generator().manual_seed(7)
        N, H, D = args.seq_len, 4, 128
        q = torch.randn(1, H, N, D, generator=g).to(dtype).to(dev)
        k = torch.randn(1, H, N, D, generator=g).to(dtype).to(dev)
        v = torch.randn(1, H, N, D, generator=g).to(dtype).to(dev)
        full = miniattn.flash_attn_fwd(q, k, v, causal=True)
        qs, ks, vs = (par.zigzag_split(t, world)[rank].contiguous() for t in (q, k, v))
        out = par.ring_forward(qs, ks, vs, causal=True, rank=rank, world=world, verify_origin=True)
        err = (out.float() - par.zigzag_split(full, world)[rank].float()).abs().max().item()
        # the two-launch form (16-bit partials + merge kernel) over the same ring
        out2 = par.ring_forward(qs, ks, vs, causal=True, rank=rank, world=world, fused=False, group=hp_group)
        err = max(err, (out2.float() - par.zigzag_split(full, world)[rank].float()).abs().max().item())
        line = f"rank {rank}/{world} ring {dtype}: max|ring - single| = {err:.3e}"
        if rank == 0:
            from oracle.attention_oracle import attention_reference_rows
            L = N // (2 * world)
            rows = torch.tensor(sorted({0, 1, L - 1, N - L, N - 1} | set(range(N - L + 5, N, max(1, L // 16)))))
            loc = torch.tensor([r if r < L else L + (r - (N - L)) for r in rows.tolist()])
            ref = attention_reference_rows(q.cpu(), k.cpu(), v.cpu(), rows, causal=True)
            e2 = (out[:, :, loc].float().cpu() - ref).abs().max().item()
            line += f"; vs CPU oracle rows = {e2:.3e}"
            err = max(err, e2)
        ok &= err <= tol
        print(line, flush=True)
        # shard mode: GQA, 2 KV heads per batch element x 4 batch elements
        qg = torch.randn(4, 8, 1024, D, generator=g).to(dtype).to(dev)
        kg = torch.randn(4, 2, 1024, D, generator=g).to(dtype).to(dev)
        vg = torch.randn(4, 2, 1024, D, generator=g).to(dtype).to(dev)
        mine = torch.zeros_like(qg)
        par.sharded_forward(qg, kg, vg, causal=True, rank=rank, world=world, out=mine)
        dist.all_reduce(mine)  # units are disjoint and the rest is zero: the sum assembles them
        errs = (mine.float() - miniattn.flash_attn_fwd(qg, kg, vg, causal=True).float()).abs().max().item()
        ok &= errs <= tol
        print(f"rank {rank}/{world} shard {dtype}: max|sharded - full| = {errs:.3e}", flush=True)
    status = miniattn.device_status(dev)
    ok &= status == 0
    flag = torch.tensor([0 if ok else 1], device=dev)
    dist.all_reduce(flag)
    dist.destroy_process_group()
    if int(flag.item()) != 0:
        print(f"rank {rank}: FAILED (status word {status})", flush=True)
        sys.exit(1)
    if rank == 0:
        print("multi-GPU check passed", flush=True)


if __name__ == "__main__":
    main()
