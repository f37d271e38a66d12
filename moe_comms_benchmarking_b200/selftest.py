"""Multi-GPU self-test of the tensor-parallel style collectives (uniform all-gather, uniform
reduce-scatter, fused reduce-scatter + residual + RMSNorm + all-gather) on the real transport.

    torchrun --nproc_per_node=N -m moe_comms_benchmarking_b200.selftest [--transport p2p]

The reference vendors these operations but never calls or checks them
(nvls/torch_symm_triton/collectives.py, fused_collectives.py); here every rank compares its
result with a plain PyTorch computation on data that all ranks can regenerate from seeds.
Prints ``[PASS]/[FAIL]`` lines like the driver's ``--validate`` and exits 0/1.
"""
from __future__ import annotations

import argparse
import sys

import torch
import torch.distributed as dist


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--transport", choices=["auto", "multimem", "p2p"], default="auto")
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--rows", type=int, default=96, help="rows per rank")
    args = ap.parse_args(argv)
    from .ops import oracle
    from .ops.dense import UniformAllGatherPlan, UniformReduceScatterPlan
    from .ops.norm import RsAddNormAgPlan
    from .parallel.dist import init_distributed
    from .parallel.symm_heap import SymmetricHeap
    group, rank, world, lr = init_distributed()
    dev = torch.device("cuda", lr)
    H, R = args.hidden, args.rows
    heap = SymmetricHeap(group, 64 << 20, dev, transport=args.transport)
    results = []

    def data(seed, shape, dtype=torch.bfloat16):
        g = torch.Generator(device=dev).manual_seed(seed)
        return torch.randn(*shape, device=dev, generator=g).to(dtype)

    # uniform all-gather of three tensors with one barrier
    srcs = [data(100 + rank, (R, H)), data(200 + rank, (R, 24), torch.float32),
            torch.arange(R * 6, device=dev, dtype=torch.int64).view(R, 6) + rank * 10000]
    dsts = [heap.alloc(f"ag{i}", [R * world, *s.shape[1:]], s.dtype) for i, s in enumerate(srcs)]
    UniformAllGatherPlan(heap, dsts, srcs).launch()
    torch.cuda.synchronize()
    dist.barrier(group)
    want = [torch.cat([data(100 + r, (R, H)) for r in range(world)]),
            torch.cat([data(200 + r, (R, 24), torch.float32) for r in range(world)]),
            torch.cat([torch.arange(R * 6, device=dev, dtype=torch.int64).view(R, 6) + r * 10000 for r in range(world)])]
    ok = all(torch.equal(d.tensor, w) for d, w in zip(dsts, want))
    results.append(("uniform all-gather x3", ok, "gathered tensors bit-exact"))

    # uniform reduce-scatter, bf16 (fp32 accumulation) and fp32
    for dtype, tol in ((torch.bfloat16, 2e-2), (torch.float32, 1e-5)):
        buf = heap.alloc(f"rs_{dtype}", [R * world, H], dtype)
        buf.tensor.copy_(data(300 + rank, (R * world, H), dtype))
        torch.cuda.synchronize()
        dist.barrier(group)
        out = torch.zeros(R, H, dtype=dtype, device=dev)
        UniformReduceScatterPlan(heap, out, buf).launch()
        torch.cuda.synchronize()
        dist.barrier(group)
        total = sum(data(300 + r, (R * world, H), dtype).float() for r in range(world))
        ok = torch.allclose(out.float(), total[rank * R:(rank + 1) * R], rtol=tol, atol=tol * world)
        results.append((f"uniform reduce-scatter {str(dtype).split('.')[-1]}", bool(ok), f"rows {R} x {H}"))

    # fused reduce-scatter + residual + RMSNorm + all-gather
    tokens = R // 4 * world
    buf = heap.alloc("norm", [tokens, H], torch.bfloat16)
    buf.tensor.copy_(data(400 + rank, (tokens, H)))
    residual = data(500 + rank, (tokens // world, H))
    weight = (1 + 0.1 * data(600, (H,), torch.float32)).to(torch.bfloat16)
    torch.cuda.synchronize()
    dist.barrier(group)
    RsAddNormAgPlan(heap, buf, residual, weight, eps=1e-5).launch()
    torch.cuda.synchronize()
    dist.barrier(group)
    want_norm, want_res = oracle.rs_add_norm_ag([data(400 + r, (tokens, H)).cpu() for r in range(world)],
                                                [data(500 + r, (tokens // world, H)).cpu() for r in range(world)],
                                                weight.cpu(), 1e-5)
    ok = (torch.allclose(buf.tensor.float().cpu(), want_norm, rtol=2e-2, atol=2e-2)
          and torch.allclose(residual.float().cpu(), want_res[rank].float(), rtol=2e-2, atol=2e-2))
    results.append(("reduce-scatter + residual + RMSNorm + all-gather", bool(ok), f"{tokens} tokens x {H}"))

    local_ok = all(ok for _, ok, _ in results)
    try:
        heap.check_status()
    except Exception as e:
        results.append(("device status", False, str(e)))
        local_ok = False
    for name, ok, detail in results:
        if rank == 0 or not ok:
            print(f"  [rank{rank}] [{'PASS' if ok else 'FAIL'}] {name}  {detail}", flush=True)
    verdict = torch.tensor([1.0 if local_ok else 0.0], device=dev)
    dist.all_reduce(verdict, op=dist.ReduceOp.MIN, group=group)
    if rank == 0:
        print(f"# SELFTEST {'PASSED' if verdict.item() > 0.5 else 'FAILED'} (all {world} ranks, transport={heap.transport})",
              flush=True)
    dist.barrier(group)
    dist.destroy_process_group()
    return 0 if verdict.item() > 0.5 else 1


if __name__ == "__main__":
    sys.exit(main())
