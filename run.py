#!/usr/bin/env python3
"""MoE dispatch/combine decode benchmark driver (one process per GPU, launched with torchrun).

    torchrun --nproc_per_node=8 run.py --impl all --batch-sizes 1,2,4,...,8192 --out results.csv
    torchrun --nproc_per_node=8 run.py --impl all --validate

Times ONE decode step = ``--num-layers`` MoE layers of paired dispatch -> (identity expert) ->
combine, captured and replayed as one CUDA graph, reported in microseconds as the max over
ranks; B is the GLOBAL token count over all expert-parallel ranks.

Command line, stdout lines, CSV schema, ``[PASS]/[FAIL]`` validation lines, verdict line and
exit codes follow the reference driver (run.py:40-62, 105-111, 137-198, 221-238).  The
implementations behind ``--impl`` are this repository's own:

  dense (alias nvls)    AllGather-V / ReduceScatter-V, hand-written sm_100a kernels over NVSwitch
  a2a   (alias deepep)  all-to-all-V with direct peer stores/loads (``--dispatch-dtype fp8`` for e4m3)
  nccl                  padded NCCL AllGather x3 + fp32 ReduceScatter (the baseline)
  fused                 dense transport fused with real SwiGLU experts (tcgen05 grouped GEMMs)
  gloo                  the dense algorithm on CPU ranks (no GPU needed)
  both = a2a + dense,  all = a2a + dense + nccl

``--expert swiglu`` replaces the identity expert by a real SwiGLU FFN per expert: ``--impl dense`` (or
``fused``) then runs the fused expert path, and ``--impl nccl`` an EXTENDED baseline that the reference
does not have (NCCL all-gather x3 + library grouped GEMMs + fp32 NCCL reduce-scatter, reported as
``nccl-swiglu``), so that the fused path has something to be compared with.
"""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from moe_comms_benchmarking_b200.config import Config  # noqa: E402
from moe_comms_benchmarking_b200.models.presets import PRESETS, get_preset  # noqa: E402
from moe_comms_benchmarking_b200.parallel.dist import init_distributed  # noqa: E402
from moe_comms_benchmarking_b200.utils.inputs import make_inputs, rank_counts  # noqa: E402
from moe_comms_benchmarking_b200.utils.report import CsvSink, Row, STDOUT_HEADER  # noqa: E402
from moe_comms_benchmarking_b200.utils.trace import phase  # noqa: E402

IMPL_CHOICES = ["deepep", "nvls", "nccl", "both", "all", "dense", "a2a", "fused", "gloo"]


def parse_args(argv=None):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--impl", choices=IMPL_CHOICES, default="all",
                   help="deepep|a2a, nvls|dense, nccl, both (a2a+dense), all (a2a+dense+nccl), fused, gloo")
    p.add_argument("--batch-sizes", default="1,2,4,8,16,32,64,128", help="comma-separated GLOBAL token counts")
    p.add_argument("--deepep-num-sms", "--num-sms", dest="deepep_num_sms", default="148",
                   help="comma-separated CTA counts to sweep for the all-to-all dispatcher "
                        "(rounded to even, clamped to the device SM count)")
    p.add_argument("--num-layers", type=int, default=None, help="MoE layers per decode step (default: the model's, 88)")
    p.add_argument("--reps", type=int, default=100)
    p.add_argument("--warmup", type=int, default=20)
    p.add_argument("--timing", choices=["graph", "eager"], default="graph")
    p.add_argument("--seed", type=int, default=1234)
    p.add_argument("--out", default=None, help="CSV output path (rank 0)")
    p.add_argument("--validate", action="store_true",
                   help="run the known-value correctness checks of each implementation and exit")
    # additive flags (defaults reproduce the reference's fixed configuration)
    p.add_argument("--model", choices=sorted(PRESETS), default="nemotron-super")
    p.add_argument("--num-experts", type=int, default=None)
    p.add_argument("--topk", type=int, default=None)
    p.add_argument("--hidden", type=int, default=None)
    p.add_argument("--intermediate", type=int, default=None)
    p.add_argument("--routing", choices=["uniform", "zipf"], default="uniform")
    p.add_argument("--counts", choices=["balanced", "multinomial"], default="balanced")
    p.add_argument("--dispatch-dtype", choices=["bf16", "fp8"], default="bf16")
    p.add_argument("--expert", choices=["identity", "swiglu"], default="identity",
                   help="swiglu: real experts (dense/fused -> the fused expert path, nccl -> NCCL + library GEMMs)")
    p.add_argument("--no-persistent", action="store_true",
                   help="dense / a2a: one kernel per operation (1 + 2 x layers / 2 x layers launches) instead of one per decode step")
    p.add_argument("--groups", type=int, default=1,
                   help="dense: pipeline groups of the persistent step kernel (1 = none)")
    p.add_argument("--phase-times", action="store_true",
                   help="fused: after each batch size print how long block 0 of rank 0 spent in each phase of the last "
                        "layer (dispatch, routing, experts, combine and the grid barriers between them)")
    p.add_argument("--no-layer-kernel", action="store_true",
                   help="fused: the two-kernel form with tokens as the M operand instead of one kernel per layer")
    p.add_argument("--dense-num-sms", type=int, default=148, help="CTA cap of the dense kernels")
    p.add_argument("--transport", choices=["auto", "multimem", "p2p"], default="auto")
    p.add_argument("--heap-allocator", choices=["torch", "native"], default=None,
                   help="host-side allocator of the symmetric heap: PyTorch's symmetric memory (default) or this "
                        "library's own (driver virtual-memory API, one node); default: $MCB_HEAP_ALLOCATOR or torch")
    p.add_argument("--ll-rows", type=int, default=-1,
                   help="dense dispatcher: steps with at most this many tokens over all ranks use "
                        "low-latency flagged packets instead of barrier + multicast (0 = never, -1 = measured default)")
    p.add_argument("--a2a-ll-rows", type=int, default=-1,
                   help="all-to-all dispatcher: steps with at most this many tokens over all ranks run the packet mode "
                        "of the persistent step kernel (0 = never, -1 = measured default)")
    p.add_argument("--no-pdl", action="store_true", help="disable programmatic dependent launch")
    p.add_argument("--coop-pdl", action="store_true",
                   help="fused: also allow programmatic dependent launch on the cooperative fused kernels")
    p.add_argument("--no-fuse-dispatch", action="store_true",
                   help="fused: launch dispatch, routing and the FC1 GEMM as three kernels instead of one")
    p.add_argument("--no-fuse-combine", action="store_true",
                   help="fused: launch the FC2 GEMM and the combine as two kernels instead of one")
    p.add_argument("--weight-budget-gb", type=float, default=48.0,
                   help="fused: GPU memory for expert weights; layers share weight sets round-robin beyond it")
    p.add_argument("--resume", action="store_true", help="keep rows already in --out and skip them")
    return p.parse_args(argv)


def resolve_impls(impl: str, on_gpu: bool, expert: str = "identity") -> list[str]:
    if not on_gpu:
        return ["gloo"]
    table = {"deepep": ["a2a"], "a2a": ["a2a"], "nvls": ["dense"], "dense": ["dense"], "nccl": ["nccl"],
             "both": ["a2a", "dense"], "all": ["a2a", "dense", "nccl"], "fused": ["fused"], "gloo": ["gloo"]}
    names = table[impl]
    if expert == "swiglu":      # real experts: the fused path, and the extended NCCL baseline
        swap = {"dense": "fused", "fused": "fused", "nccl": "nccl-swiglu"}
        if any(n not in swap for n in names):
            raise SystemExit("--expert swiglu is available for --impl dense, fused and nccl")
        names = [swap[n] for n in names]
    return names


def make_config(args, world, rank, local_rank, batch_sizes) -> tuple[Config, int]:
    shape = get_preset(args.model)
    cfg = Config(num_experts=args.num_experts or shape.num_experts, topk=args.topk or shape.topk,
                 hidden=args.hidden or shape.hidden, intermediate=args.intermediate or shape.intermediate,
                 ep_size=world, rank=rank, local_rank=local_rank, per_rank_cap=-(-max(batch_sizes) // world),
                 seed=args.seed, routing=args.routing, probs=shape.probs, counts=args.counts)
    if args.counts == "multinomial":
        cfg.per_rank_cap = max(batch_sizes)          # a skewed split may put every token on one rank
    return cfg, (args.num_layers or shape.num_layers)


def build_dispatchers(names, cfg, group, args, device, sms_list):
    from moe_comms_benchmarking_b200.parallel.symm_heap import SymmetricHeap, required_bytes
    out, heap = [], None
    fp8 = args.dispatch_dtype == "fp8"
    if any(n in ("dense", "a2a", "fused") for n in names):
        from moe_comms_benchmarking_b200.parallel.a2a import A2ADispatcher
        from moe_comms_benchmarking_b200.parallel.dense import DenseDispatcher
        specs = []
        if "dense" in names:
            specs += DenseDispatcher.heap_specs(cfg, ll_rows=args.ll_rows, fp8=fp8)
        if "a2a" in names:
            specs += A2ADispatcher.heap_specs(cfg, fp8, args.a2a_ll_rows)
        if "fused" in names:
            from moe_comms_benchmarking_b200.parallel.fused import FusedExpertDispatcher
            specs += FusedExpertDispatcher.heap_specs(cfg, ll_rows=args.ll_rows)
        heap = SymmetricHeap(group, required_bytes(specs), device, transport=args.transport)
    for n in names:
        if n == "a2a":
            out.append(A2ADispatcher(cfg, group, heap, num_sms=sms_list[0], pdl=not args.no_pdl, fp8_dispatch=fp8,
                                     persistent=not args.no_persistent, ll_rows=args.a2a_ll_rows))
        elif n == "dense":
            out.append(DenseDispatcher(cfg, group, heap, num_sms=args.dense_num_sms, pdl=not args.no_pdl,
                                       ll_rows=args.ll_rows, persistent=not args.no_persistent, groups=args.groups,
                                       fp8_dispatch=fp8))
        elif n == "fused":
            out.append(FusedExpertDispatcher(cfg, group, heap, pdl=not args.no_pdl, ll_rows=args.ll_rows,
                                             num_layers=1 if args.validate else (args.num_layers or 88),
                                             weight_budget_gb=args.weight_budget_gb,
                                             fuse_combine=not args.no_fuse_combine,
                                             fuse_dispatch=not args.no_fuse_dispatch, coop_pdl=args.coop_pdl,
                                             layer_kernel=not args.no_layer_kernel, phase_trace=args.phase_times))
        elif n == "nccl":
            from moe_comms_benchmarking_b200.parallel.nccl import NCCLDispatcher
            out.append(NCCLDispatcher(cfg, group))
        elif n == "nccl-swiglu":
            from moe_comms_benchmarking_b200.parallel.nccl import NCCLSwiGLUDispatcher
            out.append(NCCLSwiGLUDispatcher(cfg, group, num_layers=1 if args.validate else (args.num_layers or 88),
                                            weight_budget_gb=args.weight_budget_gb))
        elif n == "gloo":
            from moe_comms_benchmarking_b200.parallel.gloo import GlooDenseDispatcher
            out.append(GlooDenseDispatcher(cfg, group))
    return out, heap


def cross_impl_check(benchers, cfg, world, rank, device, say):
    """Same tokens and routing through every implementation: each output must match m*x and
    the outputs must match one another (run.py:152-186 of the reference)."""
    local_ok = True
    rt = [b for b in benchers if hasattr(b, "functional_roundtrip")]
    if len(rt) < 2:
        return True
    E, K, H, epr = cfg.num_experts, cfg.topk, cfg.hidden, cfg.num_experts // world
    for B in (world * 2, 1):
        n = [B // world + (1 if r < B % world else 0) for r in range(world)][rank]
        gen = torch.Generator(device=device).manual_seed(555 + B + rank * 977)
        x = torch.randn(n, H, generator=gen, device=device).to(torch.bfloat16)
        idx = (torch.stack([torch.randperm(E, generator=gen, device=device)[:K] for _ in range(n)])
               if n else torch.empty(0, K, device=device, dtype=torch.int64))
        outs = {b.name: b.functional_roundtrip(x, idx).to(torch.float32).clone() for b in rt}
        if device.type == "cuda":
            torch.cuda.synchronize()
        if n:
            m = torch.tensor([torch.unique(idx[t] // epr).numel() for t in range(n)], device=device,
                             dtype=torch.float32).view(n, 1)
            ref = m * x.float()
            scale = float(ref.abs().max()) + 1e-6
            errs = {k: float((o - ref).abs().max()) for k, o in outs.items()}
            names = list(outs)
            cross = max((float((outs[a] - outs[c]).abs().max()) for i, a in enumerate(names) for c in names[i + 1:]),
                        default=0.0)
            tol_pair = 0.08 if any("fp8" in k for k in names) else 0.02
            tol_ref = 0.08 if any("fp8" in k for k in names) else 0.05
            ok = cross / scale < tol_pair and all(e / scale < tol_ref for e in errs.values())
            detail = (f"n={n} max|pairwise|={cross:.4f} ({100 * cross / scale:.2f}% of {scale:.2f}); vs m*x: "
                      + " ".join(f"{k}={v:.4f}" for k, v in errs.items()))
        else:
            ok, detail = True, "n=0 (idle rank)"
        local_ok = local_ok and ok
        if rank == 0 or not ok:
            say(f"  [rank{rank}] [{'PASS' if ok else 'FAIL'}] cross-impl [{'='.join(outs)}] B={B:<4d}  {detail}")
    return local_ok


def main(argv=None) -> int:
    args = parse_args(argv)
    if args.heap_allocator:
        os.environ["MCB_HEAP_ALLOCATOR"] = args.heap_allocator       # every heap of this job follows
    group, rank, world, local_rank = init_distributed()
    on_gpu = torch.cuda.is_available()
    device = torch.device("cuda", local_rank) if on_gpu else torch.device("cpu")
    batch_sizes = [int(b) for b in args.batch_sizes.split(",")]
    cfg, nl = make_config(args, world, rank, local_rank, batch_sizes)

    def say(msg):
        print(msg, flush=True)

    dev_sms = torch.cuda.get_device_properties(local_rank).multi_processor_count if on_gpu else 0
    even = lambda s: max(2, min(int(s), dev_sms or int(s)) - (min(int(s), dev_sms or int(s)) % 2))  # noqa: E731
    sms_sweep = sorted({even(s) for s in args.deepep_num_sms.split(",")})
    names = resolve_impls(args.impl, on_gpu, args.expert)
    if rank == 0:
        say("# MoE dispatch/combine decode benchmark")
        say(f"# EP={world} experts={cfg.num_experts} topk={cfg.topk} hidden={cfg.hidden} "
            f"per_rank_cap={cfg.per_rank_cap} timing={args.timing} reps={args.reps}")
        say(f"# impl={args.impl} -> {'+'.join(names)} num_layers={nl} device_sms={dev_sms} "
            f"num_sms_sweep={sms_sweep} routing={cfg.routing} counts={cfg.counts} dispatch={args.dispatch_dtype}")

    with phase("build", rank):
        benchers, heap = build_dispatchers(names, cfg, group, args, device, sms_sweep)
        dist.barrier(group)
        for b in benchers:
            b.build()
        dist.barrier(group)
    if rank == 0 and heap is not None:
        say(f"# symmetric heap: {heap.bytes_used() / 2**20:.1f} MiB used, transport={heap.transport}, allocator={heap.allocator}")

    if args.validate:
        local_ok = True
        for b in benchers:
            for name, ok, detail in b.validate():
                local_ok = local_ok and ok
                if rank == 0 or not ok:
                    say(f"  [rank{rank}] [{'PASS' if ok else 'FAIL'}] {name}  {detail}")
        local_ok = cross_impl_check(benchers, cfg, world, rank, device, say) and local_ok
        verdict = torch.tensor([1.0 if local_ok else 0.0], device=device)
        dist.all_reduce(verdict, op=dist.ReduceOp.MIN, group=group)
        passed = verdict.item() > 0.5
        if rank == 0:
            say(f"# VALIDATION {'PASSED' if passed else 'FAILED'} (all {world} ranks)")
        dist.barrier(group)
        for b in benchers:
            b.destroy()
        dist.destroy_process_group()
        return 0 if passed else 1

    from moe_comms_benchmarking_b200.utils.timing import timed_with_fallback
    sink = CsvSink(args.out if rank == 0 else None, resume=args.resume)
    done = set(sink.done)
    if args.resume and world > 1:       # every rank must skip the same rows
        box = [sorted(done)] if rank == 0 else [None]
        dist.broadcast_object_list(box, src=0, group=group)
        done = {tuple(k) for k in box[0]}
    for b in benchers:
        sweep = sms_sweep if b.name.startswith("a2a") else [b.num_sms]
        for sms in sweep:
            if b.name.startswith("a2a"):
                b.set_num_sms(sms)
            for B in batch_sizes:
                if (b.name, B, sms, "decode_step") in done:
                    continue
                counts = rank_counts(cfg, B)
                hidden, topk_idx, topk_w = make_inputs(cfg, B, device, n=counts[rank])
                b.setup_batch(hidden, topk_idx, topk_w)
                if on_gpu:
                    with phase(f"time {b.name} B={B}", rank):
                        (_, step_us), used_graph = timed_with_fallback(lambda: b.decode_step(nl), group, args.warmup,
                                                                       args.reps, args.timing, rank)
                    b.check_health()
                    if args.phase_times and getattr(b, "phase_trace", False):
                        torch.cuda.synchronize()
                        say(f"    phases of the last layer (block 0, rank {rank}): "
                            + ", ".join(f"{n} {us:.1f}us" for n, us in b.layer_plan.phase_times())) if rank == 0 else None
                else:
                    import time
                    for _ in range(args.warmup):
                        b.decode_step(nl)
                    dist.barrier(group)
                    t0 = time.perf_counter()
                    for _ in range(args.reps):
                        b.decode_step(nl)
                    t = torch.tensor([(time.perf_counter() - t0) * 1e6 / args.reps], dtype=torch.float64)
                    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
                    step_us, used_graph = float(t.item()), False
                row = Row(b.name, B, sms, "decode_step", counts, step_us, used_graph)
                if rank == 0:
                    sink.add(row)
                    say(row.progress_line(nl))
    if rank == 0:
        say("\n" + STDOUT_HEADER)
        for r in sink.rows:
            say(r.stdout_csv_line())
        if args.out:
            say(f"# wrote {args.out}")
    for b in benchers:
        b.destroy()
    dist.barrier(group)
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
