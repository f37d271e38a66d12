"""Per-kernel timing of the expert path on ONE GPU with the per-rank load of an EP=W run.

    python -m moe_comms_benchmarking_b200.bench_experts --tokens 64,512,4096,8192 --ep 8

Gathered tokens T are routed over all 512 experts; only the 512/W experts of "this rank" are
local, which reproduces the work one rank of an EP=W job does per layer.  Every kernel is timed
with CUDA events after warm-up, with a 256 MiB write between iterations (L2 flush); the report
gives algorithmic bytes and FLOPs against the measured peaks in MEASURED_PEAKS.json when present.
"""
from __future__ import annotations

import argparse
import json
import os

import torch


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", default="64,512,4096,8192")
    ap.add_argument("--ep", type=int, default=8)
    ap.add_argument("--experts", type=int, default=512)
    ap.add_argument("--topk", type=int, default=22)
    ap.add_argument("--hidden", type=int, default=1024)
    ap.add_argument("--intermediate", type=int, default=1024)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--only", default="", help="comma-separated subset of route,fc1,fc2,ffn,combine to time")
    args = ap.parse_args(argv)
    from moe_comms_benchmarking_b200.ops import _ext
    from moe_comms_benchmarking_b200.ops.experts import (ExpertCombinePlan, ExpertFfnPlan, ExpertWeights, GroupedGemmPlan,
                                                         RouteBuffers, RoutePlan)
    from moe_comms_benchmarking_b200.parallel.symm_heap import SymmetricHeap
    dev = "cuda:0"
    torch.cuda.set_device(0)
    peaks = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "src": "fallback"}
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    if os.path.exists(os.path.join(root, "MEASURED_PEAKS.json")):
        p = json.load(open(os.path.join(root, "MEASURED_PEAKS.json")))
        peaks = {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "src": "measured"}
    E, K, H, I = args.experts // args.ep, args.topk, args.hidden, args.intermediate
    tokens = [int(t) for t in args.tokens.split(",")]
    cap = max(tokens)
    heap = SymmetricHeap(None, cap * H * 2 + (1 << 20), dev)
    partial = heap.alloc("partial", [cap, H], torch.bfloat16)
    weights = ExpertWeights(E, H, I, dev, seed=1, layout="split")       # tokens-as-rows GEMM kernels
    weights_il = ExpertWeights(E, H, I, dev, seed=1)                    # weights-as-M FFN kernel (packed tiles)
    route = RouteBuffers(cap, K, E, dev)
    xs = torch.randn(cap, H, device=dev).to(torch.bfloat16)
    idxs = torch.zeros(cap, K, dtype=torch.int64, device=dev)
    ws = torch.rand(cap, K, device=dev)
    act = torch.zeros(route.max_pairs, I, dtype=torch.bfloat16, device=dev)
    y = torch.zeros(route.max_pairs, H, dtype=torch.bfloat16, device=dev)
    out = torch.zeros(cap, H, dtype=torch.bfloat16, device=dev)
    ntok = torch.zeros(1, dtype=torch.int32, device=dev)
    meta = torch.zeros(4, dtype=torch.int32, device=dev)
    st = heap.status
    plans = {
        "route": RoutePlan(route, idxs, ws, ntok, expert_begin=0, status=st),
        "fc1": GroupedGemmPlan(_ext.GEMM_FC1, weights.map_gate_up, route, xs, act, 2 * I, H, st),
        "fc2": GroupedGemmPlan(_ext.GEMM_FC2, weights.map_down, route, act, y, H, I, st),
        "ffn": ExpertFfnPlan(weights_il, route, xs, act, y, st),
        "combine": ExpertCombinePlan(heap, y, route, partial, out, ntok, meta, cap),
    }
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    print(f"# per-rank load of EP={args.ep}: {E} local experts, top-{K}, H={H}, I={I}; peaks ({peaks['src']}): "
          f"{peaks['hbm_gbs']:.0f} GB/s, {peaks['bf16_tflops']:.0f} TFLOP/s bf16")
    for T in tokens:
        g = torch.Generator(device=dev).manual_seed(T)
        scores = torch.rand(T, args.experts, device=dev, generator=g)
        idxs[:T] = torch.topk(scores, K, dim=-1).indices
        ntok.fill_(T)
        meta.copy_(torch.tensor([T, 0, T, 1], dtype=torch.int32))
        times = {}
        only = [k for k in args.only.split(",") if k]
        for name, plan in plans.items():
            if only and name not in only:
                times[name] = float("nan")
                continue
            for _ in range(args.warmup):
                for p in plans.values():
                    p.launch()
            torch.cuda.synchronize()
            evs = []
            for _ in range(args.iters):
                for n2, p in plans.items():       # keep the chain's data dependencies fresh
                    if n2 == name:
                        if not args.no_flush:
                            flush.zero_()
                        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        s.record(); p.launch(); e.record()
                        evs.append((s, e))
                    else:
                        p.launch()
            torch.cuda.synchronize()
            times[name] = sorted(s.elapsed_time(e) * 1e3 for s, e in evs)[len(evs) // 2]
        # back-to-back launches of the weight-streaming kernels (no host gap, no flush needed: a layer's
        # weights are several times the L2): the kernel time without launch latency
        b2b = {}
        for name in ("fc1", "fc2", "ffn"):
            if only and name not in only:
                b2b[name] = float("nan")
                continue
            reps = max(args.iters, 5)
            plans[name].launch()
            torch.cuda.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(reps):
                plans[name].launch()
            e.record()
            torch.cuda.synchronize()
            b2b[name] = s.elapsed_time(e) * 1e3 / reps
        heap.check_status()
        pairs = int(route.expert_offset[E])
        tiles = int(route.num_m_tiles)
        w1, w2 = E * 2 * I * H * 2, E * H * I * 2
        f1, f2 = 2.0 * pairs * 2 * I * H, 2.0 * pairs * H * I
        f1p, f2p = 2.0 * tiles * 128 * 2 * I * H, 2.0 * tiles * 128 * H * I    # FLOPs issued incl. row padding
        def frac(us, nbytes, flops):
            return max(nbytes / (peaks["hbm_gbs"] * 1e3) / us, flops / (peaks["bf16_tflops"] * 1e6) / us)
        print(f"T={T:5d} pairs={pairs:6d} m_tiles={tiles:4d} | route {times['route']:7.1f}us | "
              f"fc1 {times['fc1']:7.1f}us ({w1 / times['fc1'] / 1e3:6.0f} GB/s weights, {f1 / times['fc1'] / 1e6:6.0f} useful / "
              f"{f1p / times['fc1'] / 1e6:6.0f} issued TFLOP/s, {100 * frac(times['fc1'], w1 + pairs * (H + I) * 2, f1):4.0f}% of roofline) | "
              f"fc2 {times['fc2']:7.1f}us ({w2 / times['fc2'] / 1e3:6.0f} GB/s, {f2 / times['fc2'] / 1e6:6.0f}/{f2p / times['fc2'] / 1e6:6.0f} TFLOP/s, "
              f"{100 * frac(times['fc2'], w2 + pairs * (H + I) * 2, f2):4.0f}%) | "
              f"ffn (gate/up + down, weights as M, one launch) {times['ffn']:7.1f}us ({(w1 + w2) / times['ffn'] / 1e3:6.0f} GB/s weights, "
              f"{100 * frac(times['ffn'], w1 + w2 + pairs * (H + 2 * I + H) * 2, f1 + f2):4.0f}% of roofline) | "
              f"combine {times['combine']:7.1f}us | back to back: fc1 {b2b['fc1']:6.1f} fc2 {b2b['fc2']:6.1f} "
              f"ffn {b2b['ffn']:6.1f}us ({(w1 + w2) / b2b['ffn'] / 1e3:5.0f} GB/s)", flush=True)


if __name__ == "__main__":
    main()
