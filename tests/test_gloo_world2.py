"""CPU/gloo world_size=2 plumbing: dense AllGather -> identity expert -> ReduceScatter
(emulated as all_reduce + slice).  16 experts, top-4, hidden 128, fp32, seed 0; B=8 split 4/4
over 2 layers and B=1 with one idle rank; the combine output must equal m*x with m the number of
distinct destination ranks.  Also runs the driver's --validate and a timed sweep as 2 ranks."""
import os
import subprocess
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT, free_port


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    from moe_comms_benchmarking_b200.config import Config
    from moe_comms_benchmarking_b200.ops import oracle
    from moe_comms_benchmarking_b200.parallel.dist import all_rank_counts, init_distributed
    from moe_comms_benchmarking_b200.parallel.gloo import GlooDenseDispatcher
    from moe_comms_benchmarking_b200.utils.inputs import make_inputs
    group, r, w, _ = init_distributed(backend="gloo")
    cfg = Config(num_experts=16, topk=4, hidden=128, ep_size=w, rank=r, per_rank_cap=4, seed=0)
    d = GlooDenseDispatcher(cfg, group)
    d.build()
    ok, ms = True, []
    for B in (8, 1):
        counts = all_rank_counts(B, w)
        h, idx, probs = make_inputs(cfg, B, "cpu")
        x = torch.randn(counts[r], 128, generator=torch.Generator().manual_seed(B * 10 + r))   # fp32 N(0,1)
        assert h.shape[0] == counts[r]
        d.setup_batch(x, idx, probs)
        for _ in range(2):                                  # 2 layers
            d.step()
        ref = oracle.roundtrip_identity(x, idx, 16, w)
        ok = ok and d.out.shape == ref.shape and bool(torch.allclose(d.out, ref, atol=1e-6))
        if counts[r]:
            ms += oracle.dest_rank_multiplicity(idx, 16, w).tolist()
    ok = ok and all(passed for _, passed, _ in d.validate())
    q.put((r, ok, ms))
    dist.barrier()
    dist.destroy_process_group()


def test_gloo_dense_roundtrip_world2():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok, _ in res)
    ms = [m for _, _, v in res for m in v]
    assert ms and all(1 <= m <= 2 for m in ms)


def _torchrun(extra, port):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "run.py"), "--model", "tiny-cpu"] + extra
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    return subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)


def test_driver_validate_two_cpu_ranks():
    res = _torchrun(["--validate"], free_port())
    assert res.returncode == 0, res.stdout + res.stderr
    assert "# VALIDATION PASSED (all 2 ranks)" in res.stdout
    assert "[rank0] [PASS] gloo dispatch->combine" in res.stdout


def test_driver_sweep_csv_and_resume(tmp_path):
    out = str(tmp_path / "r.csv")
    res = _torchrun(["--batch-sizes", "1,8", "--reps", "2", "--warmup", "1", "--out", out], free_port())
    assert res.returncode == 0, res.stdout + res.stderr
    lines = open(out).read().splitlines()
    assert lines[0] == "impl,global_B,num_sms,phase,per_rank_counts,latency_us,timing"
    assert lines[1].startswith('gloo,1,-1,decode_step,"[1, 0]",') and lines[2].startswith('gloo,8,-1,decode_step,"[4, 4]",')
    assert "# impl,global_B,num_sms,phase,latency_us,timing" in res.stdout
    res = _torchrun(["--batch-sizes", "1,8,16", "--reps", "2", "--warmup", "1", "--out", out, "--resume"], free_port())
    assert res.returncode == 0, res.stdout + res.stderr
    lines2 = open(out).read().splitlines()
    assert lines2[:3] == lines[:3] and len(lines2) == 4 and lines2[3].startswith("gloo,16,")
