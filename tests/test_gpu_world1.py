"""Dispatchers, engine and driver on ONE GPU (EP=1): the degenerate world still runs every
kernel of the library (peer transport onto its own heap)."""
import json
import os
import subprocess
import sys

import pytest
import torch

from conftest import ROOT, free_port

pytestmark = pytest.mark.gpu


def _cfg(cap=32, **kw):
    from moe_comms_benchmarking_b200.config import Config
    return Config(ep_size=1, rank=0, local_rank=0, per_rank_cap=cap, **kw)


@pytest.mark.parametrize("pdl", [False, True])
def test_dense_dispatcher_validate_and_graph_reuse(world1, pdl):
    from moe_comms_benchmarking_b200.parallel.dense import DenseDispatcher
    from moe_comms_benchmarking_b200.utils.inputs import make_inputs
    from moe_comms_benchmarking_b200.utils.timing import capture_graph
    cfg = _cfg(64)
    d = DenseDispatcher(cfg, world1, pdl=pdl)
    d.build()
    for name, ok, detail in d.validate():
        assert ok, f"{name}: {detail}"
    # one graph, two batch sizes: the token count is read from device memory at replay
    h, i, w = make_inputs(cfg, 40, "cuda:0")
    d.setup_batch(h, i, w)
    g = capture_graph(lambda: d.decode_step(3))
    for n in (40, 7, 0, 64):
        h, i, w = make_inputs(cfg, n, "cuda:0")
        d.setup_batch(h, i, w)
        d.rsv.tensor.normal_()
        g.replay()
        torch.cuda.synchronize()
        assert d.step_metadata[:3].tolist() == [n, 0, n]
        gh, gr, gp = d.gathered()           # the parity the last layer of the step wrote
        assert torch.equal(gh[:n], h) and torch.equal(gr[:n], i) and torch.equal(gp[:n], w)
        assert torch.equal(d.out, d.rsv.tensor[:n])        # world of one: the sum is the row itself
    d.check_health()
    d.destroy()


@pytest.mark.parametrize("persistent", [True, False])
def test_set_num_sms_on_every_dispatcher(world1, persistent):
    """Changing the CTA-count knob on a built dispatcher rebuilds its plans and keeps it correct."""
    from moe_comms_benchmarking_b200.parallel.a2a import A2ADispatcher
    from moe_comms_benchmarking_b200.parallel.dense import DenseDispatcher
    from moe_comms_benchmarking_b200.utils.inputs import make_inputs
    cfg = _cfg(32)
    for d in (DenseDispatcher(cfg, world1, persistent=persistent), A2ADispatcher(cfg, world1)):
        d.build()
        for sms in (16, 148, 64):
            d.set_num_sms(sms)
            h, i, w = make_inputs(cfg, 20, "cuda:0")
            d.setup_batch(h, i, w)
            d.decode_step(2)
            torch.cuda.synchronize()
            d.check_health()
            for name, ok, detail in d.validate():
                assert ok, f"{d.name} sms={sms} {name}: {detail}"
        d.destroy()


def test_dense_capacity_overflow_is_reported(world1):
    from moe_comms_benchmarking_b200.parallel.dense import DenseDispatcher
    from moe_comms_benchmarking_b200.parallel.symm_heap import DeviceStatusError
    d = DenseDispatcher(_cfg(8), world1)
    d.build()
    d.n_local.fill_(9)          # bypass the host check on purpose
    d.decode_step(1)
    torch.cuda.synchronize()
    with pytest.raises(DeviceStatusError) as e:
        d.check_health()
    assert e.value.code == 2
    d.heap.reset_sync_state()
    d.n_local.fill_(3)
    d.decode_step(1)
    torch.cuda.synchronize()
    d.check_health()
    d.destroy()


@pytest.mark.parametrize("fp8", [False, True])
def test_a2a_dispatcher_validate(world1, fp8):
    from moe_comms_benchmarking_b200.parallel.a2a import A2ADispatcher
    d = A2ADispatcher(_cfg(32), world1, fp8_dispatch=fp8)
    d.build()
    for name, ok, detail in d.validate():
        assert ok, f"{name}: {detail}"
    d.decode_step(4)
    torch.cuda.synchronize()
    d.check_health()
    d.destroy()


def test_nccl_baseline_validate(world1):
    from moe_comms_benchmarking_b200.parallel.nccl import NCCLDispatcher
    d = NCCLDispatcher(_cfg(32), world1)
    d.build()
    for name, ok, detail in d.validate():
        assert ok, f"{name}: {detail}"


def test_engine_end_to_end_from_pinned_host(world1):
    from moe_comms_benchmarking_b200.models.engine import MoEDecodeEngine
    from moe_comms_benchmarking_b200.utils.inputs import make_inputs
    cfg = _cfg(48)
    eng = MoEDecodeEngine(cfg, world1, impl="dense", num_layers=4).build().capture()
    for n in (48, 5):
        h, i, w = make_inputs(cfg, n, "cuda:0")
        eng.dispatcher.rsv.tensor.normal_()
        out = eng.step_host(h.cpu().pin_memory(), i.cpu().pin_memory(), w.cpu().pin_memory())
        assert out.shape == (n, cfg.hidden)
        assert torch.equal(out, eng.dispatcher.rsv.tensor[:n].cpu())
        assert torch.equal(eng.dispatcher.gathered()[0][:n].cpu(), h.cpu())
    eng.check_health()
    eng.destroy()


def test_uniform_collectives_world1(world1):
    from moe_comms_benchmarking_b200.ops.dense import UniformAllGatherPlan, UniformReduceScatterPlan
    from moe_comms_benchmarking_b200.parallel.symm_heap import SymmetricHeap
    heap = SymmetricHeap(world1, 4 << 20, "cuda:0")
    src = torch.randn(33, 512, device="cuda:0").to(torch.bfloat16)
    dst = heap.alloc("ag", [33, 512], torch.bfloat16)
    UniformAllGatherPlan(heap, [dst], [src]).launch()
    out = torch.zeros(33, 512, dtype=torch.bfloat16, device="cuda:0")
    UniformReduceScatterPlan(heap, out, dst).launch()
    torch.cuda.synchronize()
    assert torch.equal(dst.tensor, src) and torch.equal(out, src)
    heap.check_status()


def _run(cmd, timeout=600):
    # children rendezvous on their own port, not on the one this process's group listens on
    env = dict(os.environ, MASTER_PORT=str(free_port()))
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        env.pop(k, None)
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, cwd=ROOT, env=env)


def test_driver_validate_and_sweep_one_gpu(tmp_path):
    base = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "1", "--master-addr",
            "127.0.0.1"]
    res = _run(base + ["--master-port", str(free_port()), "run.py", "--impl", "all", "--validate"])
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "# VALIDATION PASSED (all 1 ranks)" in res.stdout
    assert "cross-impl [a2a=dense=nccl]" in res.stdout
    out = str(tmp_path / "r.csv")
    res = _run(base + ["--master-port", str(free_port()), "run.py", "--impl", "all", "--batch-sizes", "1,64",
                       "--num-layers", "8", "--reps", "5", "--warmup", "2", "--out", out])
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    rows = open(out).read().splitlines()
    assert len(rows) == 7 and all(r.endswith(",graph") for r in rows[1:]), rows


def test_bench_contract_one_gpu():
    res = _run([sys.executable, "bench.py", "--steps", "3", "--warmup", "3", "--sweep", "64"])
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    line = json.loads(res.stdout.strip().splitlines()[-1])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "e2e", "gpu_launches", "clocks"):
        assert key in line, key
    assert line["n_gpus"] == 1 and line["steps"] == 3 and line["gpu_launches"] == 3 * 1      # one persistent kernel per step
    assert line["value"] > 0 and line["e2e"]["value"] >= line["value"] * 0.5
    assert line["e2e"]["h2d_bytes_per_step"] == 8192 * 2312 + 4
    # the real-expert path and the all-to-all dispatcher are timed by child jobs and reported beside the headline
    assert set(line["fused_ms_by_global_batch"]) == {"64", "512", "4096"}, line.get("fused_detail")
    assert set(line["a2a_ms_by_global_batch"]) == {"1", "64", "512", "8192"}, line["a2a_ms_by_global_batch"]
