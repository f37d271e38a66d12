"""Real multi-GPU runs (skipped where fewer than two GPUs are visible): the driver's
--validate on every transport, and a rank that leaves between steps."""
import os
import subprocess
import sys
import textwrap

import pytest
import torch

from conftest import ROOT, free_port

pytestmark = pytest.mark.gpu


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _torchrun(n, script_args, env=None, timeout=900):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(n), "--master-addr",
           "127.0.0.1", "--master-port", str(free_port())] + script_args
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, cwd=ROOT,
                          env=dict(os.environ, **(env or {})))


@pytest.mark.parametrize("transport", ["auto", "p2p"])
def test_validate_all_impls_multi_gpu(transport):
    n = _ngpu()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    n = 8 if n >= 8 else (4 if n >= 4 else 2)
    res = _torchrun(n, ["run.py", "--impl", "all", "--validate", "--transport", transport])
    assert res.returncode == 0, res.stdout[-4000:] + res.stderr[-4000:]
    assert f"# VALIDATION PASSED (all {n} ranks)" in res.stdout


@pytest.mark.parametrize("transport", ["auto", "p2p"])
def test_tensor_parallel_collectives_multi_gpu(transport):
    n = _ngpu()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    n = 4 if n >= 4 else 2
    res = _torchrun(n, ["-m", "moe_comms_benchmarking_b200.selftest", "--transport", transport])
    assert res.returncode == 0, res.stdout[-4000:] + res.stderr[-4000:]
    assert f"# SELFTEST PASSED (all {n} ranks" in res.stdout


def test_fp8_dispatch_on_both_paths_multi_gpu():
    """1 x 128 block-scaled e4m3 dispatch on the dense path and on the all-to-all path, each against its
    own checks and against each other (cross-impl [a2a-fp8=dense-fp8])."""
    n = _ngpu()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    n = 4 if n >= 4 else 2
    res = _torchrun(n, ["run.py", "--impl", "both", "--validate", "--dispatch-dtype", "fp8"])
    assert res.returncode == 0, res.stdout[-4000:] + res.stderr[-4000:]
    assert f"# VALIDATION PASSED (all {n} ranks)" in res.stdout
    assert "cross-impl [a2a-fp8=dense-fp8]" in res.stdout


@pytest.mark.parametrize("extra", [[], ["--no-layer-kernel"], ["--transport", "p2p"]])
def test_fused_experts_validate_multi_gpu(extra):
    n = _ngpu()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    res = _torchrun(2, ["run.py", "--impl", "fused", "--validate", "--num-experts", "64", "--topk", "6",
                        "--hidden", "512", "--intermediate", "256"] + extra)
    assert res.returncode == 0, res.stdout[-4000:] + res.stderr[-4000:]
    assert "# VALIDATION PASSED (all 2 ranks)" in res.stdout


def test_extended_baseline_validate_multi_gpu():
    """NCCL + library GEMMs with real experts (the extended baseline of the fused path) against the oracle."""
    n = _ngpu()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    res = _torchrun(2, ["run.py", "--impl", "nccl", "--expert", "swiglu", "--validate", "--num-experts", "64", "--topk", "6",
                        "--hidden", "512", "--intermediate", "256"])
    assert res.returncode == 0, res.stdout[-4000:] + res.stderr[-4000:]
    assert "# VALIDATION PASSED (all 2 ranks)" in res.stdout


def test_rank_leaving_between_steps_is_seen_on_the_host(tmp_path):
    """Rank 1 announces that it leaves after step 2 (nothing in flight) and exits; rank 0 reads
    the announcement before its next launch and stops instead of waiting in a kernel.  No rank's
    memory is bound to an NVSwitch multicast object (the heap is built with multicast=False and the
    script checks that no multicast address exists before anyone may leave), NCCL's NVLS is off, and
    the kernels use plain peer access, as required when a rank may disappear."""
    if _ngpu() < 2:
        pytest.skip("needs at least 2 GPUs")
    script = tmp_path / "leaver.py"
    script.write_text(textwrap.dedent(f"""
        import os, sys, time
        sys.path.insert(0, {ROOT!r})
        import torch, torch.distributed as dist
        from moe_comms_benchmarking_b200.config import Config
        from moe_comms_benchmarking_b200.parallel.dense import DenseDispatcher
        from moe_comms_benchmarking_b200.parallel.dist import init_distributed
        from moe_comms_benchmarking_b200.parallel.health import Membership, RankLeft
        from moe_comms_benchmarking_b200.parallel.symm_heap import SymmetricHeap, required_bytes
        from moe_comms_benchmarking_b200.utils.inputs import make_inputs
        group, rank, world, lr = init_distributed(timeout_s=20)
        cfg = Config(ep_size=world, rank=rank, local_rank=lr, per_rank_cap=8)
        try:
            heap = SymmetricHeap(group, required_bytes(DenseDispatcher.heap_specs(cfg)), f"cuda:{{lr}}",
                                 transport="p2p", multicast=False)
            bound = torch.tensor([1.0 if heap.mc_ptr else 0.0], device=f"cuda:{{lr}}")
        except RuntimeError as e:
            print(f"rank {{rank}}: {{e}}", flush=True)
            bound = torch.tensor([1.0], device=f"cuda:{{lr}}")
        dist.all_reduce(bound, op=dist.ReduceOp.MAX)
        if bound.item() > 0:
            # Some rank still has a multicast binding: nobody leaves; every rank shuts down in order.
            print("MULTICAST_STILL_BOUND", flush=True)
            dist.barrier()
            dist.destroy_process_group()
            sys.exit(77)
        d = DenseDispatcher(cfg, group, heap=heap, transport="p2p")
        d.build()
        d.heap.set_timeout(1.0)
        d._make_plans()
        h, i, w = make_inputs(cfg, 8 * world, f"cuda:{{lr}}")
        d.setup_batch(h, i, w)
        mem = Membership(rank, world)
        dist.barrier()
        code = 0
        for step in range(6):
            try:
                mem.check()
            except RankLeft as e:
                print(f"rank {{rank}} saw {{e}} before step {{step}}", flush=True)
                code = 42
                break
            d.decode_step(2)
            torch.cuda.synchronize()
            d.check_health()
            mem.beat(step)
            if rank == 1 and step == 2:
                mem.leave()
                break
            time.sleep(0.3 if rank == 0 else 0.0)
        os._exit(code)
    """))
    res = _torchrun(2, [str(script)], env={"NCCL_NVLS_ENABLE": "0", "TORCH_SYMM_MEM_DISABLE_MULTICAST": "1"},
                    timeout=300)
    out = res.stdout + res.stderr
    if "MULTICAST_STILL_BOUND" in out:
        pytest.skip("this PyTorch binds a multicast object regardless; a rank departure is not exercised on GPUs")
    assert "rank 0 saw rank(s) [1] left the job" in out, out[-4000:]


def test_native_heap_allocator_multi_gpu():
    """The library's own symmetric-heap allocator (driver virtual-memory API, descriptors over unix sockets,
    one multicast object) under both dispatchers and the tensor-parallel collectives: the same checks as with
    PyTorch's allocator, and the heap must have a multicast address of its own."""
    n = _ngpu()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    n = 4 if n >= 4 else 2
    env = {"MCB_HEAP_ALLOCATOR": "native"}
    res = _torchrun(n, ["run.py", "--impl", "both", "--validate"], env=env)
    assert res.returncode == 0, res.stdout[-4000:] + res.stderr[-4000:]
    assert f"# VALIDATION PASSED (all {n} ranks)" in res.stdout
    res = _torchrun(n, ["-m", "moe_comms_benchmarking_b200.selftest"], env=env)
    assert res.returncode == 0, res.stdout[-4000:] + res.stderr[-4000:]
    assert f"# SELFTEST PASSED (all {n} ranks, transport=multimem" in res.stdout
