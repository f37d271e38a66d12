"""Driver logic that needs neither GPUs nor a process group: the cross-implementation check and
property tests of the generators and the oracle."""
import importlib

import torch
from hypothesis import given, settings, strategies as st

from moe_comms_benchmarking_b200.config import Config
from moe_comms_benchmarking_b200.ops import oracle
from moe_comms_benchmarking_b200.parallel.dist import all_rank_counts
from moe_comms_benchmarking_b200.utils.inputs import make_inputs, rank_counts


class _FakeBencher:
    """Computes the round trip analytically; ``scale`` != 1 models a broken implementation."""

    def __init__(self, name, cfg, scale=1.0):
        self.name, self.cfg, self.scale = name, cfg, scale

    def functional_roundtrip(self, x, idx):
        return oracle.roundtrip_identity(x, idx, self.cfg.num_experts, self.cfg.ep_size) * self.scale


def test_cross_impl_check_accepts_agreeing_and_rejects_diverging_implementations():
    run = importlib.import_module("run")
    cfg = Config(num_experts=16, topk=4, hidden=32, ep_size=4, rank=1, per_rank_cap=8)
    lines = []
    good = [_FakeBencher("a", cfg), _FakeBencher("b", cfg, 1.001)]
    assert run.cross_impl_check(good, cfg, 4, 1, torch.device("cpu"), lines.append)
    assert lines == []                       # rank 1 prints only failures
    bad = [_FakeBencher("a", cfg), _FakeBencher("b", cfg, 1.2)]
    assert not run.cross_impl_check(bad, cfg, 4, 1, torch.device("cpu"), lines.append)
    assert any("[FAIL] cross-impl [a=b]" in l for l in lines)
    assert run.cross_impl_check([_FakeBencher("only", cfg)], cfg, 4, 1, torch.device("cpu"), lines.append)


@settings(max_examples=40, deadline=None)
@given(b=st.integers(0, 5000), w=st.sampled_from([1, 2, 4, 8, 16]))
def test_balanced_split_properties(b, w):
    c = all_rank_counts(b, w)
    assert sum(c) == b and max(c) - min(c) <= 1 and c == sorted(c, reverse=True)


@settings(max_examples=25, deadline=None)
@given(b=st.integers(1, 300), w=st.sampled_from([2, 4, 8]), seed=st.integers(0, 1000))
def test_multinomial_split_properties(b, w, seed):
    cfg = Config(ep_size=w, per_rank_cap=b, counts="multinomial", seed=seed)
    c = rank_counts(cfg, b)
    assert sum(c) == b and min(c) == 0 and max(c) <= b and all(v >= 0 for v in c)


@settings(max_examples=20, deadline=None)
@given(n=st.integers(1, 40), k=st.integers(1, 8), w=st.sampled_from([1, 2, 4]), seed=st.integers(0, 99))
def test_roundtrip_multiplicity_bounds(n, k, w, seed):
    e = 8 * w
    cfg = Config(num_experts=e, topk=min(k, e), hidden=8, ep_size=w, rank=0, per_rank_cap=n * w, seed=seed)
    x, idx, wts = make_inputs(cfg, n * w, "cpu")
    m = oracle.dest_rank_multiplicity(idx, e, w)
    assert (m >= 1).all() and (m <= min(cfg.topk, w)).all()
    assert torch.allclose(wts.sum(-1), torch.ones(idx.shape[0]), atol=1e-5)
    recv = oracle.a2a_dispatch([x] + [x[:0]] * (w - 1), [idx] + [idx[:0]] * (w - 1), e, w)
    assert sum(recv[d][0][0].numel() for d in range(w)) == int(m.sum())


@settings(max_examples=20, deadline=None)
@given(rows=st.integers(1, 6), blocks=st.integers(1, 4), scale=st.floats(1e-3, 1e3))
def test_block_quant_error_bound(rows, blocks, scale):
    x = torch.randn(rows, blocks * 128, generator=torch.Generator().manual_seed(rows * 7 + blocks)) * scale
    q, s = oracle.quant_e4m3_1x128(x)
    back = oracle.dequant_e4m3_1x128(q, s)
    amax = x.view(rows, blocks, 128).abs().amax(-1)
    assert torch.allclose(s, torch.where(amax > 0, amax / 448, torch.ones_like(amax)))
    assert ((back - x).abs() <= 0.0625 * x.abs() + 2e-3 * s.repeat_interleave(128, dim=1)).all()


def test_bench_child_job_csv_is_parsed(monkeypatch, tmp_path):
    """bench.py times the expert path and the all-to-all dispatcher through run.py in a child job and reads
    the child's CSV: the command line names the implementation and the batches, rows of other
    implementations or phases are ignored, a failing child raises."""
    import subprocess
    import sys
    import os
    import pytest
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import bench
    seen = {}

    def fake_run(cmd, **kw):
        seen["cmd"] = cmd
        out = cmd[cmd.index("--out") + 1]
        with open(out, "w") as f:
            f.write("impl,global_B,num_sms,phase,per_rank_counts,latency_us,timing\n")
            f.write('a2a,1,148,decode_step,"[1, 0]",610.5,graph\n')
            f.write('a2a,64,148,dispatch,"[32, 32]",5.0,graph\n')
            f.write('dense,64,148,decode_step,"[32, 32]",590.0,graph\n')
            f.write('a2a,64,148,decode_step,"[32, 32]",713.72,graph\n')
        return subprocess.CompletedProcess(cmd, seen.get("rc", 0), "", "boom")

    monkeypatch.setattr(subprocess, "run", fake_run)
    ms = bench.run_child(2, "a2a", [1, 64], ["--reps", "10"])
    assert ms == {"1": 0.6105, "64": 0.7137}
    cmd = seen["cmd"]
    assert cmd[cmd.index("--impl") + 1] == "a2a" and cmd[cmd.index("--batch-sizes") + 1] == "1,64"
    assert cmd[cmd.index("--nproc-per-node") + 1] == "2" and "--reps" in cmd
    seen["rc"] = 3
    with pytest.raises(RuntimeError):
        bench.run_child(2, "a2a", [1], [])
