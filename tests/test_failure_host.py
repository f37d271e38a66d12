"""Failure detection without touching a GPU: a rank that never joins, a capture that fails,
a clock record that shows throttling."""
import os
import subprocess
import sys
import textwrap

from conftest import ROOT, free_port

from moe_comms_benchmarking_b200.utils.clocks import parse_samples


def test_missing_rank_ends_with_an_error_not_a_hang(tmp_path):
    """World of 2 where rank 1 never starts: rank 0's rendezvous must give up within its
    timeout and exit non-zero."""
    script = tmp_path / "lonely.py"
    script.write_text(textwrap.dedent(f"""
        import os, sys
        sys.path.insert(0, {ROOT!r})
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT="{free_port()}", RANK="0", WORLD_SIZE="2", LOCAL_RANK="0")
        from moe_comms_benchmarking_b200.parallel.dist import init_distributed
        try:
            g, r, w, _ = init_distributed(backend="gloo", timeout_s=3)
            import torch, torch.distributed as dist
            dist.all_reduce(torch.zeros(1))
        except Exception as e:
            print("DETECTED", type(e).__name__)
            sys.exit(7)
        sys.exit(0)
    """))
    res = subprocess.run([sys.executable, str(script)], capture_output=True, text=True, timeout=120,
                         env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    assert res.returncode == 7 and "DETECTED" in res.stdout, res.stdout + res.stderr


def test_graph_capture_failure_falls_back_to_eager(monkeypatch):
    from moe_comms_benchmarking_b200.utils import timing
    calls = []

    def fake_time_region(fn, group, warmup, iters, use_graph):
        calls.append(use_graph)
        if use_graph:
            raise RuntimeError("capture is not permitted")
        return 1.0, 2.0

    monkeypatch.setattr(timing, "time_region", fake_time_region)
    monkeypatch.setattr(timing.dist, "barrier", lambda group=None: None)
    logs = []
    (local, mx), used = timing.timed_with_fallback(lambda: None, None, 1, 1, "graph", 0,
                                                   log=lambda *a, **k: logs.append(a[0]))
    assert calls == [True, False] and not used and (local, mx) == (1.0, 2.0)
    assert "falling back to eager" in logs[0]


def test_clock_samples_parse_and_flag_throttling():
    text = ("0, 1350, 1965, 990.1, 0x0000000000000004, Not Active, Not Active, Not Active, Active\n"
            "0, 1400, 1965, 1001.0, 0x0, Not Active, Not Active, Not Active, Not Active\n"
            "0, 900, 1965, 500.0, 0x8, Active, Not Active, Not Active, Not Active\n")
    c = parse_samples(text)
    assert c["sm_mhz"] == 1350 and c["sm_max_mhz"] == 1965 and c["samples"] == 3
    assert c["reasons"] == ["hw_slowdown", "sw_power_cap"]
    assert parse_samples("")["samples"] == 0
