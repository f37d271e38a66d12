"""Command line, row formats, CSV append/resume, plot loader (CPU)."""
import importlib
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from moe_comms_benchmarking_b200.utils.report import CSV_HEADER, CsvSink, Row, load_rows  # noqa: E402


def test_cli_defaults_match_reference_driver():
    run = importlib.import_module("run")
    a = run.parse_args([])
    assert a.impl == "all" and a.batch_sizes == "1,2,4,8,16,32,64,128"
    assert a.deepep_num_sms == "148" and a.reps == 100 and a.warmup == 20
    assert a.timing == "graph" and a.seed == 1234 and a.out is None and not a.validate
    cfg, nl = run.make_config(a, 4, 1, 1, [1, 128])
    assert (cfg.num_experts, cfg.topk, cfg.hidden, nl) == (512, 22, 1024, 88)
    assert cfg.per_rank_cap == 32
    for alias, want in (("nvls", ["dense"]), ("deepep", ["a2a"]), ("both", ["a2a", "dense"]),
                        ("all", ["a2a", "dense", "nccl"])):
        assert run.resolve_impls(alias, True) == want
    assert run.resolve_impls("all", False) == ["gloo"]
    # real experts: the fused path and the extended NCCL baseline
    assert run.resolve_impls("dense", True, "swiglu") == ["fused"]
    assert run.resolve_impls("nccl", True, "swiglu") == ["nccl-swiglu"]
    with pytest.raises(SystemExit):
        run.resolve_impls("a2a", True, "swiglu")
    with pytest.raises(SystemExit):
        run.parse_args(["--impl", "bogus"])
    a = run.parse_args(["--model", "deepseek-v3", "--num-layers", "3", "--dispatch-dtype", "fp8"])
    cfg, nl = run.make_config(a, 8, 0, 0, [4096])
    assert (cfg.num_experts, cfg.topk, cfg.hidden, cfg.probs, nl) == (256, 8, 7168, "sigmoid", 3)


def test_row_formats():
    r = Row("dense", 16, 148, "decode_step", [4, 4, 4, 4], 1234.5678, True)
    assert r.csv_line() == 'dense,16,148,decode_step,"[4, 4, 4, 4]",1234.5678,graph'
    assert r.stdout_csv_line() == "dense,16,148,decode_step,1234.568,graph"
    line = r.progress_line(88)
    assert "B=  16 sms=148 counts=[4, 4, 4, 4] decode_step(88L)=  1234.57us (per-layer= 14.03us)  [graph]" in line
    assert " sms= na" in Row("nccl", 1, -1, "decode_step", [1], 5.0, False).progress_line(88)


def test_csv_sink_append_and_resume(tmp_path):
    path = str(tmp_path / "r.csv")
    s = CsvSink(path)
    s.add(Row("dense", 1, 148, "decode_step", [1, 0], 10.0, True))
    s.add(Row("nccl", 1, -1, "decode_step", [1, 0], 99.5, False))
    text = open(path).read().splitlines()
    assert text[0] == CSV_HEADER and len(text) == 3
    s2 = CsvSink(path, resume=True)
    assert ("dense", 1, 148, "decode_step") in s2.done and len(s2.rows) == 2
    s2.add(Row("dense", 2, 148, "decode_step", [1, 1], 11.0, True))
    rows = load_rows(path)
    assert [r.global_b for r in rows] == [1, 1, 2] and rows[1].counts == [1, 0] and not rows[1].used_graph


def test_plot_loader_and_ticks(tmp_path, capsys):
    plot = importlib.import_module("plot_results")
    path = str(tmp_path / "r.csv")
    s = CsvSink(path)
    s.add(Row("dense", 1024, 148, "decode_step", [256] * 4, 1550.0, True))
    s.add(Row("dense", 1 << 20, 148, "decode_step", [1 << 18] * 4, 787030.0, True))
    s.add(Row("nccl", 1024, -1, "other_phase", [256] * 4, 1.0, True))
    rows, ep = plot.load(path)
    assert ep == 4 and len(rows) == 2 and abs(rows[0]["ms"] - 1.55) < 1e-9
    assert [plot.ktick(v) for v in (1, 512, 1024, 131072, 1 << 20)] == ["1", "512", "1k", "128k", "1M"]
    assert "EP=4" in plot.subtitle(4)
    assert plot.main(["--csv", path, "--out", str(tmp_path / "o.png")]) == 0
    out = capsys.readouterr().out
    assert "wrote" in out
    svg = plot.render_svg(rows, "title line 1\ntitle line 2")
    import xml.dom.minidom
    doc = xml.dom.minidom.parseString(svg)
    assert len(doc.getElementsByTagName("polyline")) == 1          # one implementation
    texts = [t.firstChild.data for t in doc.getElementsByTagName("text") if t.firstChild]
    assert "1k" in texts and "1M" in texts and "787.03" in texts    # tick labels and last-point annotation


def test_phase_tracing(monkeypatch, capsys):
    from moe_comms_benchmarking_b200.utils import trace
    trace.clear()
    monkeypatch.setenv("MCB_TRACE", "1")
    with trace.phase("unit-test phase"):
        pass
    assert trace.records()[-1][0] == "unit-test phase" and trace.records()[-1][1] >= 0
    assert "# [trace] unit-test phase:" in capsys.readouterr().out
    monkeypatch.setenv("MCB_TRACE", "0")
    with trace.phase("quiet"):
        pass
    assert "quiet" not in capsys.readouterr().out
