"""Token split, seeded generators, shape presets (CPU)."""
import pytest
import torch

from moe_comms_benchmarking_b200.config import Config
from moe_comms_benchmarking_b200.models.presets import get_preset
from moe_comms_benchmarking_b200.parallel.dist import all_rank_counts, local_token_count
from moe_comms_benchmarking_b200.utils.inputs import make_inputs, rank_counts, size_mb


def test_balanced_split():
    assert all_rank_counts(10, 4) == [3, 3, 2, 2]
    assert all_rank_counts(1, 4) == [1, 0, 0, 0]
    assert all_rank_counts(0, 3) == [0, 0, 0]
    for b in (1, 7, 64, 8191):
        for w in (1, 2, 4, 8):
            c = all_rank_counts(b, w)
            assert sum(c) == b and max(c) - min(c) <= 1
            assert c[0] == local_token_count(b, 0, w)


def test_config_properties_and_checks():
    cfg = Config(ep_size=8, per_rank_cap=16)
    assert cfg.num_local_experts == 64 and cfg.global_cap == 128
    with pytest.raises(ValueError):
        Config(num_experts=10, ep_size=4)
    with pytest.raises(ValueError):
        Config(num_experts=4, topk=8)


def test_presets():
    n = get_preset("nemotron-super")
    assert (n.num_experts, n.topk, n.hidden, n.num_layers) == (512, 22, 1024, 88)
    d = get_preset("deepseek-v3")
    assert (d.num_experts, d.topk, d.hidden, d.num_layers, d.probs) == (256, 8, 7168, 58, "sigmoid")
    with pytest.raises(ValueError):
        get_preset("nope")


def test_make_inputs_contract():
    cfg = Config(num_experts=64, topk=6, hidden=32, ep_size=2, rank=1, per_rank_cap=8)
    h, i, w = make_inputs(cfg, 9, "cpu")
    assert h.shape == (4, 32) and h.dtype == torch.bfloat16
    assert i.shape == (4, 6) and i.dtype == torch.int64
    assert w.dtype == torch.float32
    assert torch.allclose(w.sum(-1), torch.ones(4), atol=1e-5)
    for row in i.tolist():
        assert len(set(row)) == 6 and all(0 <= e < 64 for e in row)
    h2, i2, w2 = make_inputs(cfg, 9, "cpu")
    assert torch.equal(h, h2) and torch.equal(i, i2) and torch.equal(w, w2)
    cfg0 = Config(num_experts=64, topk=6, hidden=32, ep_size=2, rank=0, per_rank_cap=8)
    assert not torch.equal(make_inputs(cfg0, 9, "cpu")[1][:4], i)       # per-rank seed
    e = make_inputs(cfg, 1, "cpu")                                       # rank 1 idle at B=1
    assert e[0].shape == (0, 32) and e[1].shape == (0, 6) and e[2].shape == (0, 6)


def test_zipf_routing_is_skewed_and_distinct():
    cfg = Config(num_experts=128, topk=8, hidden=16, ep_size=1, per_rank_cap=512, routing="zipf")
    _, idx, _ = make_inputs(cfg, 512, "cpu")
    for row in idx.tolist():
        assert len(set(row)) == 8
    hist = torch.bincount(idx.flatten(), minlength=128).float()
    top = hist.sort(descending=True).values
    assert top[:8].sum() > 3 * top[-8:].sum()          # heavy head
    cfgu = Config(num_experts=128, topk=8, hidden=16, ep_size=1, per_rank_cap=512)
    histu = torch.bincount(make_inputs(cfgu, 512, "cpu")[1].flatten(), minlength=128).float()
    assert hist.max() > 2 * histu.max()


def test_sigmoid_probs_normalised():
    cfg = Config(num_experts=32, topk=4, hidden=16, probs="sigmoid", per_rank_cap=8)
    _, _, w = make_inputs(cfg, 8, "cpu")
    assert torch.allclose(w.sum(-1), torch.ones(8), atol=1e-5) and (w > 0).all()


def test_multinomial_counts_have_an_idle_rank():
    cfg = Config(ep_size=8, per_rank_cap=8192, counts="multinomial")
    for b in (1, 8, 256, 8192):
        c = rank_counts(cfg, b)
        assert sum(c) == b and min(c) == 0 and len(c) == 8
        assert c == rank_counts(cfg, b)
    assert rank_counts(Config(ep_size=4, per_rank_cap=4), 10) == [3, 3, 2, 2]


def test_size_mb():
    assert size_mb([1], torch.int32) == 1
    assert size_mb([1024, 1024], torch.bfloat16) == 2
    assert size_mb([1024, 1025], torch.bfloat16) == 3


def test_low_latency_limit_and_heap_sizing():
    from moe_comms_benchmarking_b200.ops.dense import agv_ll_stage_bytes, rsv_ll_stage_bytes
    from moe_comms_benchmarking_b200.parallel.dense import DenseDispatcher, resolve_ll_rows
    from moe_comms_benchmarking_b200.parallel.symm_heap import required_bytes
    assert resolve_ll_rows(Config(ep_size=1, per_rank_cap=64), -1) == 0           # nobody to talk to
    assert resolve_ll_rows(Config(ep_size=8, per_rank_cap=1024), -1) == 512
    assert resolve_ll_rows(Config(ep_size=8, per_rank_cap=4), -1) == 32           # never above the capacity
    assert resolve_ll_rows(Config(ep_size=2, per_rank_cap=4096), 100) == 100
    assert resolve_ll_rows(Config(ep_size=2, per_rank_cap=4096), 0) == 0
    # one 16-byte packet per 8 bytes of row, two parities
    assert agv_ll_stage_bytes(256, [2048, 176, 88]) == 2 * 256 * 289 * 16
    assert rsv_ll_stage_bytes(8, 256, 1024, 2048) == 2 * 8 * 256 * 256 * 16
    assert rsv_ll_stage_bytes(8, 256, 64, 2048) == 2 * 8 * 64 * 256 * 16
    cfg = Config(ep_size=8, per_rank_cap=1024)
    specs = DenseDispatcher.heap_specs(cfg)
    assert specs[0][0] == [2, 8192, 1024] and len(specs) == 7     # gathered rows: two layer parities
    assert required_bytes(specs) > 8192 * (2 * (2048 + 176 + 88) + 2048)


def test_all_to_all_packet_mode_limit_and_staging_sizes():
    from moe_comms_benchmarking_b200.ops.a2a import a2a_ll_specs, a2a_ll_words, a2a_meta_row_bytes
    from moe_comms_benchmarking_b200.parallel.a2a import A2ADispatcher, resolve_a2a_ll_rows
    assert resolve_a2a_ll_rows(Config(ep_size=1, per_rank_cap=64), -1) == 0
    assert resolve_a2a_ll_rows(Config(ep_size=8, per_rank_cap=1024), -1) == 1024
    assert resolve_a2a_ll_rows(Config(ep_size=8, per_rank_cap=4), -1) == 32          # never above the capacity
    assert resolve_a2a_ll_rows(Config(ep_size=2, per_rank_cap=4096), 0) == 0
    # a dispatched token: header word + row words + (e4m3: two scales per word) + metadata words
    meta = a2a_meta_row_bytes(22)
    assert meta % 16 == 0 and meta >= 8 + 8 * 22
    assert a2a_ll_words(1024, 22, False) == (1 + 256 + meta // 8, 256)
    assert a2a_ll_words(1024, 22, True) == (1 + 128 + 4 + meta // 8, 256)
    x, y, credits = a2a_ll_specs(8, 1024, 1024, 22, False, 256)
    xw, yw = a2a_ll_words(1024, 22, False)
    assert x[0] == [2 * 8 * 256 * xw * 16] and y[0] == [2 * 8 * 256 * yw * 16]       # two parities, one region per source
    assert a2a_ll_specs(8, 1024, 1024, 22, False, 0) == [] and a2a_ll_specs(1, 64, 1024, 22, False, 256) == []
    cfg = Config(ep_size=8, per_rank_cap=1024)
    assert len(A2ADispatcher.heap_specs(cfg, False, 0)) + 3 == len(A2ADispatcher.heap_specs(cfg, False, 256))
