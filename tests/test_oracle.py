"""The CPU oracle itself (it is the ground truth of every GPU test)."""
import math

import torch

from moe_comms_benchmarking_b200.ops import oracle


def test_metadata():
    assert oracle.metadata([3, 0, 2]) == [[5, 0, 3], [5, 3, 3], [5, 3, 3]]


def test_gather_and_reduce_scatter():
    a, b = torch.arange(6.).view(3, 2), torch.arange(4.).view(2, 2) + 10
    full = oracle.all_gather_v([a, b])
    assert full.shape == (5, 2) and torch.equal(full[3:], b)
    outs = oracle.reduce_scatter_v([full, full * 2], [3, 2])
    assert torch.equal(outs[0], a * 3) and torch.equal(outs[1], b * 3)


def test_multiplicity_expectation():
    # E[m] = W * (1 - C(E - E/W, K) / C(E, K)); (16 experts, top-4, 2 ranks) -> 1.92
    g = torch.Generator().manual_seed(0)
    idx = torch.stack([torch.randperm(16, generator=g)[:4] for _ in range(4000)])
    m = oracle.dest_rank_multiplicity(idx, 16, 2)
    want = 2 * (1 - math.comb(8, 4) / math.comb(16, 4))
    assert abs(float(m.mean()) - want) < 0.03
    x = torch.randn(4000, 8)
    assert torch.equal(oracle.roundtrip_identity(x, idx, 16, 2), m.view(-1, 1) * x)


def test_a2a_dispatch_lists():
    idx = [torch.tensor([[0, 1], [0, 3]]), torch.tensor([[2, 3]])]
    xs = [torch.tensor([[1.], [2.]]), torch.tensor([[3.]])]
    recv = oracle.a2a_dispatch(xs, idx, 4, 2)
    assert recv[0][0][0].tolist() == [0, 1] and recv[1][0][0].tolist() == [1]
    assert recv[0][1][0].tolist() == [] and recv[1][1][1].tolist() == [[3.]]


def test_fp8_block_quant_roundtrip():
    x = torch.randn(5, 256) * torch.tensor([0.01, 1.0, 50.0, 0.0, 3.0]).view(5, 1)
    q, s = oracle.quant_e4m3_1x128(x)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (5, 2)
    back = oracle.dequant_e4m3_1x128(q, s)
    err = (back - x).abs()
    assert (err <= 0.0625 * x.abs() + 1e-3 * s.repeat_interleave(128, dim=1) + 1e-12).all()
    assert torch.equal(back[3], torch.zeros(256)) and torch.equal(s[3], torch.ones(2))


def test_swiglu_and_moe_layer_agree():
    g = torch.Generator().manual_seed(1)
    E, H, I, T, K = 4, 16, 8, 6, 2
    wgu = (torch.randn(E, 2 * I, H, generator=g) * 0.1).to(torch.bfloat16)
    wd = (torch.randn(E, H, I, generator=g) * 0.1).to(torch.bfloat16)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)])
    w = torch.rand(T, K, generator=g)
    out = oracle.moe_layer(x, idx, w, wgu, wd)
    t = 3
    want = sum(w[t, k] * oracle.swiglu_ffn(x[t:t + 1], wgu[idx[t, k]], wd[idx[t, k]])[0] for k in range(K))
    assert torch.allclose(out[t], want, atol=1e-5)


def test_rs_add_norm_ag_shapes():
    g = torch.Generator().manual_seed(2)
    parts = [torch.randn(4, 16, generator=g).to(torch.bfloat16) for _ in range(2)]
    res = [torch.randn(2, 16, generator=g).to(torch.bfloat16) for _ in range(2)]
    wt = torch.ones(16, dtype=torch.bfloat16)
    normed, new_res = oracle.rs_add_norm_ag(parts, res, wt, 1e-5)
    assert normed.shape == (4, 16) and new_res[1].shape == (2, 16)
    assert torch.allclose(normed.pow(2).mean(-1), torch.ones(4), atol=3e-2)
