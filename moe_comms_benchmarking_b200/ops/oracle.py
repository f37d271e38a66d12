"""CPU oracle: plain fp32 PyTorch restatements of every kernel, used by the tests as the
ground truth for the CUDA kernels (the stand-in for a device-side sanitizer on machines
where none is available).  Every function takes the data of ALL ranks as lists."""
from __future__ import annotations

import torch


def metadata(counts: list[int]) -> list[list[int]]:
    """Per rank ``[valid, offset, max]`` (nvls/metadata.py:99-108)."""
    total, mx = sum(counts), max(counts) if counts else 0
    out, pre = [], 0
    for c in counts:
        out.append([total, pre, mx])
        pre += c
    return out


def all_gather_v(per_rank: list[torch.Tensor]) -> torch.Tensor:
    """Packed variable all-gather: rows of rank 0, then rank 1, ..."""
    return torch.cat(list(per_rank), dim=0)


def reduce_scatter_v(per_rank_full: list[torch.Tensor], counts: list[int], out_dtype=None) -> list[torch.Tensor]:
    """Sum the ranks' full ``[valid, H]`` tensors in fp32 and give each rank its own rows."""
    total = torch.stack([t.to(torch.float32) for t in per_rank_full]).sum(0)
    outs, pre = [], 0
    for c in counts:
        o = total[pre:pre + c]
        outs.append(o.to(out_dtype) if out_dtype is not None else o)
        pre += c
    return outs


def dest_rank_multiplicity(topk_idx: torch.Tensor, num_experts: int, world: int) -> torch.Tensor:
    """m[t] = number of distinct destination ranks of token t (owner = expert // (E / world))."""
    epr = num_experts // world
    if topk_idx.numel() == 0:
        return torch.zeros(0, dtype=torch.float32)
    owners = (topk_idx // epr).cpu()
    onehot = torch.zeros(owners.shape[0], world, dtype=torch.bool)
    onehot.scatter_(1, owners, True)
    return onehot.sum(1).to(torch.float32)


def roundtrip_identity(x: torch.Tensor, topk_idx: torch.Tensor, num_experts: int, world: int) -> torch.Tensor:
    """dispatch -> identity expert on every destination rank -> unweighted combine = m * x."""
    m = dest_rank_multiplicity(topk_idx, num_experts, world).view(-1, 1)
    return m * x.detach().cpu().to(torch.float32)


def a2a_dispatch(xs, idxs, num_experts: int, world: int):
    """Per destination rank d: list over sources s of (source token ids, rows) that s sends to d."""
    epr = num_experts // world
    recv = [[None] * world for _ in range(world)]
    for s in range(world):
        owners = idxs[s] // epr if idxs[s].numel() else idxs[s]
        for d in range(world):
            if idxs[s].numel():
                sel = (owners == d).any(dim=1).nonzero().flatten()
            else:
                sel = torch.zeros(0, dtype=torch.int64)
            recv[d][s] = (sel, xs[s][sel])
    return recv


def quant_e4m3_1x128(x: torch.Tensor):
    """1x128 block scaling: scale = amax / 448 per 128 columns (1 where the block is all zero),
    values = saturating round-to-nearest e4m3 of x / scale.  Returns (q float8, scale fp32)."""
    rows, h = x.shape
    xb = x.to(torch.float32).view(rows, h // 128, 128)
    amax = xb.abs().amax(dim=-1)
    scale = torch.where(amax > 0, amax / 448.0, torch.ones_like(amax))
    q = (xb / scale.unsqueeze(-1)).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
    return q.view(rows, h), scale


def dequant_e4m3_1x128(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    rows, h = q.shape
    return (q.to(torch.float32).view(rows, h // 128, 128) * scale.unsqueeze(-1)).view(rows, h)


def rs_add_norm_ag(partials: list[torch.Tensor], residuals: list[torch.Tensor], weight: torch.Tensor, eps: float):
    """Returns (normalised [tokens, H] fp32 that every rank ends with, new residual per rank).
    Rounding points follow the kernel: bf16 sum, bf16 residual add, fp32 norm, bf16 result."""
    world = len(partials)
    total = torch.stack([p.to(torch.float32) for p in partials]).sum(0).to(torch.bfloat16)
    tpr = total.shape[0] // world
    new_res, normed = [], []
    for r in range(world):
        s = (total[r * tpr:(r + 1) * tpr].to(torch.float32) + residuals[r].to(torch.float32)).to(torch.bfloat16)
        new_res.append(s)
        sf = s.to(torch.float32)
        rrms = torch.rsqrt(sf.pow(2).mean(dim=-1, keepdim=True) + eps)
        normed.append((sf * rrms * weight.to(torch.float32)).to(torch.bfloat16).to(torch.float32))
    return torch.cat(normed, 0), new_res


def swiglu_ffn(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    """One expert: ``down(silu(x Wg^T) * (x Wu^T))`` with ``w_gate_up = [2I, H]`` (gate rows then
    up rows) and ``w_down = [H, I]``.  fp32 math on bf16-rounded inputs; the intermediate is
    rounded to bf16 as the kernels store it."""
    xf, wgu, wd = x.to(torch.float32), w_gate_up.to(torch.float32), w_down.to(torch.float32)
    inter = wgu.shape[0] // 2
    gu = xf @ wgu.t()
    act = (torch.nn.functional.silu(gu[:, :inter]) * gu[:, inter:]).to(torch.bfloat16).to(torch.float32)
    return act @ wd.t()


def moe_layer(x_all: torch.Tensor, idx_all: torch.Tensor, w_all: torch.Tensor, w_gate_up: torch.Tensor,
              w_down: torch.Tensor) -> torch.Tensor:
    """Full MoE layer over ALL tokens and ALL experts: out[t] = sum_k w[t,k] * FFN_{idx[t,k]}(x[t])."""
    out = torch.zeros(x_all.shape[0], w_down.shape[1], dtype=torch.float32)
    for e in range(w_gate_up.shape[0]):
        tok, k = (idx_all == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        y = swiglu_ffn(x_all[tok], w_gate_up[e], w_down[e])
        out.index_add_(0, tok, y * w_all[tok, k].to(torch.float32).unsqueeze(-1))
    return out
