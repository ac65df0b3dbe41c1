"""Routed mixture-of-experts oracle (test infrastructure).

* ``moe_reference_fp32`` restates the reference's MoE definition of correct:
  per token, per selected expert ``wt * (silu(x @ Wg^T) * (x @ Wu^T)) @ W2^T``
  in fp32 on dequantised weights
  (``tools/ct_fp8_mixed_moe_numtest_vllm021.sh:61-73``;
  ``tools/turbomind_ab/stage_d_full_moe.py:109-170``).  Acceptance, as in those
  scripts: cosine > 0.9999 and relative L2 < 2e-2.
* ``moe_reference_fp16_chain`` restates the arithmetic order of the reference's
  grouped path (``src/fp8_w8a16_sm70/vllm_serve.py:1862-1995``): w13 output
  rounded to FP16, ``silu(gate) * up`` on FP16 tensors, w2 output rounded to
  FP16, route weight cast to FP16 (``:1804``), ``index_add_`` into FP16 zeros.
* ``remap_expert_ids`` restates ``vllm_serve.py:2237-2243`` (global -> local ids,
  non-local -> -1, which contributes exactly zero).
* ``align_routes`` restates the sync-free route table of
  ``src/fp8_w8a16_sm70/compressed_tensors_v100.py:776-784`` (argsort by expert,
  scatter_add counts, cumsum offsets).
* ``route_topk`` — PARITY UNPINNED.  The reference never computes routing; it
  receives ``topk_ids`` / ``topk_weights`` from vLLM (pinned ``vllm==0.18.0``,
  ``pyproject.toml:14``; ``fused_topk`` -> ``topk_softmax``) and its own tests draw
  random ids.  The rule fixed here, following that published algorithm:
  fp32 softmax over the logits; the k largest are taken in descending order,
  ties to the lowest expert index (selection is done on the logits, which
  order exactly as their softmax values do); weights are the selected
  probabilities, renormalised to sum to one when ``renormalize`` is set.
"""

from __future__ import annotations

import numpy as np
import torch
import torch.nn.functional as F

from .dequant import dequant_block_scaled

COS_TOL = 0.9999
L2REL_TOL = 2e-2


def route_topk(logits: torch.Tensor, k: int, renormalize: bool = True):
    """logits [M,E] -> (ids int32 [M,k], weights fp32 [M,k]).  Parity unpinned."""
    lg = logits.detach().cpu().float()
    probs = torch.softmax(lg, dim=-1)
    order = torch.sort(lg, dim=-1, descending=True, stable=True).indices[:, :k]
    w = torch.gather(probs, 1, order)
    if renormalize:
        w = w / w.sum(dim=-1, keepdim=True)
    return order.to(torch.int32), w.float()


def remap_expert_ids(topk_ids: torch.Tensor, expert_map) -> torch.Tensor:
    """vllm_serve.py:2237-2243."""
    local = topk_ids.to(torch.long)
    if expert_map is None:
        return local
    safe = torch.clamp(local, min=0)
    mapped = expert_map.to(torch.long)[safe]
    return torch.where(topk_ids < 0, torch.full_like(mapped, -1), mapped)


def align_routes(expert_ids: torch.Tensor, num_experts: int):
    """Flat local expert ids [R] (invalid: <0 or >=E) ->
    (counts int32 [E], offsets int32 [E+1], sorted_route int32 [n_valid]).
    Order inside an expert is by ascending route index (stable)."""
    ids = expert_ids.detach().cpu().reshape(-1).to(torch.long)
    valid = (ids >= 0) & (ids < num_experts)
    key = torch.where(valid, ids, torch.full_like(ids, num_experts))
    order = torch.sort(key, stable=True).indices
    n_valid = int(valid.sum())
    counts = torch.bincount(ids[valid], minlength=num_experts)[:num_experts]
    offsets = torch.zeros(num_experts + 1, dtype=torch.long)
    offsets[1:] = torch.cumsum(counts, 0)
    return counts.to(torch.int32), offsets.to(torch.int32), order[:n_valid].to(torch.int32)


def _dq(w_u8: torch.Tensor, scales, bh: int, bw: int) -> torch.Tensor:
    E, N, K = w_u8.shape
    s = scales.detach().cpu()
    out = np.empty((E, N, K), dtype=np.float16)
    wn = w_u8.detach().cpu().numpy()
    for e in range(E):
        out[e] = dequant_block_scaled(wn[e], s[e], N, K, bh, bw)
    return torch.from_numpy(out)


def silu_mul(gate_up: torch.Tensor, I: int, activation: str = "silu") -> torch.Tensor:
    """vllm_serve.py:1627-1636 + :1953-1960: act(gate) * up with act = SiLU or GELU (erf form)."""
    act = F.silu if activation == "silu" else F.gelu
    return act(gate_up[..., :I]) * gate_up[..., I:]


def moe_reference_fp32(x, topk_w, topk_ids, w13_u8, s13, w2_u8, s2, block_h=128, block_w=128,
                       experts=None, activation: str = "silu") -> torch.Tensor:
    """fp32 reference, routed-only output [M,H] fp32.  Ids that are negative or
    >= E contribute zero.  ``experts`` optionally limits dequant to the experts
    actually hit (only a speed-up)."""
    x = x.detach().cpu().float()
    M, H = x.shape
    E, N13, _ = w13_u8.shape
    I = N13 // 2
    ids = topk_ids.detach().cpu().to(torch.long)
    tw = topk_w.detach().cpu().float()
    out = torch.zeros(M, H, dtype=torch.float32)
    hit = sorted(set(int(e) for e in ids.reshape(-1).tolist() if 0 <= int(e) < E))
    for e in hit:
        w13 = torch.from_numpy(dequant_block_scaled(w13_u8[e].cpu().numpy(), s13[e].cpu(), N13, H, block_h, block_w).copy()).float()
        w2 = torch.from_numpy(dequant_block_scaled(w2_u8[e].cpu().numpy(), s2[e].cpu(), H, I, block_h, block_w).copy()).float()
        tok, slot = torch.nonzero(ids == e, as_tuple=True)
        gu = x[tok] @ w13.T
        h = silu_mul(gu, I, activation)
        y = h @ w2.T
        out.index_add_(0, tok, y * tw[tok, slot].unsqueeze(-1))
    return out


def moe_reference_fp16_chain(x, topk_w, topk_ids, w13_u8, s13, w2_u8, s2, block_h=128, block_w=128) -> torch.Tensor:
    """Same layer with the reference grouped path's FP16 rounding points
    (vllm_serve.py:1862-1995); fp32 accumulation inside each GEMM."""
    x16 = x.detach().cpu().to(torch.float16)
    M, H = x16.shape
    E, N13, _ = w13_u8.shape
    I = N13 // 2
    ids = topk_ids.detach().cpu().to(torch.long)
    tw16 = topk_w.detach().cpu().to(torch.float16)
    out = torch.zeros(M, H, dtype=torch.float32)
    hit = sorted(set(int(e) for e in ids.reshape(-1).tolist() if 0 <= int(e) < E))
    for e in hit:
        w13 = torch.from_numpy(dequant_block_scaled(w13_u8[e].cpu().numpy(), s13[e].cpu(), N13, H, block_h, block_w).copy()).float()
        w2 = torch.from_numpy(dequant_block_scaled(w2_u8[e].cpu().numpy(), s2[e].cpu(), H, I, block_h, block_w).copy()).float()
        tok, slot = torch.nonzero(ids == e, as_tuple=True)
        gu = (x16[tok].float() @ w13.T).to(torch.float16)
        h = (F.silu(gu[:, :I].float()).to(torch.float16).float() * gu[:, I:].float()).to(torch.float16)
        y = (h.float() @ w2.T).to(torch.float16)
        y = (y.float() * tw16[tok, slot].float().unsqueeze(-1)).to(torch.float16)
        out.index_add_(0, tok, y.float())
    return out


def moe_error_stats(y: torch.Tensor, ref: torch.Tensor) -> dict:
    y = y.detach().cpu().double().flatten()
    ref = ref.detach().cpu().double().flatten()
    return {
        "l2rel": float((y - ref).norm() / ref.norm().clamp_min(1e-30)),
        "cos": float(F.cosine_similarity(y, ref, dim=0)) if ref.norm() > 0 else 1.0,
        "max_abs": float((y - ref).abs().max()) if y.numel() else 0.0,
    }


def check_moe(y: torch.Tensor, ref: torch.Tensor) -> dict:
    st = moe_error_stats(y, ref)
    assert torch.isfinite(y).all(), "non-finite MoE output"
    assert st["cos"] > COS_TOL, f"cos {st['cos']:.6f} <= {COS_TOL}"
    assert st["l2rel"] < L2REL_TOL, f"l2rel {st['l2rel']:.4g} >= {L2REL_TOL}"
    return st
