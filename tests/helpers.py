"""Seeded synthetic inputs shared by the tests (CPU generator: identical bytes on every machine)."""
import numpy as np
import torch

from oracle import linear as olin


def f16_from_bits(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.view(np.float16).copy())


def bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def make_dense(M, N, K, seed=0, scheme="block", x_scale=1.0, w_std=0.02):
    """BASELINE-style synthetic layer: W ~ N(0, w_std) quantised per 128x128 block (scale = blockmax/448, fp32)
    or per output channel; x ~ N(0,1) * x_scale in FP16."""
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(N, K, generator=g) * w_std
    x = (torch.randn(M, K, generator=g) * x_scale).to(torch.float16)
    if scheme == "block":
        q8, s = olin.quantize_block_fp8(w)
        return x, q8, s, 128
    q8, s = olin.quantize_channel_fp8(w)
    s_grid = s.expand(N, -(-K // 128)).contiguous()
    return x, q8, s_grid, 1


def make_moe(E, I, H, M, topk, seed=0, scheme="block", invalid_frac=0.0):
    g = torch.Generator().manual_seed(seed)
    w13 = torch.randn(E, 2 * I, H, generator=g) * 0.02
    w2 = torch.randn(E, H, I, generator=g) * 0.02
    if scheme == "block":
        q13, s13 = zip(*[olin.quantize_block_fp8(w13[e]) for e in range(E)])
        q2, s2 = zip(*[olin.quantize_block_fp8(w2[e]) for e in range(E)])
        bh = 128
        s13, s2 = torch.stack(s13), torch.stack(s2)
    else:
        q13, s13 = zip(*[olin.quantize_channel_fp8(w13[e]) for e in range(E)])
        q2, s2 = zip(*[olin.quantize_channel_fp8(w2[e]) for e in range(E)])
        bh = 1
        s13 = torch.stack(s13).expand(E, 2 * I, -(-H // 128)).contiguous()
        s2 = torch.stack(s2).expand(E, H, -(-I // 128)).contiguous()
    q13, q2 = torch.stack(q13), torch.stack(q2)
    x = torch.randn(M, H, generator=g).to(torch.float16)
    logits = torch.randn(M, E, generator=g)
    ids = torch.stack([torch.randperm(E, generator=g)[:topk] for _ in range(M)]).to(torch.int32)
    tw = torch.softmax(torch.randn(M, topk, generator=g), dim=-1).float()
    if invalid_frac > 0:
        mask = torch.rand(M, topk, generator=g) < invalid_frac
        ids = torch.where(mask, torch.full_like(ids, -1), ids)
    return dict(x=x, w13=q13, s13=s13.to(torch.float16), w2=q2, s2=s2.to(torch.float16), ids=ids, tw=tw, logits=logits, bh=bh)
