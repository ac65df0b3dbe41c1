"""On-disk formats either side of the hot path: reading FP8 checkpoints into the layouts the engine takes.

Two families, as the reference serves them:

* native ``quant_method = fp8``: per linear ``<prefix>.weight`` (F8_E4M3 ``[N, K]``) and ``<prefix>.weight_scale_inv``
  (BF16 / F32 ``[ceil(N/128), ceil(K/128)]``) — what ``FP8W8A16Linear.from_safetensors`` reads
  (``src/fp8_w8a16_sm70/module.py:65-89``) and what vLLM hands to ``process_weights_after_loading``
  (``src/fp8_w8a16_sm70/vllm_serve.py:1450-1523``);
* compressed-tensors: ``<prefix>.weight`` plus ``<prefix>.weight_scale`` that is ``[N/128, K/128]`` (block), ``[N, 1]``
  (channel) or a scalar per logical shard (tensor) (``src/fp8_w8a16_sm70/compressed_tensors_v100.py:231-270``).

Fused modules are built the way vLLM's merged parameters lay them out: Q, K, V (or gate, up) concatenated along the
output dimension together with their scale rows (``tests/test_attention_shapes.py:97-101``); MoE experts stacked into
``w13 [E, 2I, H]`` (gate rows then up rows) and ``w2 [E, H, I]`` (``tools/turbomind_ab/stage_d_full_moe.py:73-81``).

Everything here is host-side bookkeeping on tensors: bytes are never re-quantised or re-scaled, scales are cast to FP16
exactly once (the cast the reference does at load), and a layout this engine cannot serve raises instead of being
converted silently.
"""

from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, Iterable, List, Optional, Sequence, Tuple, Union

import torch

BLOCK = 128


# ------------------------------------------------------------------------------------------------
# tensor source: one .safetensors file, or a directory with model.safetensors.index.json
# ------------------------------------------------------------------------------------------------
class TensorSource:
    """Random access to the tensors of a checkpoint by name, without loading whole files."""

    def __init__(self, path: Union[str, Path]):
        self.path = Path(path)
        self._key_to_file: Dict[str, Path] = {}
        self._open: Dict[Path, object] = {}
        if self.path.is_dir():
            index = self.path / "model.safetensors.index.json"
            if index.exists():
                wmap = json.loads(index.read_text())["weight_map"]
                self._key_to_file = {k: self.path / v for k, v in wmap.items()}
            else:
                for f in sorted(self.path.glob("*.safetensors")):
                    for k in self._handle(f).keys():
                        self._key_to_file[k] = f
        elif self.path.suffix == ".safetensors" and self.path.exists():
            for k in self._handle(self.path).keys():
                self._key_to_file[k] = self.path
        else:
            raise FileNotFoundError(f"{self.path}: not a .safetensors file or a checkpoint directory")

    def _handle(self, f: Path):
        if f not in self._open:
            from safetensors import safe_open
            self._open[f] = safe_open(f, framework="pt")
        return self._open[f]

    def keys(self) -> Iterable[str]:
        return self._key_to_file.keys()

    def __contains__(self, key: str) -> bool:
        return key in self._key_to_file

    def get(self, key: str) -> torch.Tensor:
        if key not in self._key_to_file:
            raise KeyError(f"{key!r} is not in {self.path}")
        return self._handle(self._key_to_file[key]).get_tensor(key)


Source = Union[TensorSource, Dict[str, torch.Tensor], str, Path]


def _src(src: Source):
    if isinstance(src, (str, Path)):
        return TensorSource(src)
    return src


def _get(src, key: str) -> torch.Tensor:
    if isinstance(src, TensorSource):
        return src.get(key)
    if key not in src:
        raise KeyError(f"{key!r} is not in the state dict")
    return src[key]


# ------------------------------------------------------------------------------------------------
# one linear
# ------------------------------------------------------------------------------------------------
@dataclass
class Fp8Weight:
    """A linear as the engine takes it: raw E4M3 bytes ``[N, K]`` and an FP16 scale grid ``[ceil(N/block_h), ceil(K/128)]``
    (``block_h = 128``: block scales; ``block_h = 1``: one scale per output row, repeated over the K blocks)."""
    weight: torch.Tensor
    scale: torch.Tensor
    block_h: int
    bias: Optional[torch.Tensor] = None
    logical_widths: List[int] = field(default_factory=list)

    @property
    def N(self) -> int:
        return int(self.weight.shape[0])

    @property
    def K(self) -> int:
        return int(self.weight.shape[1])

    def to(self, device) -> "Fp8Weight":
        return Fp8Weight(self.weight.to(device), self.scale.to(device), self.block_h,
                         None if self.bias is None else self.bias.to(device), list(self.logical_widths))


def _as_bytes(w: torch.Tensor) -> torch.Tensor:
    if w.dtype == torch.uint8:
        return w.contiguous()
    if w.dtype == torch.float8_e4m3fn:
        return w.contiguous().view(torch.uint8)
    raise ValueError(f"weight dtype {w.dtype} is not FP8 E4M3 (float8_e4m3fn or raw uint8)")


def _fp16_scale(s: torch.Tensor, what: str) -> torch.Tensor:
    s16 = s.to(torch.float16)
    if s16.numel() and not bool(torch.isfinite(s16).all()):
        raise ValueError(f"{what}: scale is not representable in FP16 (inf / nan after the cast)")
    return s16.contiguous()


def block_weight(weight: torch.Tensor, scale: torch.Tensor, bias: Optional[torch.Tensor] = None,
                 block=(BLOCK, BLOCK), what: str = "linear") -> Fp8Weight:
    """Block-128 layout (native ``weight_scale_inv`` and compressed-tensors BLOCK ``weight_scale`` are the same numbers:
    dequantised weight = fp8 value x block scale, compressed_tensors_v100.py:307-312)."""
    if tuple(block) != (BLOCK, BLOCK):
        raise NotImplementedError(f"{what}: weight_block_size {tuple(block)} is not supported (only [128, 128])")
    w = _as_bytes(weight)
    N, K = w.shape
    nb, kb = -(-N // BLOCK), -(-K // BLOCK)
    if tuple(scale.shape) != (nb, kb):
        raise ValueError(f"{what}: scale grid {tuple(scale.shape)} does not match weight [{N}, {K}] (expected [{nb}, {kb}])")
    return Fp8Weight(w, _fp16_scale(scale, what), BLOCK, None if bias is None else bias.to(torch.float16), [N])


def channel_weight(weight: torch.Tensor, scale: torch.Tensor, bias: Optional[torch.Tensor] = None,
                   what: str = "linear") -> Fp8Weight:
    """Per-output-channel scales ``[N, 1]`` (or ``[N]``) become the ``block_h = 1`` grid ``[N, ceil(K/128)]``
    (compressed_tensors_v100.py:488-492)."""
    w = _as_bytes(weight)
    N, K = w.shape
    if scale.numel() != N:
        raise ValueError(f"{what}: {scale.numel()} channel scales for N={N}; refusing to dequantise unsafely")
    s = _fp16_scale(scale.reshape(N, 1), what).expand(N, -(-K // BLOCK)).contiguous()
    return Fp8Weight(w, s, 1, None if bias is None else bias.to(torch.float16), [N])


def tensor_weight(weight: torch.Tensor, scale: torch.Tensor, logical_widths: Optional[Sequence[int]] = None,
                  bias: Optional[torch.Tensor] = None, what: str = "linear") -> Fp8Weight:
    """Per-tensor scales: one per logical shard of a fused module, expanded to per-row scales over the shard's rows first
    (what ``convert_to_channelwise`` does, compressed_tensors_v100.py:247-256)."""
    w = _as_bytes(weight)
    N, K = w.shape
    widths = list(logical_widths) if logical_widths else [N]
    s = scale.reshape(-1)
    if s.numel() == 1 and len(widths) > 1:
        s = s.repeat(len(widths))
    if s.numel() != len(widths) or sum(widths) != N:
        raise ValueError(f"{what}: {s.numel()} tensor scales for logical widths {widths} (N={N})")
    per_row = torch.repeat_interleave(s, torch.tensor(widths))
    out = channel_weight(w, per_row, bias, what)
    out.logical_widths = widths
    return out


def load_linear(src: Source, prefix: str, fmt: str = "auto", block=(BLOCK, BLOCK)) -> Fp8Weight:
    """Read one linear.  ``fmt``: "native" (``weight_scale_inv``), "ct" (compressed-tensors ``weight_scale``; block,
    channel or tensor is told from its shape) or "auto" (whichever key exists)."""
    s = _src(src)
    w = _get(s, f"{prefix}.weight")
    bias = _get(s, f"{prefix}.bias") if f"{prefix}.bias" in s else None
    has_inv, has_ct = f"{prefix}.weight_scale_inv" in s, f"{prefix}.weight_scale" in s
    if fmt == "auto":
        if has_inv == has_ct:
            raise KeyError(f"{prefix}: need exactly one of weight_scale_inv (native fp8) / weight_scale (compressed-tensors)")
        fmt = "native" if has_inv else "ct"
    if fmt == "native":
        return block_weight(w, _get(s, f"{prefix}.weight_scale_inv"), bias, block, prefix)
    if fmt != "ct":
        raise ValueError(f"unknown checkpoint format {fmt!r}")
    sc = _get(s, f"{prefix}.weight_scale")
    N, K = w.shape
    if sc.dim() == 2 and tuple(sc.shape) == (-(-N // BLOCK), -(-K // BLOCK)) and sc.shape[1] > 1:
        return block_weight(w, sc, bias, block, prefix)
    if sc.numel() == N and N > 1:
        return channel_weight(w, sc, bias, prefix)
    if sc.numel() == 1:
        return tensor_weight(w, sc, [N], bias, prefix)
    raise ValueError(f"{prefix}: weight_scale of shape {tuple(sc.shape)} fits neither block, channel nor tensor layout of [{N}, {K}]")


# ------------------------------------------------------------------------------------------------
# fused modules
# ------------------------------------------------------------------------------------------------
def fuse_column(parts: Sequence[Fp8Weight], what: str = "fused") -> Fp8Weight:
    """Merged column-parallel module (QKV, gate_up): rows and scale rows concatenated in order
    (tests/test_attention_shapes.py:97-101).  Block-scaled parts must each be a multiple of 128 rows, or a scale row
    would straddle two of them."""
    if not parts:
        raise ValueError(f"{what}: nothing to fuse")
    bh, K = parts[0].block_h, parts[0].K
    for p in parts:
        if p.block_h != bh or p.K != K:
            raise ValueError(f"{what}: parts disagree on layout (block_h {p.block_h} vs {bh}, K {p.K} vs {K})")
    if bh == BLOCK:
        for p in parts[:-1]:
            if p.N % BLOCK:
                raise ValueError(f"{what}: a block-scaled part of {p.N} rows cannot be followed by another (not a multiple of 128)")
    bias = None
    if any(p.bias is not None for p in parts):
        bias = torch.cat([p.bias if p.bias is not None else torch.zeros(p.N, dtype=torch.float16) for p in parts])
    widths = [w for p in parts for w in (p.logical_widths or [p.N])]
    return Fp8Weight(torch.cat([p.weight for p in parts], 0).contiguous(), torch.cat([p.scale for p in parts], 0).contiguous(),
                     bh, bias, widths)


def load_fused(src: Source, prefixes: Sequence[str], fmt: str = "auto") -> Fp8Weight:
    s = _src(src)
    return fuse_column([load_linear(s, p, fmt) for p in prefixes], what="+".join(prefixes))


@dataclass
class Fp8Experts:
    """Routed experts as the MoE entry points take them: ``w13 [E, 2I, H]`` (gate rows, then up rows), ``w2 [E, H, I]``,
    FP16 scale grids per expert, ``block_h`` as in :class:`Fp8Weight`."""
    w13: torch.Tensor
    s13: torch.Tensor
    w2: torch.Tensor
    s2: torch.Tensor
    block_h: int

    def to(self, device) -> "Fp8Experts":
        return Fp8Experts(self.w13.to(device), self.s13.to(device), self.w2.to(device), self.s2.to(device), self.block_h)

    def local(self, ep_size: int, ep_rank: int) -> "Fp8Experts":
        """Contiguous expert partition of expert parallelism."""
        E = self.w13.shape[0]
        if E % ep_size:
            raise ValueError(f"{E} experts do not divide over {ep_size} ranks")
        lo, hi = ep_rank * (E // ep_size), (ep_rank + 1) * (E // ep_size)
        return Fp8Experts(self.w13[lo:hi].contiguous(), self.s13[lo:hi].contiguous(), self.w2[lo:hi].contiguous(),
                          self.s2[lo:hi].contiguous(), self.block_h)


def load_experts(src: Source, experts_prefix: str, num_experts: Optional[int] = None, fmt: str = "auto",
                 names: Tuple[str, str, str] = ("gate_proj", "up_proj", "down_proj")) -> Fp8Experts:
    """Stack ``<experts_prefix>.<e>.{gate,up,down}_proj`` into fused ``w13`` / ``w2``
    (tools/turbomind_ab/stage_d_full_moe.py:73-81)."""
    s = _src(src)
    if num_experts is None:
        ids = set()
        head = experts_prefix + "."
        for k in (s.keys() if isinstance(s, TensorSource) else s.keys()):
            if k.startswith(head) and k.endswith(f".{names[0]}.weight"):
                ids.add(int(k[len(head):].split(".")[0]))
        if not ids or ids != set(range(len(ids))):
            raise KeyError(f"{experts_prefix}: expert ids {sorted(ids)} are not 0..E-1")
        num_experts = len(ids)
    w13, s13, w2, s2, bh = [], [], [], [], None
    for e in range(num_experts):
        b = f"{experts_prefix}.{e}"
        gu = fuse_column([load_linear(s, f"{b}.{names[0]}", fmt), load_linear(s, f"{b}.{names[1]}", fmt)], what=f"{b}.gate_up")
        dn = load_linear(s, f"{b}.{names[2]}", fmt)
        if dn.block_h != gu.block_h or (bh is not None and gu.block_h != bh):
            raise ValueError(f"{b}: experts mix scale layouts")
        bh = gu.block_h
        w13.append(gu.weight)
        s13.append(gu.scale)
        w2.append(dn.weight)
        s2.append(dn.scale)
    return Fp8Experts(torch.stack(w13).contiguous(), torch.stack(s13).contiguous(), torch.stack(w2).contiguous(),
                      torch.stack(s2).contiguous(), int(bh))


# ------------------------------------------------------------------------------------------------
# tensor-parallel shards of a loaded weight
# ------------------------------------------------------------------------------------------------
def shard(w: Fp8Weight, mode: str, tp_size: int, tp_rank: int) -> Fp8Weight:
    """Column-parallel (output rows) or row-parallel (input columns) shard, scale grid cut along with it.  A fused
    column-parallel module is cut per logical part, as vLLM's merged loaders do, so every rank holds its slice of Q, of K
    and of V (not a slice of the concatenation)."""
    from . import parallel as par
    if mode == "row":
        if w.block_h == 1:
            # per-row scales do not depend on K: any ceil(K_shard / 128) columns of the grid will do, which is what lets
            # a shard like K = 176 (1408 / 8) through (compressed_tensors_v100.py:931-950 has to go to FP16 for it)
            if w.K % tp_size:
                raise ValueError(f"K={w.K} not divisible by tp_size={tp_size}")
            k_per = w.K // tp_size
            ws = w.weight[:, tp_rank * k_per:(tp_rank + 1) * k_per].contiguous()
            ss = w.scale[:, :-(-k_per // BLOCK)].contiguous()
        else:
            ws, ss = par.shard_row_parallel(w.weight, w.scale, tp_size, tp_rank, BLOCK)
        # the bias of a row-parallel layer is added on rank 0 only, before the reduce (vllm_serve.py:2937-2945)
        return Fp8Weight(ws, ss, w.block_h, w.bias if tp_rank == 0 else None, list(w.logical_widths))
    if mode != "column":
        raise ValueError(f"unknown shard mode {mode!r}")
    widths = w.logical_widths or [w.N]
    parts, row0 = [], 0
    for width in widths:
        sl = slice(row0, row0 + width)
        srows = slice(row0 // w.block_h, -(-(row0 + width) // w.block_h))
        if w.block_h == BLOCK and row0 % BLOCK:
            raise ValueError("block-scaled logical part does not start on a 128-row boundary")
        pw, ps = par.shard_column_parallel(w.weight[sl], w.scale[srows], tp_size, tp_rank, w.block_h)
        pb = None if w.bias is None else w.bias[sl][tp_rank * (width // tp_size):(tp_rank + 1) * (width // tp_size)]
        parts.append(Fp8Weight(pw, ps, w.block_h, pb, [width // tp_size]))
        row0 += width
    return fuse_column(parts, what="column shard") if len(parts) > 1 else parts[0]


def to_linear_module(w: Fp8Weight, device="cuda"):
    """A ready :class:`FP8W8A16Linear` on ``device``."""
    from .module import FP8W8A16Linear
    d = w.to(device)
    return FP8W8A16Linear(None, d.weight, d.scale, d.block_h, BLOCK, d.bias)
