"""torch-tensor front end of the C ABI: the op surface the reference exposes through pybind
(``src/fp8_w8a16_sm70/fp8_dequant.cu:3218-3298``), on one B200 engine.

PyTorch is plumbing here: tensors carry device memory, ``torch.cuda.current_stream`` names the
stream every kernel is launched on (the reference's stream rule, ``fp8_dequant.cu:29-36``).  All
compute happens in the CUDA library; a missing library or a CPU tensor raises.
"""

from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import _cabi
from ._cabi import ALGO_AUTO, ALGO_GEMV, ALGO_TC, SCALE_F16, SCALE_F32  # noqa: F401

_WORKSPACES: dict = {}      # (device index, raw stream) -> current buffer
_RETIRED: list = []         # outgrown buffers, kept alive for launches and graphs that still hold their address
_WS_FLOOR = None
_LINEAR_WS_BYTES: dict = {}
_TICKET_BYTES = 65536


def _stream(dev: torch.device) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


def _require_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = tensors[0].device
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("fp8_w8a16 ops run on CUDA tensors only (no CPU fallback)")
        if t.device != dev:
            raise RuntimeError("all tensors must be on the same device")
        if not t.is_contiguous():
            raise RuntimeError("tensors must be contiguous")
    return dev


def _as_u8(w: torch.Tensor) -> torch.Tensor:
    if w.dtype == torch.uint8:
        return w
    if w.dtype == torch.float8_e4m3fn:
        return w.view(torch.uint8)
    raise RuntimeError(f"weight must be uint8 or float8_e4m3fn (got {w.dtype})")


def _scale_dtype(s: torch.Tensor) -> int:
    if s.dtype == torch.float16:
        return SCALE_F16
    if s.dtype == torch.float32:
        return SCALE_F32
    raise RuntimeError(f"scales must be float16 or float32 (got {s.dtype}); cast bf16 scales at load")


def _floor_bytes() -> int:
    """Smallest workspace ever handed out: the largest need of any dense call (the 256-token tile's partial tiles,
    ~39 MB), so that dense layers never make a workspace grow, whatever order decode and prefill shapes arrive in."""
    global _WS_FLOOR
    if _WS_FLOOR is None:
        _WS_FLOOR = max(int(_cabi.load().fp8w8a16_linear_workspace_bytes(m, 128, 128)) for m in (1, 16, 32, 64, 128, 256))
    return _WS_FLOOR


def workspace(dev: torch.device, nbytes: int, stream: Optional[int] = None) -> torch.Tensor:
    """Per (device, stream) scratch buffer.  The first 64 KiB hold the kernels' hand-off counters: zero when
    allocated, left at zero by every kernel.

    A buffer that has been handed out is NEVER freed: launches already enqueued and CUDA graphs captured earlier
    keep its address (they write fp32 partial tiles and ticket counters there), so a buffer that is outgrown is
    retired to a keep-alive list and a larger zeroed one takes its place for new launches.  Creating or growing a
    workspace while the stream is being captured raises: the new buffer would belong to the graph's private pool.
    Run each shape once outside capture first (that is what a warm-up does)."""
    key = (dev.index if dev.index is not None else torch.cuda.current_device(), _stream(dev) if stream is None else stream)
    ws = _WORKSPACES.get(key)
    if ws is None or ws.numel() < nbytes:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError(f"fp8_w8a16: this call needs a {'larger ' if ws is not None else ''}workspace ({int(nbytes)} bytes) "
                               "on a stream that is being captured; run the same shape once outside the capture first")
        size = max(int(nbytes), _floor_bytes())
        if ws is not None:
            size = max(size, 2 * ws.numel())     # geometric growth: few retired buffers
            _RETIRED.append(ws)
        ws = torch.zeros(size, dtype=torch.uint8, device=dev)
        _WORKSPACES[key] = ws
    return ws


def reset_workspaces() -> None:
    """After a reported device-side timeout the hand-off counters may be dirty: clear the counter header of every
    workspace, current and retired, in place.  Nothing is freed (enqueued launches and captured graphs hold the
    addresses).  Synchronises the device first so that no kernel is using the counters."""
    if torch.cuda.is_available() and (_WORKSPACES or _RETIRED):
        torch.cuda.synchronize()
    for ws in list(_WORKSPACES.values()) + _RETIRED:
        ws[:_TICKET_BYTES].zero_()


class _dev_guard:
    def __init__(self, dev: torch.device):
        self.idx = dev.index if dev.index is not None else torch.cuda.current_device()
        self.prev = None

    def __enter__(self):
        cur = torch.cuda.current_device()
        if cur != self.idx:
            self.prev = cur
            torch.cuda.set_device(self.idx)

    def __exit__(self, *a):
        if self.prev is not None:
            torch.cuda.set_device(self.prev)


# ------------------------------------------------------------------------------------------------
# dequant family
# ------------------------------------------------------------------------------------------------
def fp8_e4m3_to_fp16(x: torch.Tensor) -> torch.Tensor:
    """uint8 E4M3 bytes -> flat float16 (reference op ``fp8_e4m3_to_fp16``, fp8_dequant.cu:129)."""
    x = _as_u8(x)
    dev = _require_cuda(x)
    out = torch.empty(x.numel(), dtype=torch.float16, device=dev)
    with _dev_guard(dev):
        _cabi.check(_cabi.load().fp8w8a16_e4m3_to_fp16(x.data_ptr(), out.data_ptr(), x.numel(), _stream(dev)),
                    "fp8w8a16_e4m3_to_fp16")
    return out


def fp8_e4m3_to_fp16_scaled(x: torch.Tensor, scales: torch.Tensor, group_size: int) -> torch.Tensor:
    """Per-group scaled dequant (reference op ``fp8_e4m3_to_fp16_scaled``, fp8_dequant.cu:150)."""
    x = _as_u8(x)
    dev = _require_cuda(x, scales)
    if scales.dtype != torch.float16:
        raise RuntimeError("scales must be float16")
    if scales.numel() * group_size < x.numel():
        raise RuntimeError("not enough scales for the given group size")
    out = torch.empty(x.numel(), dtype=torch.float16, device=dev)
    with _dev_guard(dev):
        _cabi.check(_cabi.load().fp8w8a16_e4m3_to_fp16_scaled(x.data_ptr(), scales.data_ptr(), out.data_ptr(), x.numel(),
                                                               int(group_size), _stream(dev)),
                    "fp8w8a16_e4m3_to_fp16_scaled")
    return out


def fp8_e4m3_to_fp16_block_scaled(w: torch.Tensor, scales: torch.Tensor, N: int, K: int, block_h: int = 128,
                                  block_w: int = 128) -> torch.Tensor:
    """Bit-exact dequantised weight, float16 [N, K] (reference op ``fp8_e4m3_to_fp16_block_scaled``,
    fp8_dequant.cu:3053)."""
    w = _as_u8(w)
    dev = _require_cuda(w, scales)
    if w.numel() != N * K:
        raise RuntimeError(f"weight has {w.numel()} elements, expected N*K={N * K}")
    nb, kb = -(-N // block_h), -(-K // block_w)
    if scales.numel() != nb * kb:
        raise RuntimeError(f"scales have {scales.numel()} elements, expected {nb}x{kb}")
    out = torch.empty((N, K), dtype=torch.float16, device=dev)
    with _dev_guard(dev):
        _cabi.check(_cabi.load().fp8w8a16_dequant_block_scaled(w.data_ptr(), scales.data_ptr(), _scale_dtype(scales),
                                                                out.data_ptr(), N, K, block_h, block_w, _stream(dev)),
                    "fp8w8a16_dequant_block_scaled")
    return out


# ------------------------------------------------------------------------------------------------
# dense W8A16 linear
# ------------------------------------------------------------------------------------------------
def _check_residual(residual: Optional[torch.Tensor], M: int, N: int, dev) -> None:
    if residual is None:
        return
    if residual.dtype != torch.float16 or tuple(residual.shape) != (M, N) or not residual.is_contiguous() or residual.device != dev:
        raise RuntimeError(f"residual must be a contiguous float16 [{M}, {N}] tensor on {dev}")


def w8a16_linear(x: torch.Tensor, w: torch.Tensor, scales: torch.Tensor, N: int, K: int, block_h: int = 128,
                 block_w: int = 128, algo: int = ALGO_AUTO, out: Optional[torch.Tensor] = None,
                 residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x float16 [M, K] @ dequant(w [N, K], scales)^T -> float16 [M, N].

    One op for the reference's dense family (gemv_coalesced, gemv_coalesced_m, gemm_a1/a2/a3,
    gemm_wmma_poc) and the dispatch among them (src/fp8_w8a16_sm70/vllm_serve.py:1032-1100).
    ``residual`` (float16 [M, N]): added to the fp32 result in the GEMM's epilogue before the one rounding
    (tensor-core path at every M); ``out`` may be the same tensor."""
    w = _as_u8(w)
    dev = _require_cuda(x, w, scales)
    if x.dtype != torch.float16:
        raise RuntimeError(f"x must be float16 (got {x.dtype})")
    if x.dim() != 2 or x.shape[1] != K:
        raise RuntimeError(f"x must be [M, {K}] (got {tuple(x.shape)})")
    if w.numel() != N * K:
        raise RuntimeError(f"weight has {w.numel()} elements, expected N*K={N * K}")
    nb, kb = -(-N // block_h), -(-K // block_w)
    if scales.numel() != nb * kb:
        raise RuntimeError(f"scales have {scales.numel()} elements, expected {nb}x{kb}")
    M = x.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=torch.float16, device=dev)
    lib = _cabi.load()
    with _dev_guard(dev):
        st = _stream(dev)
        need = _LINEAR_WS_BYTES.get((M, N, K))
        if need is None:
            need = _LINEAR_WS_BYTES[(M, N, K)] = lib.fp8w8a16_linear_workspace_bytes(M, N, K)
        ws = workspace(dev, need, st)
        if residual is not None:
            _check_residual(residual, M, N, dev)
            rc = lib.fp8w8a16_linear_residual(x.data_ptr(), w.data_ptr(), scales.data_ptr(), _scale_dtype(scales), residual.data_ptr(),
                                              out.data_ptr(), M, N, K, block_h, block_w, ws.data_ptr(), ws.numel(), st)
        else:
            rc = lib.fp8w8a16_linear(x.data_ptr(), w.data_ptr(), scales.data_ptr(), _scale_dtype(scales), out.data_ptr(),
                                     M, N, K, block_h, block_w, algo, ws.data_ptr(), ws.numel(), st)
        if rc:
            _cabi.check(rc, "fp8w8a16_linear")
    return out


def add_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, residual: Optional[torch.Tensor] = None,
                inplace_residual: bool = False) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """``z = x + residual`` (fp32 sum, one FP16 rounding; ``z = x`` without a residual), then
    ``FP16(z * rsqrt(mean(z^2) + eps)) * weight``: the step vLLM's ``fused_add_rms_norm`` performs after a row-parallel
    projection and its all-reduce.  Returns ``(normed, z)``; ``z`` is written into ``residual`` when ``inplace_residual``."""
    dev = _require_cuda(x, weight)
    if x.dtype != torch.float16 or x.dim() != 2 or weight.dtype != torch.float16 or weight.numel() != x.shape[1]:
        raise RuntimeError(f"x must be float16 [M, N] and weight float16 [N] (got {tuple(x.shape)} {x.dtype}, {tuple(weight.shape)} {weight.dtype})")
    M, N = x.shape
    _check_residual(residual, M, N, dev)
    out = torch.empty_like(x)
    z = None
    if residual is not None:
        z = residual if inplace_residual else torch.empty_like(x)
    with _dev_guard(dev):
        _cabi.check(_cabi.load().fp8w8a16_add_rmsnorm(x.data_ptr(), None if residual is None else residual.data_ptr(), weight.data_ptr(),
                                                       float(eps), out.data_ptr(), None if z is None else z.data_ptr(), M, N, _stream(dev)),
                    "fp8w8a16_add_rmsnorm")
    return out, (x if residual is None else z)


class LinearPlan:
    """Everything about one dense layer that does not change between calls, resolved once: the hook's per-call path
    (``run``) then costs one output allocation, one stream query, one dictionary look-up and the C call.  The decode
    sweep makes 28 such calls per step; at 10-50 us of GPU time each, per-call host work is what the end-to-end rate
    is made of.  ``run`` trusts its input (float16, contiguous, ``[M, K]``, on the plan's device): the hooks establish that."""

    __slots__ = ("w", "s", "w_ptr", "s_ptr", "scale_dtype", "N", "K", "block_h", "dev", "dev_index", "fn", "ws_need", "comm")

    def __init__(self, weight: torch.Tensor, scales: torch.Tensor, N: int, K: int, block_h: int, comm=None):
        w = _as_u8(weight)
        dev = _require_cuda(w, scales)
        if w.numel() != N * K:
            raise RuntimeError(f"weight has {w.numel()} elements, expected N*K={N * K}")
        if scales.numel() != (-(-N // block_h)) * (-(-K // 128)):
            raise RuntimeError(f"scales have {scales.numel()} elements, expected {-(-N // block_h)}x{-(-K // 128)}")
        self.w, self.s = w, scales                      # keep the tensors alive: only their addresses are used per call
        self.w_ptr, self.s_ptr, self.scale_dtype = w.data_ptr(), scales.data_ptr(), _scale_dtype(scales)
        self.N, self.K, self.block_h = int(N), int(K), int(block_h)
        self.dev = dev
        self.dev_index = dev.index if dev.index is not None else torch.cuda.current_device()
        self.fn = _cabi.load().fp8w8a16_linear
        self.ws_need = {}
        self.comm = comm

    def matches(self, weight: torch.Tensor, scales: torch.Tensor) -> bool:
        return weight.data_ptr() == self.w_ptr and scales.data_ptr() == self.s_ptr

    def run(self, x2d: torch.Tensor) -> torch.Tensor:
        M = x2d.shape[0]
        out = torch.empty((M, self.N), dtype=torch.float16, device=self.dev)
        if torch.cuda.current_device() != self.dev_index:
            with _dev_guard(self.dev):
                return self._call(x2d, out, M)
        return self._call(x2d, out, M)

    def _call(self, x2d, out, M):
        st = torch._C._cuda_getCurrentRawStream(self.dev_index)
        need = self.ws_need.get(M)
        if need is None:
            need = self.ws_need[M] = _cabi.load().fp8w8a16_linear_workspace_bytes(M, self.N, self.K)
        ws = _WORKSPACES.get((self.dev_index, st))
        if ws is None or ws.numel() < need:
            ws = workspace(self.dev, need, st)
        rc = self.fn(x2d.data_ptr(), self.w_ptr, self.s_ptr, self.scale_dtype, out.data_ptr(), M, self.N, self.K, self.block_h,
                     128, ALGO_AUTO, ws.data_ptr(), ws.numel(), st)
        if rc:
            _cabi.check(rc, "fp8w8a16_linear")
        return out


NOALLOC_SCRATCH_BYTES = 768 << 10


def w8a16_linear_noalloc(x: torch.Tensor, w: torch.Tensor, scales: torch.Tensor, out: torch.Tensor, N: int, K: int,
                         block_h: int = 128, block_w: int = 128) -> torch.Tensor:
    """Decode GEMV into a caller-provided ``out`` without allocating anything, for callers that may not
    touch the allocator (fixed memory pools, no-allocation policies).  Scratch is a 768 KiB array inside the library;
    larger shapes raise.  Calls that overlap on the GPU share that array and race; order them."""
    w = _as_u8(w)
    dev = _require_cuda(x, w, scales, out)
    if x.dtype != torch.float16 or out.dtype != torch.float16:
        raise RuntimeError("x and out must be float16")
    if x.dim() != 2 or x.shape[1] != K:
        raise RuntimeError(f"x must be [M, {K}] (got {tuple(x.shape)})")
    M = x.shape[0]
    if tuple(out.shape) != (M, N) or w.numel() != N * K:
        raise RuntimeError(f"shape mismatch: out {tuple(out.shape)}, weight {w.numel()} elements, expected [{M}, {N}] and N*K={N * K}")
    nb, kb = -(-N // block_h), -(-K // block_w)
    if scales.numel() != nb * kb:       # the C ABI sees only a pointer: a short grid would be read out of bounds on the device
        raise RuntimeError(f"scales have {scales.numel()} elements, expected {nb}x{kb}")
    with _dev_guard(dev):
        _cabi.check(_cabi.load().fp8w8a16_linear_noalloc(x.data_ptr(), w.data_ptr(), scales.data_ptr(), _scale_dtype(scales),
                                                          out.data_ptr(), M, N, K, block_h, block_w, _stream(dev)),
                    "fp8w8a16_linear_noalloc")
    return out


# ------------------------------------------------------------------------------------------------
# row-parallel linear with the all-reduce fused into the GEMM kernel (peer memory over NVLink)
# ------------------------------------------------------------------------------------------------
class PeerComm:
    """One rank's end of the peer-memory communicator (``fp8w8a16_comm_*``): a device buffer (FP16 staging +
    a double-buffered inbox of tagged packets) that the other ranks' GPUs map through CUDA IPC.  ``handle()`` is the 64-byte IPC handle to send
    to the peers by any host channel; ``attach(peer, handle)`` maps a peer's buffer.  All ranks must then make the
    same sequence of ``w8a16_linear_allreduce`` calls."""

    def __init__(self, rank: int, world: int, max_out_elems: int, timeout_ms: int = 2000,
                 device: Optional[torch.device] = None):
        import ctypes
        self.rank, self.world, self.max_out_elems = rank, world, max_out_elems
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        if self.device.type != "cuda":
            raise RuntimeError("PeerComm needs a CUDA device (there is no CPU path)")
        self._h = ctypes.c_void_p()
        with _dev_guard(self.device):
            _cabi.check(_cabi.load().fp8w8a16_comm_create(rank, world, max_out_elems, timeout_ms,
                                                         ctypes.byref(self._h)), "fp8w8a16_comm_create")

    def handle(self) -> bytes:
        import ctypes
        buf = ctypes.create_string_buffer(_cabi.COMM_HANDLE_BYTES)
        with _dev_guard(self.device):
            _cabi.check(_cabi.load().fp8w8a16_comm_export(self._h, buf), "fp8w8a16_comm_export")
        return buf.raw

    def attach(self, peer: int, handle: bytes) -> None:
        import ctypes
        buf = ctypes.create_string_buffer(handle, _cabi.COMM_HANDLE_BYTES)
        with _dev_guard(self.device):
            _cabi.check(_cabi.load().fp8w8a16_comm_attach(self._h, peer, buf), "fp8w8a16_comm_attach")

    def attach_ptr(self, peer: int, base: int) -> None:
        _cabi.check(_cabi.load().fp8w8a16_comm_attach_ptr(self._h, peer, base), "fp8w8a16_comm_attach_ptr")

    @property
    def base(self) -> int:
        return int(_cabi.load().fp8w8a16_comm_base(self._h) or 0)

    @property
    def nbytes(self) -> int:
        return int(_cabi.load().fp8w8a16_comm_bytes(self._h))

    def reset(self) -> None:
        """This rank's part of the collective reset (``fp8w8a16_comm_reset``): launch number back to zero, inbox
        emptied, on the current stream.  ``parallel.reset_peer_comm`` wraps it in the barriers it needs."""
        with _dev_guard(self.device):
            _cabi.check(_cabi.load().fp8w8a16_comm_reset(self._h, _stream(self.device)), "fp8w8a16_comm_reset")

    def close(self) -> None:
        if self._h is not None and self._h.value:
            with _dev_guard(self.device):
                _cabi.load().fp8w8a16_comm_destroy(self._h)
            self._h = None


def w8a16_linear_allreduce(comm: PeerComm, x: torch.Tensor, w: torch.Tensor, scales: torch.Tensor, N: int, K: int,
                           block_h: int = 128, block_w: int = 128, out: Optional[torch.Tensor] = None,
                           residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """This rank's K shard of a row-parallel linear, x [M, K_shard] @ dequant(w [N, K_shard])^T, summed over the ranks
    of ``comm`` inside the GEMM kernel: one launch replaces apply + all-reduce
    (src/fp8_w8a16_sm70/vllm_serve.py:2922-2959).  The result is bit-identical on every rank.  ``residual`` (float16
    [M, N], the same values on every rank) joins the cross-rank sum before the one rounding."""
    w = _as_u8(w)
    dev = _require_cuda(x, w, scales)
    if x.dtype != torch.float16:
        raise RuntimeError(f"x must be float16 (got {x.dtype})")
    if x.dim() != 2 or x.shape[1] != K or w.numel() != N * K:
        raise RuntimeError(f"shape mismatch: x {tuple(x.shape)}, w {w.numel()} elements, N={N} K={K}")
    M = x.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=torch.float16, device=dev)
    lib = _cabi.load()
    with _dev_guard(dev):
        st = _stream(dev)
        need = _LINEAR_WS_BYTES.get((M, N, K))
        if need is None:
            need = _LINEAR_WS_BYTES[(M, N, K)] = lib.fp8w8a16_linear_workspace_bytes(M, N, K)
        ws = workspace(dev, need, st)
        _check_residual(residual, M, N, dev)
        rc = lib.fp8w8a16_linear_allreduce_residual(comm._h, x.data_ptr(), w.data_ptr(), scales.data_ptr(), _scale_dtype(scales),
                                                    None if residual is None else residual.data_ptr(), out.data_ptr(), M, N, K, block_h,
                                                    block_w, ws.data_ptr(), ws.numel(), st)
        if rc:
            _cabi.check(rc, "fp8w8a16_linear_allreduce")
    return out


# ------------------------------------------------------------------------------------------------
# MoE
# ------------------------------------------------------------------------------------------------
_LOGIT_DTYPES = {torch.float32: _cabi.DTYPE_F32, torch.float16: _cabi.DTYPE_F16, torch.bfloat16: _cabi.DTYPE_BF16}


def moe_topk_softmax(logits: torch.Tensor, topk: int, renormalize: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """Router logits [M, E] -> (topk_weights fp32 [M, topk], topk_ids int32 [M, topk])."""
    dev = _require_cuda(logits)
    if logits.dtype not in _LOGIT_DTYPES:
        raise RuntimeError(f"unsupported logits dtype {logits.dtype}")
    M, E = logits.shape
    ids = torch.empty((M, topk), dtype=torch.int32, device=dev)
    wts = torch.empty((M, topk), dtype=torch.float32, device=dev)
    with _dev_guard(dev):
        _cabi.check(_cabi.load().fp8w8a16_moe_topk_softmax(logits.data_ptr(), _LOGIT_DTYPES[logits.dtype], M, E, topk,
                                                            1 if renormalize else 0, ids.data_ptr(), wts.data_ptr(),
                                                            _stream(dev)),
                    "fp8w8a16_moe_topk_softmax")
    return wts, ids


def moe_router_topk(x: torch.Tensor, gate_weight: torch.Tensor, topk: int, renormalize: bool = True,
                    return_logits: bool = False, shared_expert_id: int = -1, routed_scale: float = 1.0):
    """Router gate GEMV + top-k softmax in one kernel: x float16 [M, H], gate_weight [E, H] (fp16 / bf16 / fp32) ->
    (weights fp32 [M, topk], ids int32 [M, topk]) and, on request, the fp32 logits [M, E].  Stands in for the gate Linear
    and ``fused_topk`` that run before the reference's MoE hook (src/fp8_w8a16_sm70/vllm_serve.py:2799-2812).
    ``shared_expert_id >= 0`` appends the fixed route (that id, weight 1) to every token (outputs are [M, topk + 1]);
    ``routed_scale`` multiplies the routed weights."""
    dev = _require_cuda(x, gate_weight)
    if x.dtype != torch.float16 or x.dim() != 2:
        raise RuntimeError("x must be float16 [M, H]")
    if gate_weight.dtype not in _LOGIT_DTYPES or gate_weight.dim() != 2 or gate_weight.shape[1] != x.shape[1]:
        raise RuntimeError(f"gate_weight must be [E, {x.shape[1]}] in fp32 / fp16 / bf16 (got {tuple(gate_weight.shape)} {gate_weight.dtype})")
    M, H = x.shape
    E = gate_weight.shape[0]
    cols = topk + (1 if shared_expert_id >= 0 else 0)
    ids = torch.empty((M, cols), dtype=torch.int32, device=dev)
    w = torch.empty((M, cols), dtype=torch.float32, device=dev)
    logits = torch.empty((M, E), dtype=torch.float32, device=dev) if return_logits else None
    with _dev_guard(dev):
        _cabi.check(_cabi.load().fp8w8a16_moe_router_topk(x.contiguous().data_ptr(), gate_weight.contiguous().data_ptr(),
                                                           _LOGIT_DTYPES[gate_weight.dtype], M, E, H, topk, 1 if renormalize else 0,
                                                           int(shared_expert_id), float(routed_scale), ids.data_ptr(), w.data_ptr(), logits.data_ptr() if return_logits else None,
                                                           _stream(dev)), "fp8w8a16_moe_router_topk")
    return (w, ids, logits) if return_logits else (w, ids)


def moe_token_tile(R: int, num_local_experts: int) -> int:
    return int(_cabi.load().fp8w8a16_moe_token_tile(R, num_local_experts))


def moe_align(topk_ids: torch.Tensor, num_local_experts: int, token_tile: int, expert_map: Optional[torch.Tensor] = None):
    """Route table: (counts [E], offsets [E+1], tile_offsets [E+1], sorted_route [R], inv_pos [R]), all int32."""
    dev = _require_cuda(topk_ids)
    if topk_ids.dtype not in (torch.int32, torch.int64):
        raise RuntimeError("topk_ids must be int32 or int64")
    R, E = topk_ids.numel(), num_local_experts
    counts = torch.empty(E, dtype=torch.int32, device=dev)
    offsets = torch.empty(E + 1, dtype=torch.int32, device=dev)
    tile_offsets = torch.empty(E + 1, dtype=torch.int32, device=dev)
    sorted_route = torch.empty(R, dtype=torch.int32, device=dev)
    inv_pos = torch.empty(R, dtype=torch.int32, device=dev)
    emap_ptr, n_global = None, E
    if expert_map is not None:
        _require_cuda(topk_ids, expert_map)
        if expert_map.dtype != torch.int32:
            raise RuntimeError("expert_map must be int32")
        emap_ptr, n_global = expert_map.data_ptr(), expert_map.numel()
    with _dev_guard(dev):
        _cabi.check(_cabi.load().fp8w8a16_moe_align(topk_ids.data_ptr(), 1 if topk_ids.dtype == torch.int64 else 0, R,
                                                     emap_ptr, n_global, E, token_tile, counts.data_ptr(),
                                                     offsets.data_ptr(), tile_offsets.data_ptr(), sorted_route.data_ptr(),
                                                     inv_pos.data_ptr(), _stream(dev)),
                    "fp8w8a16_moe_align")
    return counts, offsets, tile_offsets, sorted_route, inv_pos


def moe_gather(x: torch.Tensor, sorted_route: torch.Tensor, topk_weights: torch.Tensor, topk: int,
               weight_on_input: bool = False):
    dev = _require_cuda(x, sorted_route, topk_weights)
    R, H = sorted_route.numel(), x.shape[1]
    xs = torch.empty((R, H), dtype=torch.float16, device=dev)
    wsorted = torch.empty(R, dtype=torch.float32, device=dev)
    with _dev_guard(dev):
        _cabi.check(_cabi.load().fp8w8a16_moe_gather(x.data_ptr(), sorted_route.data_ptr(), topk_weights.data_ptr(), R, topk, H,
                                                      1 if weight_on_input else 0, xs.data_ptr(), wsorted.data_ptr(),
                                                      _stream(dev)),
                    "fp8w8a16_moe_gather")
    return xs, wsorted


def moe_combine(y_sorted: torch.Tensor, inv_pos: torch.Tensor, M: int, topk: int) -> torch.Tensor:
    dev = _require_cuda(y_sorted, inv_pos)
    H = y_sorted.shape[1]
    out = torch.empty((M, H), dtype=torch.float16, device=dev)
    with _dev_guard(dev):
        _cabi.check(_cabi.load().fp8w8a16_moe_combine(y_sorted.data_ptr(), inv_pos.data_ptr(), M, topk, H, out.data_ptr(),
                                                       _stream(dev)),
                    "fp8w8a16_moe_combine")
    return out


def moe_grouped_gemm(x_sorted: torch.Tensor, w: torch.Tensor, scales: torch.Tensor, offsets: torch.Tensor,
                     tile_offsets: torch.Tensor, N: int, K: int, block_h: int, token_tile: int, paired: bool = False,
                     row_weight: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Grouped expert GEMM over expert-sorted rows; ``paired`` fuses SiLU(gate) * up of a [E, 2N, K] weight."""
    w = _as_u8(w)
    dev = _require_cuda(x_sorted, w, scales, offsets, tile_offsets)
    if x_sorted.dtype != torch.float16 or x_sorted.shape[1] != K:
        raise RuntimeError(f"x_sorted must be float16 [R, {K}]")
    E = w.shape[0]
    rows_w = 2 * N if paired else N
    if tuple(w.shape) != (E, rows_w, K):
        raise RuntimeError(f"weight must be [{E}, {rows_w}, {K}] (got {tuple(w.shape)})")
    R = x_sorted.shape[0]
    out = torch.empty((R, N), dtype=torch.float16, device=dev)
    lib = _cabi.load()
    with _dev_guard(dev):
        ws = workspace(dev, lib.fp8w8a16_moe_grouped_gemm_workspace_bytes(R, E, N, K, 1 if paired else 0, token_tile))
        _cabi.check(lib.fp8w8a16_moe_grouped_gemm(x_sorted.data_ptr(), w.data_ptr(), scales.data_ptr(), _scale_dtype(scales),
                                                  out.data_ptr(), None if row_weight is None else row_weight.data_ptr(),
                                                  offsets.data_ptr(), tile_offsets.data_ptr(), R, E, N, K, block_h,
                                                  1 if paired else 0, token_tile, ws.data_ptr(), ws.numel(), _stream(dev)),
                    "fp8w8a16_moe_grouped_gemm")
    return out


_ACTIVATIONS = {"silu": _cabi.ACT_SILU, "gelu": _cabi.ACT_GELU}


def moe_forward(x: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor, w13: torch.Tensor, s13: torch.Tensor,
                w2: torch.Tensor, s2: torch.Tensor, block_h: int = 128, expert_map: Optional[torch.Tensor] = None,
                weight_on_input: bool = False, out: Optional[torch.Tensor] = None, activation: str = "silu") -> torch.Tensor:
    """Routed-only MoE layer output float16 [M, H] (reference: ``_our_moe_apply``,
    src/fp8_w8a16_sm70/vllm_serve.py:2175-2411)."""
    w13, w2 = _as_u8(w13), _as_u8(w2)
    dev = _require_cuda(x, topk_weights, topk_ids, w13, s13, w2, s2)
    if x.dtype != torch.float16:
        raise RuntimeError("x must be float16")
    if activation not in _ACTIVATIONS:
        raise NotImplementedError(f"unsupported MoE activation {activation!r} (silu or gelu)")
    if topk_weights.dtype != torch.float32:
        raise RuntimeError("topk_weights must be float32")
    if topk_ids.dtype not in (torch.int32, torch.int64):
        raise RuntimeError("topk_ids must be int32 or int64")
    if s13.dtype != s2.dtype:
        raise RuntimeError("w13 and w2 scales must share a dtype")
    M, H = x.shape
    E, two_i, h2 = w13.shape
    I = two_i // 2
    if h2 != H or tuple(w2.shape) != (E, H, I):
        raise RuntimeError(f"shape mismatch: x {tuple(x.shape)}, w13 {tuple(w13.shape)}, w2 {tuple(w2.shape)}")
    topk = topk_ids.shape[-1]
    if topk_ids.numel() != M * topk or topk_weights.numel() != M * topk:
        raise RuntimeError("topk_ids / topk_weights must be [M, topk]")
    kb13, kb2 = -(-H // 128), -(-I // 128)
    if s13.numel() != E * (-(-two_i // block_h)) * kb13 or s2.numel() != E * (-(-H // block_h)) * kb2:
        raise RuntimeError("scale grid size does not match the weights and block_h")
    emap_ptr, n_global = None, E
    if expert_map is not None:
        _require_cuda(x, expert_map)
        if expert_map.dtype != torch.int32:
            raise RuntimeError("expert_map must be int32")
        emap_ptr, n_global = expert_map.data_ptr(), expert_map.numel()
    if out is None:
        out = torch.empty((M, H), dtype=torch.float16, device=dev)
    lib = _cabi.load()
    with _dev_guard(dev):
        ws = workspace(dev, lib.fp8w8a16_moe_workspace_bytes(M, topk, E, H, I))
        _cabi.check(lib.fp8w8a16_moe_forward(x.data_ptr(), topk_ids.data_ptr(), 1 if topk_ids.dtype == torch.int64 else 0,
                                             topk_weights.data_ptr(), emap_ptr, n_global, w13.data_ptr(), s13.data_ptr(),
                                             w2.data_ptr(), s2.data_ptr(), _scale_dtype(s13), out.data_ptr(), M, topk, E, H, I,
                                             block_h, 1 if weight_on_input else 0, _ACTIVATIONS[activation], ws.data_ptr(), ws.numel(),
                                             _stream(dev)),
                    "fp8w8a16_moe_forward")
    return out


class EpComm:
    """One rank's end of the expert-parallel exchange buffer (``fp8w8a16_ep_*``): an inbox for routed rows, a return
    buffer for finished rows and their headers / flags, mapped into the peers through CUDA IPC like a ``PeerComm``."""

    def __init__(self, rank: int, world: int, max_tokens: int, topk: int, hidden: int, num_experts: int, timeout_ms: int = 2000,
                 device: Optional[torch.device] = None):
        self.rank, self.world, self.max_tokens, self.topk, self.hidden, self.num_experts = rank, world, max_tokens, topk, hidden, num_experts
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        if self.device.type != "cuda":
            raise RuntimeError("EpComm needs a CUDA device (there is no CPU path)")
        self._h = ctypes.c_void_p()
        with _dev_guard(self.device):
            _cabi.check(_cabi.load().fp8w8a16_ep_create(rank, world, max_tokens, topk, hidden, num_experts, timeout_ms,
                                                       ctypes.byref(self._h)), "fp8w8a16_ep_create")

    def handle(self) -> bytes:
        buf = ctypes.create_string_buffer(_cabi.COMM_HANDLE_BYTES)
        with _dev_guard(self.device):
            _cabi.check(_cabi.load().fp8w8a16_ep_export(self._h, buf), "fp8w8a16_ep_export")
        return buf.raw

    def attach(self, peer: int, handle: bytes) -> None:
        buf = ctypes.create_string_buffer(handle, _cabi.COMM_HANDLE_BYTES)
        with _dev_guard(self.device):
            _cabi.check(_cabi.load().fp8w8a16_ep_attach(self._h, peer, buf), "fp8w8a16_ep_attach")

    def attach_ptr(self, peer: int, base: int) -> None:
        _cabi.check(_cabi.load().fp8w8a16_ep_attach_ptr(self._h, peer, base), "fp8w8a16_ep_attach_ptr")

    @property
    def base(self) -> int:
        return int(_cabi.load().fp8w8a16_ep_base(self._h) or 0)

    @property
    def nbytes(self) -> int:
        return int(_cabi.load().fp8w8a16_ep_bytes(self._h))

    def reset(self) -> None:
        with _dev_guard(self.device):
            _cabi.check(_cabi.load().fp8w8a16_ep_reset(self._h, _stream(self.device)), "fp8w8a16_ep_reset")

    def close(self) -> None:
        if self._h is not None and self._h.value:
            with _dev_guard(self.device):
                _cabi.load().fp8w8a16_ep_destroy(self._h)
            self._h = None


def _ep_args(ep: EpComm, w13: torch.Tensor, w2: torch.Tensor, s13: torch.Tensor, s2: torch.Tensor, block_h: int):
    E, two_i, H = w13.shape
    I = two_i // 2
    if H != ep.hidden or tuple(w2.shape) != (E, H, I) or E * ep.world != ep.num_experts:
        raise RuntimeError(f"expert shapes {tuple(w13.shape)} / {tuple(w2.shape)} do not match the exchange buffer "
                           f"(hidden {ep.hidden}, {ep.num_experts} experts over {ep.world} ranks)")
    if s13.dtype != s2.dtype:
        raise RuntimeError("w13 and w2 scales must share a dtype")
    if s13.numel() != E * (-(-two_i // block_h)) * (-(-H // 128)) or s2.numel() != E * (-(-H // block_h)) * (-(-I // 128)):
        raise RuntimeError("scale grid size does not match the weights and block_h")
    return E, I


def ep_moe_forward(ep: EpComm, x: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor, w13: torch.Tensor, s13: torch.Tensor,
                   w2: torch.Tensor, s2: torch.Tensor, block_h: int = 128, activation: str = "silu", m_max: Optional[int] = None,
                   out: Optional[torch.Tensor] = None, phase: str = "all") -> Optional[torch.Tensor]:
    """Expert-parallel routed MoE layer over peer memory: this rank's tokens ``x [M, H]`` with GLOBAL expert ids, this
    rank's expert slice ``w13 [E/P, 2I, H]`` / ``w2 [E/P, H, I]``.  ``m_max`` is the largest token count any rank brings
    to this call and must be the same on every rank (default: this rank's M, i.e. equal batches).  ``phase`` runs one
    step only ("dispatch", "experts", "combine") - used to drive several ranks from one process in tests."""
    w13, w2 = _as_u8(w13), _as_u8(w2)
    dev = _require_cuda(x, topk_weights, topk_ids, w13, s13, w2, s2)
    if x.dtype != torch.float16 or x.dim() != 2 or x.shape[1] != ep.hidden:
        raise RuntimeError(f"x must be float16 [M, {ep.hidden}]")
    if activation not in _ACTIVATIONS:
        raise NotImplementedError(f"unsupported MoE activation {activation!r} (silu or gelu)")
    if topk_weights.dtype != torch.float32 or topk_ids.dtype not in (torch.int32, torch.int64):
        raise RuntimeError("topk_weights must be float32 and topk_ids int32 or int64")
    M = x.shape[0]
    if topk_ids.numel() != M * ep.topk or topk_weights.numel() != M * ep.topk:
        raise RuntimeError(f"topk_ids / topk_weights must be [M, {ep.topk}]")
    E, I = _ep_args(ep, w13, w2, s13, s2, block_h)
    m_max = M if m_max is None else int(m_max)
    if not (1 <= m_max <= ep.max_tokens and M <= m_max):
        raise RuntimeError(f"m_max={m_max} must cover M={M} and fit the buffer's {ep.max_tokens} tokens per rank")
    lib = _cabi.load()
    i64 = 1 if topk_ids.dtype == torch.int64 else 0
    if out is None and phase in ("all", "combine"):
        out = torch.empty((M, ep.hidden), dtype=torch.float16, device=dev)
    with _dev_guard(dev):
        st = _stream(dev)
        ws = workspace(dev, lib.fp8w8a16_ep_workspace_bytes(ep._h, M, m_max, E, I), st)
        if phase in ("all", "dispatch"):
            _cabi.check(lib.fp8w8a16_ep_dispatch(ep._h, x.data_ptr(), topk_ids.data_ptr(), i64, topk_weights.data_ptr(), M, m_max, E, I,
                                                 ws.data_ptr(), ws.numel(), st), "fp8w8a16_ep_dispatch")
        if phase in ("all", "experts"):
            _cabi.check(lib.fp8w8a16_ep_experts(ep._h, w13.data_ptr(), s13.data_ptr(), w2.data_ptr(), s2.data_ptr(), _scale_dtype(s13), M, m_max,
                                                E, I, block_h, _ACTIVATIONS[activation], ws.data_ptr(), ws.numel(), st), "fp8w8a16_ep_experts")
        if phase in ("all", "combine"):
            _cabi.check(lib.fp8w8a16_ep_combine(ep._h, topk_ids.data_ptr(), i64, out.data_ptr(), M, st), "fp8w8a16_ep_combine")
    return out


def device_status(reset: bool = True) -> int:
    """Sticky device status word (0 = healthy).  Synchronises the device."""
    return _cabi.device_status(reset)
