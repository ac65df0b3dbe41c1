"""The allocation-free entry point (fp8w8a16_linear_noalloc), called through the C ABI.

It serves callers that cannot allocate device memory at call time — a worker whose pool was handed out at
start-up, code under a no-allocation policy, a plugin that only receives input and output buffers — by keeping the
split-K scratch in a fixed 768 KiB array inside the library.  Checked here: its output equals the workspace-taking
entry point's (same kernel, same split order, so bit for bit) on two calls in a row that reuse the array with
different shapes, and a shape whose scratch need exceeds the array is refused with a clear error.
Collected last on purpose: a run that stops at the first failure has then already run every other test."""
import ctypes

import pytest
import torch

from tests.helpers import make_dense

pytestmark = pytest.mark.gpu


def _call_noalloc(lib, x, w, s, out, M, N, K, bh):
    stream = torch.cuda.current_stream().cuda_stream
    return lib.fp8w8a16_linear_noalloc(x.data_ptr(), w.data_ptr(), s.data_ptr(), 1 if s.dtype == torch.float32 else 0,
                                       out.data_ptr(), M, N, K, bh, 128, stream)


def test_noalloc_matches_workspace_entry_point_twice_in_a_row(lib):
    from vllm_fp8_w8a16_sm70_b200 import _cabi, ops
    from oracle import linear as olin
    # two different shapes back to back: the second call finds the first one's leftovers in the array
    # (6 tokens: two launches that share the array inside one call; K = 256: too short to split, so no scratch is used at all)
    cases = [(3, 640, 4096, "block"), (1, 352, 2048, "channel"), (6, 640, 4096, "block"), (2, 384, 256, "block"), (3, 640, 4096, "block")]
    for M, N, K, scheme in cases:
        x, w, s, bh = make_dense(M, N, K, seed=M + N, scheme=scheme)
        xd, wd, sd = x.cuda(), w.cuda(), s.cuda()
        want = ops.w8a16_linear(xd, wd, sd, N, K, bh, 128, algo=ops.ALGO_GEMV)
        out = torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda")
        before = torch.cuda.memory_allocated()
        rc = _call_noalloc(lib, xd, wd, sd, out, M, N, K, bh)
        assert rc == 0, _cabi.last_error()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert torch.equal(out.view(torch.int16), want.view(torch.int16))
        olin.check_linear(out.cpu(), x, olin.oracle_linear_fp32(x, w, s, bh), K)
    out2 = torch.empty((3, 640), dtype=torch.float16, device="cuda")
    assert torch.equal(ops.w8a16_linear_noalloc(xd, wd, sd, out2, 640, 4096).view(torch.int16), want.view(torch.int16))
    with pytest.raises(RuntimeError, match="scales have"):        # a short scale grid would be read out of bounds on the device
        ops.w8a16_linear_noalloc(xd, wd, sd[:-1].contiguous(), out2, 640, 4096)
    with pytest.raises(RuntimeError, match="x must be"):
        ops.w8a16_linear_noalloc(xd.reshape(-1), wd, sd, out2, 640, 4096)


def test_noalloc_rejects_shapes_beyond_its_scratch(lib):
    from vllm_fp8_w8a16_sm70_b200 import _cabi
    # 4 tokens x 28384 outputs split 3 ways over K needs 64 KiB of counters + 1330 KiB of fp32 partial sums
    N, K, M = 28384, 8192, 4
    buf = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")   # never dereferenced: the call is refused first
    p = buf.data_ptr()
    rc = lib.fp8w8a16_linear_noalloc(p, p, p, 0, p, M, N, K, 128, 128, None)
    assert rc == _cabi.ERR_WORKSPACE and "scratch" in _cabi.last_error(), (rc, _cabi.last_error())
    assert lib.fp8w8a16_linear_noalloc(p, p, p, 0, p, 1, 128, 100, 128, 128, None) == _cabi.ERR_UNSUPPORTED
    assert lib.fp8w8a16_linear_noalloc(None, None, None, 0, None, 0, 128, 128, 128, 128, None) == 0
