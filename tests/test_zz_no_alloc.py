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
    # Large shapes at 4 tokens: how K is split is the library's choice, so each call may be served or refused - but the
    # largest one needs far more than the array whatever the split (5 splits x 4 tokens x 16384 outputs x 4 B = 1280 KiB),
    # and a refusal must name the scratch.  The buffers are real and large enough for every shape tried, so a call that is
    # accepted only touches memory that belongs to this test.
    refused = 0
    for N, K, M in ((16384, 25600, 4), (10240, 25600, 4), (28384, 8192, 4)):
        w = torch.zeros(N, K, dtype=torch.uint8, device="cuda")
        s = torch.ones(-(-N // 128), K // 128, dtype=torch.float16, device="cuda")
        x = torch.zeros(M, K, dtype=torch.float16, device="cuda")
        out = torch.zeros(M, N, dtype=torch.float16, device="cuda")
        rc = _call_noalloc(lib, x, w, s, out, M, N, K, 128)
        torch.cuda.synchronize()
        assert rc in (0, _cabi.ERR_WORKSPACE), (rc, _cabi.last_error())
        if rc == _cabi.ERR_WORKSPACE:
            assert "scratch" in _cabi.last_error()
            refused += 1
        del w, s, x, out
    assert refused >= 1, "no shape was refused: the fixed scratch array cannot hold 1280 KiB of partial sums"
    # refused by the argument checks, before anything is launched
    x = torch.zeros(16, dtype=torch.float16, device="cuda")
    p = x.data_ptr()
    assert lib.fp8w8a16_linear_noalloc(p, p, p, 0, p, 1, 128, 100, 128, 128, None) == _cabi.ERR_UNSUPPORTED
    assert lib.fp8w8a16_linear_noalloc(None, None, None, 0, None, 0, 128, 128, 128, 128, None) == 0
