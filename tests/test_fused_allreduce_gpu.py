"""Single-GPU checks of the fused GEMM + all-reduce entry points: argument validation, and the bounded wait for a
peer that never shows up (the kernel must give up, report through the device status word and leave the context usable).
The numerical test of the fused path needs two GPUs and lives in test_parallel_gpu.py."""
import pytest
import torch

from tests.helpers import make_dense

pytestmark = pytest.mark.gpu


def test_wait_for_absent_peer_times_out_and_context_survives(lib):
    from oracle import linear as olin
    from vllm_fp8_w8a16_sm70_b200 import ops
    ops.device_status()  # clear
    M, N, K = 4, 512, 512
    x, w, s, bh = make_dense(M, N, K, seed=5)
    a = ops.PeerComm(0, 2, max_out_elems=M * N, timeout_ms=50)
    b = ops.PeerComm(1, 2, max_out_elems=M * N, timeout_ms=50)   # stands in for a peer; never launches
    try:
        assert a.nbytes == b.nbytes and a.base and b.base
        a.attach_ptr(1, b.base)
        out = torch.full((M, N), 7.0, dtype=torch.float16, device="cuda")
        ops.w8a16_linear_allreduce(a, x.cuda(), w.cuda(), s.cuda(), N, K, bh, 128, out=out)
        torch.cuda.synchronize()
        assert ops.device_status() & 128, "the wait for the absent peer should have run out"
        assert torch.all(out == 7.0), "tiles whose peers never arrived must not be written"
        # the context is healthy: an ordinary linear still runs and is right
        y = ops.w8a16_linear(x.cuda(), w.cuda(), s.cuda(), N, K, bh, 128)
        st = olin.error_stats(y.cpu(), olin.oracle_linear_fp32(x, w, s, bh))
        assert st["rel_rms"] < 1e-2 and ops.device_status() == 0
    finally:
        a.close()
        b.close()


def test_fused_allreduce_argument_checks(lib):
    from vllm_fp8_w8a16_sm70_b200 import ops
    with pytest.raises(RuntimeError):
        ops.PeerComm(0, 1, max_out_elems=16)            # a world of one has nothing to reduce
    with pytest.raises(RuntimeError):
        ops.PeerComm(3, 2, max_out_elems=16)
    c = ops.PeerComm(0, 2, max_out_elems=8 * 256, timeout_ms=50)
    try:
        x, w, s, bh = make_dense(8, 256, 256, seed=6)
        with pytest.raises(RuntimeError, match="not attached"):
            ops.w8a16_linear_allreduce(c, x.cuda(), w.cuda(), s.cuda(), 256, 256, bh, 128)
        c.attach_ptr(1, c.base)
        x2, w2, s2, _ = make_dense(16, 256, 256, seed=7)
        with pytest.raises(RuntimeError, match="exceeds"):
            ops.w8a16_linear_allreduce(c, x2.cuda(), w2.cuda(), s2.cuda(), 256, 256, bh, 128)
        x3, w3, s3, _ = make_dense(2, 1022, 256, seed=8)
        with pytest.raises(RuntimeError, match="multiple of 4"):
            ops.w8a16_linear_allreduce(c, x3.cuda(), w3.cuda(), s3.cuda(), 1022, 256, bh, 128)
    finally:
        c.close()
