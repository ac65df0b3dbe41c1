"""The steps that follow a row-parallel projection, fused around the GEMM: the residual add in the GEMM's epilogue
(out = FP16(fp32 result + residual), one rounding) and the add + RMSNorm kernel.  Oracle: the fp32-accumulate linear oracle
plus the residual in fp32; the norm against an fp32 PyTorch restatement with vLLM's rounding points."""
import pytest
import torch

from oracle import linear as olin
from tests.helpers import make_dense

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(lib):
    from vllm_fp8_w8a16_sm70_b200 import ops as _ops
    return _ops


# cluster split-K with pushed slices (16 / 32 tokens), cluster split-K with pulled slices (64), stream-K, whole tiles, ragged N
@pytest.mark.parametrize("M,N,K", [(1, 5120, 5120), (8, 5120, 5120), (24, 5120, 2560), (64, 5120, 2560), (4, 38400, 1024), (300, 512, 256),
                                   (7, 1000, 384), (2048, 1024, 512)])
def test_residual_joins_the_epilogue_with_one_rounding(ops, M, N, K):
    x, w, s, bh = make_dense(M, N, K, seed=M + N)
    res = (torch.randn(M, N, generator=torch.Generator().manual_seed(K)) * 2).to(torch.float16)
    xd, wd, sd, rd = x.cuda(), w.cuda(), s.cuda(), res.cuda()
    y = ops.w8a16_linear(xd, wd, sd, N, K, bh, 128, residual=rd)
    acc = olin.oracle_linear_fp32(x, w, s, bh)
    olin.check_linear(y.cpu(), x, acc + res.float(), K)
    # one rounding: never further from the fp32 sum than rounding the plain GEMM result first and adding afterwards
    plain = ops.w8a16_linear(xd, wd, sd, N, K, bh, 128, algo=ops.ALGO_TC)
    two_step = (plain.float() + rd.float()).to(torch.float16)
    ref = (acc + res.float()).cuda()
    assert float((y.float() - ref).abs().mean()) <= float((two_step.float() - ref).abs().mean()) * 1.001 + 1e-7
    # in place: out may be the residual tensor itself
    r2 = rd.clone()
    ops.w8a16_linear(xd, wd, sd, N, K, bh, 128, residual=r2, out=r2)
    assert torch.equal(r2.view(torch.int16), y.view(torch.int16))
    with pytest.raises(RuntimeError, match="residual"):
        ops.w8a16_linear(xd, wd, sd, N, K, bh, 128, residual=rd[:, : N // 2])


@pytest.mark.parametrize("M,N", [(1, 5120), (9, 4096), (64, 5120), (3, 24576), (300, 256)])
@pytest.mark.parametrize("with_residual", [True, False])
def test_add_rmsnorm(ops, M, N, with_residual):
    g = torch.Generator().manual_seed(M * 31 + N)
    x = torch.randn(M, N, generator=g).to(torch.float16)
    r = (torch.randn(M, N, generator=g) * 3).to(torch.float16) if with_residual else None
    wt = (1 + 0.1 * torch.randn(N, generator=g)).to(torch.float16)
    eps = 1e-5
    out, z = ops.add_rmsnorm(x.cuda(), wt.cuda(), eps, residual=None if r is None else r.cuda())
    z_ref = (x.float() + r.float()).to(torch.float16) if with_residual else x
    assert torch.equal(z.cpu().view(torch.int16), z_ref.view(torch.int16)), "z = FP16(x + residual), one rounding"
    zf = z_ref.float()
    inv = torch.rsqrt(zf.pow(2).mean(dim=1, keepdim=True) + eps)
    ref = ((zf * inv).to(torch.float16) * wt).float()
    got = out.cpu().float()
    # the reciprocal square root is an approximation on both sides: allow one FP16 ulp of the normalised value
    assert torch.allclose(got, ref, atol=2e-3, rtol=2e-3), float((got - ref).abs().max())
    if with_residual:
        r2 = r.cuda()
        out2, z2 = ops.add_rmsnorm(x.cuda(), wt.cuda(), eps, residual=r2, inplace_residual=True)
        assert z2.data_ptr() == r2.data_ptr() and torch.equal(r2.cpu().view(torch.int16), z_ref.view(torch.int16))
        assert torch.equal(out2.view(torch.int16), out.view(torch.int16))


def test_projection_residual_norm_chain(ops):
    """o_proj-like projection with the residual added in its epilogue, then the norm without a second add: equals the
    unfused order (GEMM, then add + norm) up to the one rounding the fusion removes."""
    M, N, K = 16, 5120, 5120
    x, w, s, bh = make_dense(M, N, K, seed=77)
    g = torch.Generator().manual_seed(1)
    res = torch.randn(M, N, generator=g).to(torch.float16)
    wt = (1 + 0.05 * torch.randn(N, generator=g)).to(torch.float16)
    xd, wd, sd = x.cuda(), w.cuda(), s.cuda()
    z = ops.w8a16_linear(xd, wd, sd, N, K, bh, 128, residual=res.cuda())
    fused, z_same = ops.add_rmsnorm(z, wt.cuda(), 1e-6)
    assert z_same.data_ptr() == z.data_ptr()
    y = ops.w8a16_linear(xd, wd, sd, N, K, bh, 128)
    unfused, z_un = ops.add_rmsnorm(y, wt.cuda(), 1e-6, residual=res.cuda())
    assert torch.allclose(fused.float(), unfused.float(), atol=6e-3, rtol=6e-3)
    zr = olin.oracle_linear_fp32(x, w, s, bh) + res.float()
    ref = (zr * torch.rsqrt(zr.pow(2).mean(dim=1, keepdim=True) + 1e-6)) * wt.float()
    assert float((fused.cpu().float() - ref).norm() / ref.norm()) < 5e-3
