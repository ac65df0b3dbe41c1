"""GPU parity, bit-exact: FP8 -> FP16 conversion and the dequantised weight, through the C ABI."""
import numpy as np
import pytest
import torch

from oracle import dequant
from tests.helpers import bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(lib):
    from vllm_fp8_w8a16_sm70_b200 import ops as _ops
    return _ops


def test_all_256_bytes_bit_exact(ops, golden_dir):
    # reference: tests/test_fp8.py:160-179
    gold = np.load(golden_dir / "e4m3_table.npz")["fp16_bits"]
    out = ops.fp8_e4m3_to_fp16(torch.arange(256, dtype=torch.uint8, device="cuda"))
    assert (bits(out) == gold).all()
    assert ops.fp8_e4m3_to_fp16(torch.empty(0, dtype=torch.uint8, device="cuda")).numel() == 0


@pytest.mark.parametrize("N,K,bh,bw", [(256, 512, 128, 128), (200, 304, 128, 128), (352, 176, 1, 128), (1, 16, 128, 128),
                                       (130, 400, 128, 128), (64, 100, 128, 128), (77, 33, 16, 32)])
@pytest.mark.parametrize("sdtype", [torch.float16, torch.float32])
def test_block_dequant_bit_exact_random_bytes(ops, N, K, bh, bw, sdtype):
    """Every byte value incl. both NaN encodings, subnormal products (tiny scales), fp32 scales rounded to FP16."""
    g = torch.Generator().manual_seed(N * 1000 + K)
    w = torch.randint(0, 256, (N, K), generator=g, dtype=torch.uint8)
    nb, kb = -(-N // bh), -(-K // bw)
    s = (torch.rand(nb, kb, generator=g) * 0.02 + 1e-5).to(sdtype)
    s[0, 0] = 6.1e-5 if sdtype == torch.float16 else 1.0e-7   # FP16-subnormal scale
    want = dequant.dequant_block_scaled(w.numpy(), s, N, K, bh, bw)
    got = ops.fp8_e4m3_to_fp16_block_scaled(w.cuda(), s.cuda(), N, K, bh, bw)
    assert (bits(got) == want.view(np.uint16)).all()


def test_block_dequant_golden_fixture(ops, golden_dir):
    z = np.load(golden_dir / "dense_reference.npz")
    w = torch.from_numpy(z["b_w"]).cuda()
    N, K = w.shape
    got = ops.fp8_e4m3_to_fp16_block_scaled(w, torch.from_numpy(z["b_s32"]).cuda(), N, K)
    assert (bits(got) == z["b_wdq16"]).all()


def test_ct_layouts_golden_fixture(ops, golden_dir):
    z = np.load(golden_dir / "ct_dequant.npz")
    N, K = z["channel_w"].shape
    grid = torch.from_numpy(dequant.channel_scales_as_blocks(z["channel_s"], N, K)).cuda()
    got = ops.fp8_e4m3_to_fp16_block_scaled(torch.from_numpy(z["channel_w"]).cuda(), grid, N, K, 1, 128)
    assert (bits(got) == z["channel_out"]).all()
    per_row = dequant.tensor_scales_as_channel(z["tensor_s"], z["tensor_widths"].tolist())
    grid = torch.from_numpy(dequant.channel_scales_as_blocks(per_row, N, K)).cuda()
    got = ops.fp8_e4m3_to_fp16_block_scaled(torch.from_numpy(z["tensor_w"]).cuda(), grid, N, K, 1, 128)
    assert (bits(got) == z["tensor_out"]).all()


def test_group_scaled(ops):
    # reference: tests/test_fp8.py:38-107
    g = torch.Generator().manual_seed(5)
    w = torch.randint(0, 256, (4096,), generator=g, dtype=torch.uint8)
    w[(w & 0x7F) == 0x7F] = 0x3C
    s = (torch.rand(32, generator=g) * 0.1).to(torch.float16)
    want = dequant.dequant_group_scaled(w.numpy(), s, 128)
    got = ops.fp8_e4m3_to_fp16_scaled(w.cuda(), s.cuda(), 128)
    assert (bits(got) == want.view(np.uint16)).all()


def test_full_size_gate_up_weight_matches_torch_on_device(ops):
    """[51200, 5120] (the largest dense weight of the decode sweep): compared on the device with torch's own
    fp8 -> fp16 conversion and FP16 multiply, which round the same way."""
    N, K = 51200, 5120
    g = torch.Generator(device="cuda").manual_seed(0)
    w = torch.randint(0, 256, (N, K), generator=g, dtype=torch.uint8, device="cuda")
    w[(w & 0x7F) == 0x7F] = 0x11
    s = (torch.rand(N // 128, K // 128, generator=g, device="cuda") * 3e-4 + 1e-5)
    got = ops.fp8_e4m3_to_fp16_block_scaled(w, s, N, K)
    ref = w.view(torch.float8_e4m3fn).to(torch.float16) * s.to(torch.float16).repeat_interleave(128, 0).repeat_interleave(128, 1)
    assert torch.equal(got.view(torch.int16), ref.view(torch.int16))
