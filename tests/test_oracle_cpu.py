"""CPU suite: the oracle against the reference's known answers and the committed golden fixtures
(made by executing the reference's own Python, tests/golden/make_golden.py)."""
import ctypes
import json

import numpy as np
import torch

from oracle import dequant, e4m3, linear as olin, moe as omoe, tp as otp
from tests.helpers import bits, f16_from_bits


def test_e4m3_edge_table_known_answers():
    # reference: tests/test_fp8.py:119-134
    for b, v in e4m3.EDGE_CASES:
        got = float(e4m3.e4m3_to_fp16(np.array([b], np.uint8))[0])
        by_def = e4m3.e4m3_to_float_by_definition(b)
        if v is None:
            assert got != got and by_def != by_def
            assert int(e4m3.e4m3_to_fp16_bits(np.array([b], np.uint8))[0]) == ((b & 0x80) << 8 | 0x7F80)
        else:
            assert got == v == by_def, (hex(b), got, v, by_def)
            assert np.signbit(np.float16(got)) == bool(b & 0x80) or got != 0


def test_e4m3_all_256_bytes_vs_golden_and_torch(golden_dir, c_oracle):
    # reference: tests/test_fp8.py:160-179 (bit-exact for all 256 bytes)
    gold = np.load(golden_dir / "e4m3_table.npz")["fp16_bits"]
    assert (e4m3.table_bits() == gold).all()
    live = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).to(torch.float16)
    assert (bits(live) == gold).all()
    tab = np.zeros(256, np.uint16)
    c_oracle.ref_e4m3_table(tab.ctypes.data_as(ctypes.c_void_p))
    assert (tab == gold).all()
    for b in range(256):
        d = e4m3.e4m3_to_float_by_definition(b)
        h = float(gold[b:b + 1].view(np.float16)[0])
        assert (d != d and h != h) or d == h


def test_block_dequant_vs_reference_fixture(golden_dir, c_oracle):
    z = np.load(golden_dir / "dense_reference.npz")
    w, s16 = z["b_w"], z["b_s16"]
    N, K = w.shape
    out = dequant.dequant_block_scaled(w, s16.view(np.float16), N, K)
    assert (out.view(np.uint16) == z["b_wdq16"]).all()          # reference_matmul's dequantised weight
    assert (out.view(np.uint16) == z["b_wdq_fp16path"]).all()   # the reference's torch fp16 path
    # fp32 scales handed to the engine are rounded to FP16 first (vllm_serve.py:1512-1513)
    out32 = dequant.dequant_block_scaled(w, z["b_s32"], N, K)
    assert (out32.view(np.uint16) == z["b_wdq16"]).all()
    co = np.zeros((N, K), np.uint16)
    c_oracle.ref_dequant_block(w.ctypes.data_as(ctypes.c_void_p), np.ascontiguousarray(s16).ctypes.data_as(ctypes.c_void_p),
                               co.ctypes.data_as(ctypes.c_void_p), ctypes.c_int64(N), ctypes.c_int64(K), 128, 128)
    assert (co == z["b_wdq16"]).all()


def test_ct_dequant_block_channel_tensor_vs_reference(golden_dir):
    # reference: compressed_tensors_v100.py:231-270 executed by make_golden.py
    z = np.load(golden_dir / "ct_dequant.npz")
    N, K = z["block_w"].shape
    out = dequant.dequant_block_scaled(z["block_w"], torch.from_numpy(z["block_s_bf16_as_f32"]), N, K)
    assert (out.view(np.uint16) == z["block_out"]).all()
    grid = dequant.channel_scales_as_blocks(z["channel_s"], N, K)
    out = dequant.dequant_block_scaled(z["channel_w"], grid, N, K, block_h=1)
    assert (out.view(np.uint16) == z["channel_out"]).all()
    per_row = dequant.tensor_scales_as_channel(z["tensor_s"], z["tensor_widths"].tolist())
    out = dequant.dequant_block_scaled(z["tensor_w"], dequant.channel_scales_as_blocks(per_row, N, K), N, K, block_h=1)
    assert (out.view(np.uint16) == z["tensor_out"]).all()


def test_linear_oracle_vs_reference_matmul(golden_dir):
    # reference: tests/test_attention_shapes.py:104-120
    z = np.load(golden_dir / "dense_reference.npz")
    for tag in "abc":
        x = f16_from_bits(z[f"{tag}_x"])
        w = torch.from_numpy(z[f"{tag}_w"])
        s16 = f16_from_bits(z[f"{tag}_s16"])
        y = olin.oracle_linear_fp32(x, w, s16)
        ref = f16_from_bits(z[f"{tag}_y16"]).float()
        assert torch.allclose(y, ref, atol=2e-3, rtol=2e-3), tag   # fixture is rounded to FP16
        y_cpu, _ = olin.reference_cpu_linear(x, w, s16)
        olin.check_linear(y_cpu, x, y, w.shape[1])


def test_tp_sharding_vs_reference(golden_dir):
    # reference: tests/test_attention_shapes.py:75-101
    z = np.load(golden_dir / "dense_reference.npz")
    W = torch.from_numpy(z["a_w"]); S = torch.from_numpy(z["a_s16"].view(np.int16).copy())
    for r in range(4):
        wc, sc = otp.shard_col_parallel(W, S, 4, r)
        wr, sr = otp.shard_row_parallel(W, S, 4, r)
        assert (wc.numpy() == z[f"a_col{r}_w"]).all() and (sc.numpy().view(np.uint16) == z[f"a_col{r}_s16"]).all()
        assert (wr.numpy() == z[f"a_row{r}_w"]).all() and (sr.numpy().view(np.uint16) == z[f"a_row{r}_s16"]).all()
    fw, fs = otp.fuse_merged([otp.shard_col_parallel(W, S, 4, 0)[0], otp.shard_col_parallel(W, S, 4, 2)[0]],
                             [otp.shard_col_parallel(W, S, 4, 0)[1], otp.shard_col_parallel(W, S, 4, 2)[1]])
    assert (fw.numpy() == z["a_fused_w"]).all() and (fs.numpy().view(np.uint16) == z["a_fused_s16"]).all()


def test_tp_shards_recompose_the_full_layer():
    from tests.helpers import make_dense
    x, w, s, bh = make_dense(4, 512, 1024, seed=3)
    full = olin.oracle_linear_fp32(x, w, s)
    cols = [olin.oracle_linear_fp32(x, *otp.shard_col_parallel(w, s, 4, r)) for r in range(4)]
    assert torch.allclose(torch.cat(cols, 1), full, atol=1e-5)
    rows = sum(olin.oracle_linear_fp32(x[:, r * 256:(r + 1) * 256], *otp.shard_row_parallel(w, s, 4, r)) for r in range(4))
    assert torch.allclose(rows, full, atol=1e-3)


def test_moe_oracle_vs_reference_loop(golden_dir):
    # reference: tools/ct_fp8_mixed_moe_numtest_vllm021.sh:61-73 executed by make_golden.py
    z = np.load(golden_dir / "moe_reference.npz")
    E, I, H, M, topk = z["dims"].tolist()
    x = f16_from_bits(z["x"])
    s13 = f16_from_bits(z["s13"]).expand(E, 2 * I, -(-H // 128)).contiguous()
    s2 = torch.from_numpy(z["s2"]).to(torch.float16).expand(E, H, -(-I // 128)).contiguous()
    out = omoe.moe_reference_fp32(x, f16_from_bits(z["topk_w"]), torch.from_numpy(z["topk_ids"]), torch.from_numpy(z["w13"]),
                                  s13, torch.from_numpy(z["w2"]), s2, block_h=1)
    st = omoe.check_moe(out, torch.from_numpy(z["out_f32"]))
    assert st["l2rel"] < 2e-3, st   # only the FP16 rounding of s2 separates the two
    chain = omoe.moe_reference_fp16_chain(x, f16_from_bits(z["topk_w"]), torch.from_numpy(z["topk_ids"]),
                                          torch.from_numpy(z["w13"]), s13, torch.from_numpy(z["w2"]), s2, block_h=1)
    omoe.check_moe(chain, torch.from_numpy(z["out_f32"]))


def test_route_topk_rule():
    lg = torch.tensor([[0.5, 2.0, 2.0, -1.0, 0.5, 3.0]])
    ids, w = omoe.route_topk(lg, 4, renormalize=True)
    assert ids.tolist() == [[5, 1, 2, 0]]          # descending, ties to the lowest index
    assert abs(float(w.sum()) - 1.0) < 1e-6
    ids2, w2 = omoe.route_topk(lg, 4, renormalize=False)
    p = torch.softmax(lg, -1)
    assert torch.allclose(w2, p[0, ids2[0].long()].unsqueeze(0))


def test_align_and_remap_oracle():
    ids = torch.tensor([3, 1, -1, 3, 0, 7, 1, 3])
    emap = torch.tensor([0, 1, -1, 2, -1, -1, -1, -1], dtype=torch.int32)
    local = omoe.remap_expert_ids(ids, emap)
    assert local.tolist() == [2, 1, -1, 2, 0, -1, 1, 2]
    counts, offsets, order = omoe.align_routes(local, 3)
    assert counts.tolist() == [1, 2, 3] and offsets.tolist() == [0, 1, 3, 6]
    assert order.tolist() == [4, 1, 6, 0, 3, 7]     # stable inside each expert


def test_selector_collapses_reference_cases(golden_dir):
    from vllm_fp8_w8a16_sm70_b200 import backend
    cases = json.loads((golden_dir / "selector_cases.json").read_text())
    assert {c["reference_backend"] for c in cases} == {"ours", "turbomind"}
    for c in cases:
        kw = dict(c["kwargs"])
        if kw.get("weight_block_size") is not None:
            kw["weight_block_size"] = tuple(kw["weight_block_size"])
        # every weight the reference serves on either of its engines is served by the one engine
        assert backend.select_backend(**kw)[0] == "b200"
    import pytest
    with pytest.raises(RuntimeError):   # unsupported weight fails loudly, as turbomind mode does (turbomind_fp8_backend.py:198-202)
        backend.select_backend(strategy="BLOCK", weight_block_size=(64, 64), local_n=128, local_k=128)
    with pytest.raises(RuntimeError):
        backend.select_backend(strategy="CHANNEL", weight_block_size=None, local_n=8, local_k=8)
