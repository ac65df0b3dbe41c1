"""The C-ABI library loads without a GPU and exports every symbol include/*.h declares; argument
validation answers with error codes before any device work."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "fp8w8a16_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fp8w8a16_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound(lib):
    from vllm_fp8_w8a16_sm70_b200 import _cabi
    syms = declared_symbols()
    assert len(syms) >= 15
    for s in syms:
        assert hasattr(lib, s), f"{s} declared in the header but not exported"
        assert s in _cabi.PROTOTYPES, f"{s} has no ctypes prototype"
    assert set(_cabi.PROTOTYPES) == set(syms)
    assert lib.fp8w8a16_version() >= 100


def test_validation_returns_codes_without_a_gpu(lib):
    from vllm_fp8_w8a16_sm70_b200 import _cabi
    rc = lib.fp8w8a16_linear(None, None, None, 0, None, 4, 128, 128, 128, 128, 0, None, 0, None)
    assert rc == _cabi.ERR_INVALID and "null" in _cabi.last_error()
    buf = (ctypes.c_char * 64)()
    p = ctypes.addressof(buf)
    p16 = (p + 15) & ~15
    rc = lib.fp8w8a16_linear(p16, p16, p16, 0, p16, 4, 128, 100, 128, 128, 0, None, 0, None)
    assert rc == _cabi.ERR_UNSUPPORTED and "multiple of 16" in _cabi.last_error()
    rc = lib.fp8w8a16_linear(p16, p16, p16, 0, p16, 4, 128, 128, 128, 64, 0, None, 0, None)
    assert rc == _cabi.ERR_UNSUPPORTED and "block_w" in _cabi.last_error()
    rc = lib.fp8w8a16_linear(p16 + 2, p16, p16, 0, p16, 4, 128, 128, 128, 128, 0, None, 0, None)
    assert rc == _cabi.ERR_INVALID and "aligned" in _cabi.last_error()
    rc = lib.fp8w8a16_moe_topk_softmax(p16, 0, 1, 4096, 8, 1, p16, p16, None)
    assert rc == _cabi.ERR_UNSUPPORTED
    # empty problems are a no-op, not an error (reference tests R = 0)
    assert lib.fp8w8a16_linear(None, None, None, 0, None, 0, 128, 128, 128, 128, 0, None, 0, None) == 0
    assert lib.fp8w8a16_e4m3_to_fp16(None, None, 0, None) == 0
    assert lib.fp8w8a16_linear_workspace_bytes(1, 5120, 5120) >= 65536
    assert lib.fp8w8a16_moe_token_tile(8, 128) == 16 and lib.fp8w8a16_moe_token_tile(16384, 128) == 128


def test_ops_refuse_cpu_tensors(lib):
    from vllm_fp8_w8a16_sm70_b200 import ops
    x = torch.zeros(2, 128, dtype=torch.float16)
    w = torch.zeros(128, 128, dtype=torch.uint8)
    s = torch.ones(1, 1, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ops.w8a16_linear(x, w, s, 128, 128)
    with pytest.raises(RuntimeError):
        ops.fp8_e4m3_to_fp16(w)


def test_linear_method_load_time_rules(lib):
    """process_weights_after_loading: BF16 scale -> FP16, layouts kept, non-block fails closed
    (vllm_serve.py:1450-1523, :2629-2635); scale range guard."""
    import types
    from vllm_fp8_w8a16_sm70_b200 import Fp8LinearMethod, CompressedTensorsW8A16Fp8
    layer = types.SimpleNamespace(weight=torch.zeros(256, 384, dtype=torch.uint8).view(torch.float8_e4m3fn),
                                  weight_scale_inv=torch.full((2, 3), 0.01, dtype=torch.bfloat16), weight_block_size=[128, 128],
                                  input_size_per_partition=384, output_size_per_partition=256, input_scale=torch.ones(1))
    Fp8LinearMethod((128, 128)).process_weights_after_loading(layer)
    assert layer.weight_scale_inv.dtype == torch.float16 and layer.input_scale is None
    assert layer.weight.dtype == torch.float8_e4m3fn and tuple(layer.weight.shape) == (256, 384)
    with pytest.raises(NotImplementedError):
        Fp8LinearMethod(None).process_weights_after_loading(layer)
    layer.weight_scale_inv = torch.full((2, 3), 1.0e6)   # overflows FP16
    with pytest.raises(RuntimeError, match="scale"):
        Fp8LinearMethod((128, 128)).process_weights_after_loading(layer)
    # compressed-tensors channel: [N,1] -> [N, Kb] block_h = 1 grid (compressed_tensors_v100.py:488-492)
    ct = types.SimpleNamespace(weight=torch.zeros(352, 384, dtype=torch.uint8), weight_scale=torch.rand(352, 1) * 0.02 + 0.01)
    m = CompressedTensorsW8A16Fp8("channel")
    m.process_weights_after_loading(ct)
    assert tuple(ct.weight_scale.shape) == (352, 3) and ct._b200_block_h == 1
    assert (ct.weight_scale[:, 0] == ct.weight_scale[:, 2]).all()
    # tensor: one scale per logical shard (compressed_tensors_v100.py:247-256)
    ct = types.SimpleNamespace(weight=torch.zeros(352, 384, dtype=torch.uint8), weight_scale=torch.tensor([0.01, 0.02, 0.03]),
                               logical_widths=[128, 64, 160])
    CompressedTensorsW8A16Fp8("tensor").process_weights_after_loading(ct)
    assert float(ct.weight_scale[127, 0]) == pytest.approx(0.01, rel=1e-3)
    assert float(ct.weight_scale[128, 0]) == pytest.approx(0.02, rel=1e-3)
    assert float(ct.weight_scale[351, 2]) == pytest.approx(0.03, rel=1e-3)
    bad = types.SimpleNamespace(weight=torch.zeros(352, 384, dtype=torch.uint8), weight_scale=torch.rand(7))
    with pytest.raises(ValueError):
        CompressedTensorsW8A16Fp8("channel").process_weights_after_loading(bad)


def test_variant_counters_exported_and_named(lib):
    """The per-variant call counters: one name per FP8W8A16_VARIANT_* index, all zero before any GPU call here."""
    from vllm_fp8_w8a16_sm70_b200 import _cabi
    counts = _cabi.variant_counts()
    assert list(counts) == list(_cabi.VARIANT_NAMES) and len(counts) == 8
    assert all(isinstance(v, int) and v >= 0 for v in counts.values())


def test_observability_summary_without_gpu(lib, monkeypatch, capsys):
    from vllm_fp8_w8a16_sm70_b200 import observability as obs
    obs.reset()
    monkeypatch.setenv("FP8W8A16_VARIANT_LOG_EVERY", "2")
    monkeypatch.setenv("FP8W8A16_PREFIX_PROFILE", "1")
    obs.reload_env()
    import types
    obs.on_apply(types.SimpleNamespace(prefix="model.layers.0.mlp.down_proj"))
    assert capsys.readouterr().err == ""
    obs.on_apply(types.SimpleNamespace(prefix="model.layers.0.mlp.down_proj"))
    err = capsys.readouterr().err
    assert "kernel variant counts after 2 hook calls" in err and "model.layers.0.mlp.down_proj: calls=2" in err
    monkeypatch.setenv("FP8W8A16_VARIANT_LOG_EVERY", "0")
    obs.reload_env()
    obs.on_apply(None)
    assert capsys.readouterr().err == ""
    obs.reset()
    with pytest.raises(RuntimeError, match="GPU"):
        import torch
        obs.selfcheck_linear(torch.zeros(128, 128, dtype=torch.uint8), torch.ones(1, 1, dtype=torch.float16), 128, 128, 128)
