"""The vLLM hook installer lands on the classes the reference patches (reference: tests/test_wrapper_imports.py)
and can be undone.  Skipped where vLLM is not importable."""
import pytest


def test_install_and_uninstall_patch_the_hook_attributes():
    fp8 = pytest.importorskip("vllm.model_executor.layers.quantization.fp8")
    from vllm_fp8_w8a16_sm70_b200 import plugin
    before = (fp8.Fp8LinearMethod.apply, fp8.Fp8LinearMethod.process_weights_after_loading, fp8.Fp8MoEMethod.apply)
    patched = plugin.install()
    try:
        assert any(p.endswith("Fp8LinearMethod.apply") for p in patched)
        assert any(p.endswith("Fp8MoEMethod.apply") for p in patched)
        assert fp8.Fp8LinearMethod.apply is not before[0]
        assert fp8.Fp8LinearMethod.apply.__module__ == "vllm_fp8_w8a16_sm70_b200.plugin"
        assert fp8.Fp8MoEMethod.maybe_make_prepare_finalize(object()) is None
        ct_moe = plugin._ct_moe_class()
        if ct_moe is not None:      # the four attributes the reference assigns (compressed_tensors_v100.py:1226-1229)
            for name in ("__init__", "process_weights_after_loading", "apply", "get_fused_moe_quant_config"):
                assert any(p.endswith(f"CompressedTensorsW8A8Fp8MoEMethod.{name}") for p in patched), name
                assert getattr(ct_moe, name).__module__ == "vllm_fp8_w8a16_sm70_b200.plugin"
            assert ct_moe.get_fused_moe_quant_config(object(), None) is None
    finally:
        plugin.uninstall()
    assert (fp8.Fp8LinearMethod.apply, fp8.Fp8LinearMethod.process_weights_after_loading, fp8.Fp8MoEMethod.apply) == before
    ct_moe = plugin._ct_moe_class()
    assert ct_moe is None or ct_moe.apply.__module__ != "vllm_fp8_w8a16_sm70_b200.plugin"


def test_ct_moe_method_expands_every_scale_layout_to_a_row_grid():
    """process_weights_after_loading of the compressed-tensors MoE hook on CPU tensors (no kernel runs): channel
    ``[E, rows, 1]``, per-tensor ``[E]`` and per-shard ``[E, 2]`` scales all become the ``block_h = 1`` grid
    ``[E, rows, ceil(K/128)]`` the engine reads; block grids pass through; anything else raises."""
    import types
    import torch
    from vllm_fp8_w8a16_sm70_b200.moe_method import CompressedTensorsFp8MoEMethod
    E, I, H = 3, 176, 256
    w13 = torch.zeros(E, 2 * I, H, dtype=torch.uint8)
    w2 = torch.zeros(E, H, I, dtype=torch.uint8)
    g = torch.Generator().manual_seed(0)
    ch13, ch2 = torch.rand(E, 2 * I, 1, generator=g) + 0.1, torch.rand(E, H, 1, generator=g) + 0.1
    lay = types.SimpleNamespace(w13_weight=w13, w2_weight=w2, w13_weight_scale=ch13, w2_weight_scale=ch2)
    m = CompressedTensorsFp8MoEMethod(types.SimpleNamespace(strategy=types.SimpleNamespace(name="CHANNEL")))
    assert m.strategy == "CHANNEL" and m.block_h == 1
    m.process_weights_after_loading(lay)
    assert tuple(lay.w13_weight_scale.shape) == (E, 2 * I, 2) and tuple(lay.w2_weight_scale.shape) == (E, H, 2)
    assert torch.equal(lay.w13_weight_scale[:, :, 1], ch13.to(torch.float16)[:, :, 0]) and lay.w2_weight_scale.is_contiguous()
    lay = types.SimpleNamespace(w13_weight=w13, w2_weight=w2, w13_weight_scale=torch.tensor([[1., 2.], [3., 4.], [5., 6.]]),
                                w2_weight_scale=torch.tensor([7., 8., 9.]))
    CompressedTensorsFp8MoEMethod(strategy="tensor").process_weights_after_loading(lay)
    assert bool((lay.w13_weight_scale[1, :I] == 3).all()) and bool((lay.w13_weight_scale[1, I:] == 4).all())
    assert bool((lay.w2_weight_scale[2] == 9).all())
    lay = types.SimpleNamespace(w13_weight=w13, w2_weight=w2, w13_weight_scale=torch.ones(E, 5), w2_weight_scale=ch2)
    with pytest.raises(ValueError):
        CompressedTensorsFp8MoEMethod(strategy="CHANNEL").process_weights_after_loading(lay)


def test_moe_block_folds_shared_expert_into_the_stack():
    """Constructor logic of the router + shared-expert block (no kernel runs): the shared expert becomes expert E."""
    import pytest
    import torch
    from vllm_fp8_w8a16_sm70_b200.moe_block import MoEBlock
    E, I, H = 4, 128, 256
    gate = torch.zeros(E, H, dtype=torch.float16)
    w13, s13 = torch.zeros(E, 2 * I, H, dtype=torch.uint8), torch.ones(E, 2, 2, dtype=torch.float16)
    w2, s2 = torch.zeros(E, H, I, dtype=torch.uint8), torch.ones(E, 2, 1, dtype=torch.float16)
    shared = (torch.full((2 * I, H), 7, dtype=torch.uint8), torch.full((2, 2), 0.5, dtype=torch.float16),
              torch.full((H, I), 9, dtype=torch.uint8), torch.full((2, 1), 0.25))
    blk = MoEBlock(gate, w13, s13, w2, s2, topk=2, shared=shared)
    assert blk.shared_id == E and blk.num_routed == E
    assert tuple(blk.w13.shape) == (E + 1, 2 * I, H) and bool((blk.w13[E] == 7).all()) and bool((blk.w2[E] == 9).all())
    assert blk.s2.dtype == torch.float16 and bool((blk.s2[E] == 0.25).all()) and bool((blk.s13[E] == 0.5).all())
    plain = MoEBlock(gate, w13, s13, w2, s2, topk=2)
    assert plain.shared_id == -1 and plain.w13.shape[0] == E
    with pytest.raises(ValueError):
        MoEBlock(gate[:, :128], w13, s13, w2, s2, topk=2)
    with pytest.raises(ValueError):
        MoEBlock(gate, w13, s13, w2, s2, topk=2, shared=(shared[0][:128], shared[1], shared[2], shared[3]))
    with pytest.raises(ValueError):
        MoEBlock(gate, w13, s13, w2, s2, topk=2, shared=(shared[0], shared[1][:1], shared[2], shared[3]))


def test_pyproject_declares_the_vllm_plugin_entry_point():
    """The packaging metadata names a `vllm.general_plugins` entry point that resolves to a callable of this package."""
    import importlib
    import tomllib
    from pathlib import Path
    meta = tomllib.loads((Path(__file__).resolve().parent.parent / "pyproject.toml").read_text())
    eps = meta["project"]["entry-points"]["vllm.general_plugins"]
    assert eps, "no vllm.general_plugins entry point"
    for target in eps.values():
        mod, fn = target.split(":")
        assert callable(getattr(importlib.import_module(mod), fn))
