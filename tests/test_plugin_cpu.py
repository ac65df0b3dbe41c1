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
    finally:
        plugin.uninstall()
    assert (fp8.Fp8LinearMethod.apply, fp8.Fp8LinearMethod.process_weights_after_loading, fp8.Fp8MoEMethod.apply) == before


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
