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
