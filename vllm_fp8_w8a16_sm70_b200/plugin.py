"""Installs the B200 engine behind vLLM's FP8 quantization-method hooks.

The reference does this by attribute assignment on vLLM's classes at import of its launcher
(``src/fp8_w8a16_sm70/vllm_serve.py:2579-2719``; compressed-tensors:
``src/fp8_w8a16_sm70/compressed_tensors_v100.py:448-451, 548-574, 1226-1229``).  ``install()`` performs the
same assignments with this package's hook bodies and returns what it patched; ``uninstall()`` restores the
originals.  Nothing else of the reference's launcher (capability overrides, Marlin switches, attention
bridges, profiling hooks) is reproduced: on Blackwell vLLM needs none of them.

Only the hot-path hooks are replaced:

* ``Fp8LinearMethod.process_weights_after_loading`` / ``.apply`` (block-quantised checkpoints only; anything
  else keeps vLLM's own method, as the reference falls back at ``vllm_serve.py:1471-1475``)
* ``Fp8MoEMethod`` / ``Fp8OnlineMoEMethod``: ``process_weights_after_loading``, ``apply`` (5- and 6-argument
  forms), ``maybe_make_prepare_finalize``
* ``CompressedTensorsW8A16Fp8.process_weights_after_loading`` / ``.apply_weights``
* ``CompressedTensorsW8A8Fp8MoEMethod.__init__`` / ``.process_weights_after_loading`` / ``.apply`` /
  ``.get_fused_moe_quant_config`` (the four attributes the reference assigns, compressed_tensors_v100.py:1226-1229);
  the experts stay FP8-resident here instead of being dequantised to FP16 at load
"""

from __future__ import annotations

from typing import Dict, List

from . import linear_method as _lm
from . import moe_method as _mm

_ORIGINALS: Dict[tuple, object] = {}


def _patch(cls, name: str, fn) -> str:
    key = (cls, name)
    if key not in _ORIGINALS:
        _ORIGINALS[key] = cls.__dict__.get(name, None)
    setattr(cls, name, fn)
    return f"{cls.__module__}.{cls.__qualname__}.{name}"


def _strategy_name(self) -> str:
    strat = getattr(self, "strategy", "")
    return str(getattr(strat, "name", strat)).upper()


def install() -> List[str]:
    """Patch the vLLM classes that are importable in this environment; returns the patched attribute paths."""
    patched: List[str] = []
    from vllm.model_executor.layers.quantization import fp8 as vfp8

    orig_pwal = vfp8.Fp8LinearMethod.process_weights_after_loading
    orig_apply = vfp8.Fp8LinearMethod.apply

    def linear_pwal(self, layer):
        if not getattr(self, "block_quant", False):
            return orig_pwal(self, layer)          # non-block FP8 is not this engine's scope
        _lm.Fp8LinearMethod.process_weights_after_loading(self, layer)
        layer._b200_fp8 = True

    def linear_apply(self, layer, x, bias=None):
        if not getattr(layer, "_b200_fp8", False):
            return orig_apply(self, layer, x, bias)
        return _lm.Fp8LinearMethod.apply(self, layer, x, bias)

    patched.append(_patch(vfp8.Fp8LinearMethod, "process_weights_after_loading", linear_pwal))
    patched.append(_patch(vfp8.Fp8LinearMethod, "apply", linear_apply))

    for cls_name in ("Fp8MoEMethod", "Fp8OnlineMoEMethod"):
        cls = getattr(vfp8, cls_name, None)
        if cls is None:
            continue

        def moe_pwal(self, layer):
            if not hasattr(self, "weight_scale_name"):
                self.weight_scale_name = "weight_scale_inv" if getattr(self, "block_quant", False) else "weight_scale"
            if not hasattr(self, "block_h"):
                self.block_h = 128
            _mm.Fp8MoEMethod.process_weights_after_loading(self, layer)

        def moe_apply(self, layer, x, topk_weights, topk_ids, *shared, **kw):
            if not hasattr(self, "block_h"):
                self.block_h = 128
            return _mm.Fp8MoEMethod.apply(self, layer, x, topk_weights, topk_ids)

        patched.append(_patch(cls, "process_weights_after_loading", moe_pwal))
        patched.append(_patch(cls, "apply", moe_apply))
        patched.append(_patch(cls, "maybe_make_prepare_finalize", _mm.Fp8MoEMethod.maybe_make_prepare_finalize))

    try:
        from vllm.model_executor.layers.quantization.compressed_tensors.schemes import CompressedTensorsW8A16Fp8 as VCT
    except Exception:  # compressed-tensors is optional in a vLLM build
        VCT = None
    if VCT is not None:
        def ct_pwal(self, layer):
            shim = _lm.CompressedTensorsW8A16Fp8(_strategy_name(self), getattr(self, "weight_block_size", None))
            shim.process_weights_after_loading(layer)

        def ct_apply(self, layer, x, bias=None):
            return _lm.CompressedTensorsW8A16Fp8.apply_weights(self, layer, x, bias)

        patched.append(_patch(VCT, "process_weights_after_loading", ct_pwal))
        patched.append(_patch(VCT, "apply_weights", ct_apply))
    patched.extend(_install_ct_moe())
    return patched


def _ct_moe_class():
    """The compressed-tensors FP8 MoE method class: a submodule of ``compressed_tensors_moe`` in newer vLLM, defined
    inline in that module in older ones (the reference binds to whichever exists, compressed_tensors_v100.py:1003-1010)."""
    try:
        from vllm.model_executor.layers.quantization.compressed_tensors.compressed_tensors_moe import (
            compressed_tensors_moe_w8a8_fp8 as mod)
    except Exception:
        try:
            from vllm.model_executor.layers.quantization.compressed_tensors import compressed_tensors_moe as mod
        except Exception:
            return None
    return getattr(mod, "CompressedTensorsW8A8Fp8MoEMethod", None)


def _install_ct_moe() -> List[str]:
    cls = _ct_moe_class()
    if cls is None:
        return []
    orig_init = cls.__init__

    def shim_of(self):
        shim = getattr(self, "_b200_moe", None)
        if shim is None:
            shim = self._b200_moe = _mm.CompressedTensorsFp8MoEMethod(getattr(self, "weight_quant", None))
        return shim

    def ct_moe_init(self, weight_quant, input_quant, moe, layer_name=None):
        orig_init(self, weight_quant, input_quant, moe, layer_name)
        self._b200_moe = _mm.CompressedTensorsFp8MoEMethod(weight_quant, input_quant, moe, layer_name)

    def ct_moe_pwal(self, layer):
        shim_of(self).process_weights_after_loading(layer)

    def ct_moe_apply(self, layer, x, topk_weights, topk_ids, *shared, **kw):
        return shim_of(self).apply(layer, x, topk_weights, topk_ids)

    def ct_moe_quant_config(self, layer):
        return None

    return [_patch(cls, "__init__", ct_moe_init), _patch(cls, "process_weights_after_loading", ct_moe_pwal),
            _patch(cls, "apply", ct_moe_apply), _patch(cls, "get_fused_moe_quant_config", ct_moe_quant_config)]


def register() -> None:
    """``vllm.general_plugins`` entry point (declared in pyproject.toml): vLLM calls it once per process at start-up.
    Builds nothing and touches no GPU; a missing library surfaces at the first layer that calls into the engine."""
    install()


def uninstall() -> None:
    for (cls, name), orig in list(_ORIGINALS.items()):
        if orig is None:
            try:
                delattr(cls, name)
            except AttributeError:
                pass
        else:
            setattr(cls, name, orig)
    _ORIGINALS.clear()
