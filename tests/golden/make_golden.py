"""Generates tests/golden/*.npz by EXECUTING the reference's own Python (run where the reference
checkout is present; the fixtures are committed, this script documents how they were made).

    python tests/golden/make_golden.py /path/to/reference

What is executed, unmodified, from the reference tree (function bodies are taken from its files
with ``ast`` so that module-level imports of its CUDA extension are not triggered):

* ``tests/test_fp8.py:160-166``            torch CPU ``uint8.view(float8_e4m3fn).to(float16)`` byte table
* ``tests/test_attention_shapes.py``       ``reference_matmul``, ``shard_col_parallel``,
                                           ``shard_row_parallel``, ``fuse_qkv_merged``
* ``src/fp8_w8a16_sm70/compressed_tensors_v100.py``  ``_dequant_ct_weight_to_fp16`` (block / channel / tensor)
* ``tools/ct_fp8_mixed_moe_numtest_vllm021.sh``      ``ref_moe`` (the embedded Python reference loop)
* ``src/fp8_w8a16_sm70/turbomind_fp8_backend.py``    ``select_backend`` decisions of its ``_selftest`` cases

Inputs are small and seeded (CPU generator), so the files stay a few hundred KB.
"""

from __future__ import annotations

import ast
import importlib.util
import sys
import types
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

HERE = Path(__file__).resolve().parent


def _functions_from(path: Path, names, extra_globals=None, text=None):
    src = text if text is not None else path.read_text()
    tree = ast.parse(src)
    ns = {"torch": torch, "F": F}
    ns.update(extra_globals or {})
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name in names:
            code = compile(ast.Module(body=[node], type_ignores=[]), str(path), "exec")
            exec(code, ns)
    missing = [n for n in names if n not in ns]
    assert not missing, f"{path}: functions not found: {missing}"
    return [ns[n] for n in names]


def _u16(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def quant_block(w: torch.Tensor, bh=128, bw=128):
    N, K = w.shape
    Nb, Kb = -(-N // bh), -(-K // bw)
    wp = torch.zeros(Nb * bh, Kb * bw)
    wp[:N, :K] = w
    blk = wp.reshape(Nb, bh, Kb, bw)
    s = blk.abs().amax(dim=(1, 3)) / 448.0
    s = torch.where(s > 0, s, torch.ones_like(s))
    q = (blk / s[:, None, :, None]).reshape(Nb * bh, Kb * bw)[:N, :K]
    return q.to(torch.float8_e4m3fn).view(torch.uint8).contiguous(), s.contiguous()


def main(ref_root: Path) -> None:
    torch.set_num_threads(4)
    # ---- 1. byte table (tests/test_fp8.py:160-166) ----
    all_bytes = torch.arange(256, dtype=torch.uint8)
    cpu_all = all_bytes.view(torch.float8_e4m3fn).to(torch.float16)
    np.savez_compressed(HERE / "e4m3_table.npz", bytes=all_bytes.numpy(), fp16_bits=_u16(cpu_all))

    # ---- 2. dense reference + TP sharding (tests/test_attention_shapes.py:75-120) ----
    ref_mm, col, row, fuse = _functions_from(
        ref_root / "tests/test_attention_shapes.py",
        ["reference_matmul", "shard_col_parallel", "shard_row_parallel", "fuse_qkv_merged"])
    g = torch.Generator().manual_seed(0)
    dense = {}
    for tag, (M, N, K) in {"a": (16, 512, 512), "b": (5, 200, 384), "c": (1, 128, 1024)}.items():
        w = torch.randn(N, K, generator=g) * 0.02
        q8, s32 = quant_block(w)
        s16 = s32.to(torch.float16)
        x = torch.randn(M, K, generator=g).to(torch.float16)
        y16, wdq32 = ref_mm(x, q8, s16, 128, 128)
        dense[f"{tag}_x"] = _u16(x)
        dense[f"{tag}_w"] = q8.numpy()
        dense[f"{tag}_s16"] = _u16(s16)
        dense[f"{tag}_s32"] = s32.numpy()
        dense[f"{tag}_y16"] = _u16(y16)
        if tag == "b":
            # the reference's fp32 product of two halves is exact, so rounding it once gives the
            # FP16 dequantised weight; also record its torch path w.to(fp16) * scale.to(fp16)
            dense[f"{tag}_wdq16"] = _u16(wdq32.to(torch.float16))
            dense[f"{tag}_wdq_fp16path"] = _u16(q8.view(torch.float8_e4m3fn).to(torch.float16) *
                                                s16.repeat_interleave(128, 0).repeat_interleave(128, 1)[:N, :K])
    # TP=4 shards of case a (column- and row-parallel) and a fused 2-partition module
    q8 = torch.from_numpy(dense["a_w"]); s16 = torch.from_numpy(dense["a_s16"].view(np.float16).copy())
    for r in range(4):
        wc, sc = col(q8, s16, 4, r)
        wr, sr = row(q8, s16, 4, r)
        dense[f"a_col{r}_w"], dense[f"a_col{r}_s16"] = wc.numpy(), _u16(sc)
        dense[f"a_row{r}_w"], dense[f"a_row{r}_s16"] = wr.numpy(), _u16(sr)
    fw, fs = fuse([col(q8, s16, 4, 0)[0], col(q8, s16, 4, 2)[0]], [col(q8, s16, 4, 0)[1], col(q8, s16, 4, 2)[1]])
    dense["a_fused_w"], dense["a_fused_s16"] = fw.numpy(), _u16(fs)
    np.savez_compressed(HERE / "dense_reference.npz", **dense)

    # ---- 3. compressed-tensors dequant (compressed_tensors_v100.py:231-270) ----
    (dq_ct,) = _functions_from(ref_root / "src/fp8_w8a16_sm70/compressed_tensors_v100.py", ["_dequant_ct_weight_to_fp16"])
    ct = {}
    N, K = 352, 384
    w = torch.randn(N, K, generator=g) * 0.05
    # block
    q8, s32 = quant_block(w)
    layer = types.SimpleNamespace(weight=types.SimpleNamespace(data=q8.view(torch.float8_e4m3fn)),
                                  weight_scale=types.SimpleNamespace(data=s32.to(torch.bfloat16)))
    ct["block_w"], ct["block_s_bf16_as_f32"] = q8.numpy(), s32.to(torch.bfloat16).float().numpy()
    ct["block_out"] = _u16(dq_ct(layer, "block", [128, 128]))
    # channel
    sc = (w.abs().amax(dim=1, keepdim=True) / 448.0)
    qc = (w / sc).to(torch.float8_e4m3fn)
    layer = types.SimpleNamespace(weight=types.SimpleNamespace(data=qc), weight_scale=types.SimpleNamespace(data=sc))
    ct["channel_w"], ct["channel_s"] = qc.view(torch.uint8).numpy(), sc.numpy()
    ct["channel_out"] = _u16(dq_ct(layer, "channel", None))
    # tensor, fused module with 3 logical shards
    widths = [128, 64, 160]
    st = torch.tensor([0.011, 0.023, 0.007])
    per_row = torch.repeat_interleave(st, torch.tensor(widths)).reshape(N, 1)
    qt = (w / per_row).to(torch.float8_e4m3fn)
    layer = types.SimpleNamespace(weight=types.SimpleNamespace(data=qt), weight_scale=st.clone(), logical_widths=widths)
    ct["tensor_w"], ct["tensor_s"], ct["tensor_widths"] = qt.view(torch.uint8).numpy(), st.numpy(), np.array(widths)
    ct["tensor_out"] = _u16(dq_ct(layer, "tensor", None))
    np.savez_compressed(HERE / "ct_dequant.npz", **ct)

    # ---- 4. MoE reference loop (tools/ct_fp8_mixed_moe_numtest_vllm021.sh:61-73) ----
    sh = (ref_root / "tools/ct_fp8_mixed_moe_numtest_vllm021.sh").read_text()
    start = sh.index("def ref_moe(")
    end = sh.index("def run_case(")
    (ref_moe,) = _functions_from(Path("ct_fp8_mixed_moe_numtest_vllm021.sh"), ["ref_moe"], text=sh[start:end])
    E, I, H, M, topk = 4, 176, 256, 6, 2
    s13 = torch.rand(E, 2 * I, 1, generator=g) * 0.02 + 0.01
    w13_q = (torch.randn(E, 2 * I, H, generator=g) * 0.1 / s13).to(torch.float8_e4m3fn)
    s2 = torch.rand(E, H, 1, generator=g) * 0.02 + 0.01
    w2_q = (torch.randn(E, H, I, generator=g) * 0.1 / s2).to(torch.float8_e4m3fn)
    w2_dq = (w2_q.to(torch.float32) * s2).to(torch.float16)          # the reference keeps w2 as FP16
    x = (torch.randn(M, H, generator=g) * 0.1).to(torch.float16)
    ids = torch.stack([torch.randperm(E, generator=g)[:topk] for _ in range(M)]).to(torch.int64)
    tw = (torch.rand(M, topk, generator=g) * 0.5 + 0.1).to(torch.float16)
    out = ref_moe(x, tw, ids, w13_q, s13.to(torch.float16), w2_dq, I)
    np.savez_compressed(HERE / "moe_reference.npz", x=_u16(x), topk_ids=ids.numpy(), topk_w=_u16(tw),
                        w13=w13_q.view(torch.uint8).numpy(), s13=_u16(s13.to(torch.float16)),
                        w2=w2_q.view(torch.uint8).numpy(), s2=s2.numpy(), w2_dq16=_u16(w2_dq), out_f32=out.numpy(),
                        dims=np.array([E, I, H, M, topk]))

    # ---- 5. backend selector decisions (turbomind_fp8_backend.py:259-300) ----
    spec = importlib.util.spec_from_file_location("ref_tb", ref_root / "src/fp8_w8a16_sm70/turbomind_fp8_backend.py")
    tb = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(tb)
    cases = [
        dict(strategy="BLOCK", weight_block_size=(128, 128), local_n=1024, local_k=2048, has_ops=True, mode="auto"),
        dict(strategy="BLOCK", weight_block_size=(128, 128), local_n=1024, local_k=2048, need_moe=True, has_ops=True, mode="auto"),
        dict(strategy="CHANNEL", weight_block_size=None, local_n=4096, local_k=1408, has_ops=True, mode="auto"),
        dict(strategy="TENSOR", weight_block_size=None, local_n=4096, local_k=4096, has_ops=True, mode="auto"),
        dict(strategy="BLOCK", weight_block_size=(128, 128), local_n=4096, local_k=64, has_ops=True, mode="auto"),
        dict(strategy="BLOCK", weight_block_size=(128, 128), local_n=1024, local_k=2048, has_ops=False, mode="auto"),
        dict(strategy="BLOCK", weight_block_size=(128, 128), local_n=1024, local_k=2048, has_ops=True, mode="ours"),
    ]
    import json
    rec = []
    for kw in cases:
        backend, _ = tb.select_backend(quiet=True, **kw)
        rec.append({"kwargs": {k: (list(v) if isinstance(v, tuple) else v) for k, v in kw.items()}, "reference_backend": backend})
    (HERE / "selector_cases.json").write_text(json.dumps(rec, indent=1))
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <path to a checkout of the reference project>")
    main(Path(sys.argv[1]))
