"""The torch.library registrations: schema, fake (shape-only) implementations under FakeTensorMode, and that the hooks
trace through them without a graph break.  No kernel runs here."""
import types

import pytest
import torch


def test_ops_are_registered_with_schemas(lib):
    from vllm_fp8_w8a16_sm70_b200 import custom_ops  # noqa: F401
    lin = torch.ops.fp8w8a16_b200.linear.default
    moe = torch.ops.fp8w8a16_b200.moe_forward.default
    assert "Tensor x" in str(lin._schema) and "block_h" in str(lin._schema)
    assert "Tensor? expert_map" in str(moe._schema)


def test_fake_implementations_give_shapes(lib):
    from torch._subclasses.fake_tensor import FakeTensorMode
    from vllm_fp8_w8a16_sm70_b200 import custom_ops
    with FakeTensorMode():
        x = torch.empty(5, 256, dtype=torch.float16)
        w = torch.empty(384, 256, dtype=torch.uint8)
        s = torch.empty(3, 2, dtype=torch.float16)
        y = custom_ops.linear(x, w, s, 384, 256, 128, 128)
        assert tuple(y.shape) == (5, 384) and y.dtype == torch.float16
        w13 = torch.empty(4, 256, 256, dtype=torch.uint8)
        w2 = torch.empty(4, 256, 128, dtype=torch.uint8)
        s13, s2 = torch.empty(4, 2, 2, dtype=torch.float16), torch.empty(4, 2, 1, dtype=torch.float16)
        out = custom_ops.moe_forward(x, torch.empty(5, 2), torch.empty(5, 2, dtype=torch.int32), w13, s13, w2, s2, 128, False, "silu", None)
        assert tuple(out.shape) == (5, 256)
        with pytest.raises(Exception):
            custom_ops.linear(torch.empty(5, 100, dtype=torch.float16), w, s, 384, 256, 128, 128)


def test_hook_traces_without_graph_break(lib):
    """Dynamo sees the linear hook as ONE graph with the registered op inside (backend that only records the graph)."""
    from vllm_fp8_w8a16_sm70_b200 import Fp8LinearMethod, custom_ops  # noqa: F401
    from torch._subclasses.fake_tensor import FakeTensorMode
    method = Fp8LinearMethod((128, 128))
    graphs = []

    def recorder(gm, example_inputs):
        graphs.append(gm)
        return gm.forward

    def fn(x, w, s):
        layer = types.SimpleNamespace(weight=w, weight_scale_inv=s, weight_block_size=[128, 128], input_size_per_partition=256,
                                      output_size_per_partition=384)
        return method.apply(layer, x) * 2

    torch._dynamo.reset()
    try:
        explain = torch._dynamo.explain(fn)(torch.zeros(5, 256, dtype=torch.float16, device="meta"),
                                            torch.zeros(384, 256, dtype=torch.uint8, device="meta"),
                                            torch.zeros(3, 2, dtype=torch.float16, device="meta"))
    finally:
        torch._dynamo.reset()
    assert explain.graph_break_count == 0, explain.break_reasons
    targets = [str(n.target) for g in explain.graphs for n in g.graph.nodes if n.op == "call_function"]
    assert any("fp8w8a16_b200.linear" in t for t in targets), targets
