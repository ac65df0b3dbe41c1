"""CPU oracle for the block-scaled FP8 (E4M3) W8A16 linear / MoE path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
directory.  The only callers are the parity tests, the smoke check and the
CPU-baseline leg of the benchmark, and there it is the checker, never the
thing that is measured or shipped.

Each function restates, on the CPU, what the reference project
(KumphanartDansiri/vllm-fp8-w8a16-sm70) defines as the correct result and
cites the reference file:line it follows.  Pinning: the restatement is
checked against the reference's own known-answer vectors (the 14-byte edge
table and the exhaustive 256-byte sweep of ``tests/test_fp8.py:119-179``)
and against fixtures produced by executing the reference's own Python
helpers (``tests/golden/make_golden.py``).  MoE routing from router logits
is NOT pinned by the reference (it consumes ``topk_ids`` produced by vLLM
and never computes them in its own tests); ``oracle.moe.route_topk`` states
the rule this build fixes and says "parity unpinned" for that one function.
"""

from . import e4m3, dequant, linear, moe, tp  # noqa: F401
