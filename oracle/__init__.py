"""CPU oracle for the Qwen3.5 decoder hot path (MoE block, paged attention, gated delta net).

TEST INFRASTRUCTURE ONLY.  These modules restate, in plain torch on the CPU, the reference's own
Python/torch golden implementations (each function cites the reference file:line it follows).
They exist to check the CUDA kernels and to be timed as the CPU baseline.  Nothing in the product
package may import them: only the tests, the smoke check and the benchmark's CPU-baseline legs do.

Parity status: PINNED.  The codecs, the router, the causal conv, the GDN recurrence and the whole
GDN sublayer are checked against outputs of the reference's own functions (imported from the
reference checkout with the NPU DSL stubbed out, see tests/golden/make_golden.py) stored under
tests/golden/.  Goldens that the reference only has inline inside a check function (routed
experts, slots, combine, paged decode) are restated from those lines and cross-checked against
independent float64 formulations.
"""
from . import codecs, moe, attention, gdn, stack, speculative  # noqa: F401
