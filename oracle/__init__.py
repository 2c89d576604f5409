"""CPU restatement of the reference's decode-time research-attention path.

TEST INFRASTRUCTURE ONLY.  Nothing under this package is part of the product:
it is imported by `tests/`, by `__graft_entry__.smoke()` as the checker and by
`bench.py` for the timed CPU baseline.  The product (`sparse_attention_hub`)
never imports it and has no CPU path of its own.

Every function restates, in numpy, one function of
skylight-org/sparse-attention-hub and cites it by file:line.  Where the
reference leaves a floating-point summation order or a tie order to its tensor
library, the restatement fixes one (stated in the function's docstring) and the
CUDA kernels follow the same one, so that integer results (index sets, hash
and LSH codes) can be compared bit for bit.  The restatement is pinned against
outputs of the reference itself: `tests/golden/make_golden.py` imports the
reference, runs it on seeded inputs and stores its outputs as fixtures;
`tests/test_oracle_golden.py` checks this package against them.
"""

from . import attention, bf16, hashattention, mask_ops, qk, stacks, topk  # noqa: F401
