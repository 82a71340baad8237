"""CPU oracle for the fused-MoE path.  TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package may import this: it exists so that the tests,
the smoke check and the benchmark's CPU-baseline leg have an independent
restatement of what the reference computes.

Pinning status
--------------
* Routing conversion (``oracle.routing.topk_to_routing``): pinned against the
  reference's own ``_standard_topk_to_triton_kernels``
  (src/flaggems_sglang/ops/fused_moe.py:103-130) run on CPU; the vectors are
  committed under ``tests/golden/`` with the script that made them.
* Block alignment (``oracle.routing.moe_align_block_size``): the reference has
  no such function; pinned against the worked example in the ecosystem's
  documented contract and against a brute-force stable sort.
* bf16 forward (``oracle.moe.fused_experts``): pinned against outputs of the
  reference's Triton op recorded on a B200 when those fixtures exist under
  ``tests/golden/``; otherwise "parity unpinned".
* FP8 block-quant and int4 AWQ forwards: the reference rejects these modes
  (fused_moe.py:154-169), so no reference output can exist: "parity unpinned".
"""
