"""CPU oracle for the ragged attention path.  TEST INFRASTRUCTURE ONLY.

Nothing in the product package may import this; only ``tests/``, the smoke
check and the CPU-baseline / reference legs of ``bench.py`` do, and there only
as the checker or the timed CPU baseline.  Each function restates, in plain
PyTorch-eager / numpy code, what the reference (w4096/mini-vllm) computes and
cites the reference file:line it follows.

Pin status
----------
* packing, RoPE, block manager, scheduler, model wiring: pinned against
  outputs of the reference's own code (``tests/golden/make_golden.py`` imports
  it and commits the vectors).
* KV-cache write: the reference kernel is Triton (GPU only); restated from
  ``minivllm/models/layers/attention.py:13-33``, a pure copy.
* attention arithmetic: lives in the third-party ``mini_flash_attention``
  package (``requirements.txt:7``, unpinned git HEAD, not vendored, absent
  here) and the reference has no test or golden vector for it, so this part is
  **parity unpinned**: the oracle is the published softmax(QK^T * scale)V
  definition over keys gathered through the block table, in fp32.
"""
