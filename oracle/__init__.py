"""CPU restatement of the reference's attention path.  TEST INFRASTRUCTURE ONLY.

Nothing under the product package may import this package: it is the checker
for the CUDA path (tests/, the smoke run, and the CPU-baseline leg of bench.py),
never the thing that is measured or shipped.

What it restates (files of ChandlerGuan/mercury_artifact):
  * the out/LSE merge of utils/flash_attn_dsl.py:31-71 and the packed merge :293-305
  * the per-rank ring protocol emitted by mercury/backend/pytorch/codegen.py:443-494
    (single ring), :480-491 (double ring) and :99-190 (backward accumulators with the
    write-back hop), with the index helpers of mercury/backend/pytorch/utils.py:41-106,171-192
  * the block attention forward/backward that the generated code calls.  That math lives in
    the third-party flash-attn wheel (setup.py:16, ">=2.7.0", not vendored in the reference),
    so it is restated from the published algorithm: softmax(scale * q k^T) v with the natural
    log-sum-exp of the scaled scores, and its analytic gradient.

Pinning: tests/golden/*.npz were produced by running the reference's own compiler and
generated code (imported from the reference checkout) on CPU/gloo; tests/test_oracle_golden.py
checks this restatement against them.  The reference holds no stored golden vectors of its own.
Causal ring schedules have no reference behaviour at all (the reference forwards `causal`
unchanged to every block, which is only right for causal=False): for them parity is UNPINNED
and the check is against single-device fp32 attention.
"""
