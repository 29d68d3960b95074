"""CPU restatement of the reference algorithms (TEST INFRASTRUCTURE ONLY).

Nothing in the shipped package may import this directory.  It exists so the
tests, the smoke check and the CPU-baseline leg of the benchmark can compare
the CUDA path against an independent statement of what the reference computes:

* ``fp8_gemm``  - dequantise-and-matmul FP8 block-scaled GEMM
                  (reference: scripts/problems/gemm/reference.py:40-85)
* ``moe``       - DeepSeek-style MoE layer, end to end and stage by stage
                  (reference: scripts/problems/moe/reference.py:10-142,
                  src/moe/moe_topk_kernel.cpp:15-251,
                  tests/moe/moe_topk_test.cpp:198-351)

Parity pin: both modules are checked against outputs of the reference's own
PyTorch ``ref_kernel`` functions (imported unmodified, run on CPU) stored as
fixtures under ``tests/golden/`` together with the script that made them.
"""
