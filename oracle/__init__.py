"""CPU oracle for the routed-expert MoE / FP8 trunk GEMV path.

TEST INFRASTRUCTURE ONLY.  These numpy functions restate the reference's
arithmetic (each cites the reference file:line it follows) so that the CUDA
kernels can be checked against them.  Nothing in the shipped package imports
this directory; only the test-suite, the smoke check and the benchmark's CPU
baseline leg do, and there only as the checker / the timed CPU arm.

Parity status per module:
  fp4.py      pinned   -- bit-compared with the reference's own numpy module
                          (model/fp4.py) on committed fixtures.
  fp8.py      pinned   -- block-32 / E8M0 form bit-compared with the
                          reference's numpy module (model/fp8_ref.py); the
                          block-128 / fp32-scale form is the same code with a
                          different block and scale rule.
  affine.py   parity unpinned for matmul output bits (the arithmetic lives in
              MLX, which is not available); packing layout, dequant formula and
              rounding points are pinned by the reference's in-code known
              answers.
  router.py   parity unpinned beyond the reference's tie rules and formulas
              (MLX / Metal only).
  mxfp4.py    parity unpinned beyond the reference's rounding table
              (MLX only).
  prefill.py  parity unpinned beyond the reference's ordering rules.
"""
