"""CPU oracle for the quantized-Linear hot path of fms-model-optimizer.

TEST INFRASTRUCTURE ONLY.  Nothing under ``oracle/`` is part of the product: only ``tests/``,
``__graft_entry__.smoke()`` and the CPU-baseline / reference legs of ``bench.py`` may import it, and
only as the checker or as the timed CPU baseline.  The product package
(``fms_model_optimizer_b200``) never imports it and has no CPU path of its own.

Every function restates, in plain PyTorch CPU / numpy arithmetic, one piece of the reference and
cites the file and lines it follows (paths relative to the fms-model-optimizer source tree).  The
reference is itself eager PyTorch, so its rounding behaviour (round-half-to-even ``torch.round``,
fp32 division, ``float8_e4m3fn`` casts, bf16 / fp16 intermediate rounding) is reproduced by calling
the same ATen CPU operators in the same order.

Pinning.  ``tests/golden/make_golden.py`` ran the reference itself (imported from its source tree)
on small seeded inputs and stored its outputs under ``tests/golden/``; ``tests/test_oracle_golden.py``
checks every oracle function against those files and against the six W8A8 golden vectors of the
reference's own test-suite (``tests/artifacts/aiu_addons/ref_*.pt``, stored as
``tests/golden/aiu_i8i8_vectors.pt``).  Two pieces have no reference run behind them because the
reference implements them only as Triton GPU kernels: the chunk-truncated integer GEMM
(``imatmul_kernel``) and the float GEMM (``matmul_kernel``).  The integer one is pinned indirectly
against the reference's own PyTorch emulation of the same arithmetic
(``QLinearINT8Deploy.iaddmm_int``); the float one is "parity unpinned" beyond the properties the
reference's tests state (relative error against a plain matmul).
"""
