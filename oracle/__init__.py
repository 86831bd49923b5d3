"""CPU oracle for the quantized lm_head + fused sampler path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
directory: it is the checker used by ``tests/``, by ``__graft_entry__.smoke``
and by the ``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``.

Every function restates, in numpy (torch-CPU only where a torch dtype cast is
the arithmetic being pinned), one piece of the reference plugin
``himikk/vllm-quant-kernels`` and cites the reference ``file:line`` it follows.

Parity pin: the restatements are checked in ``tests/test_oracle_golden.py``
against vectors produced by running the reference's own Python code on CPU
(its torch quantizers directly, its Triton kernels under ``TRITON_INTERPRET=1``);
the generating script is ``tests/golden/make_golden.py``.  ``tl.dot_scaled``
does not run in the Triton interpreter, so the MXFP8 / MXFP4 *logits* are
pinned through the reference's quantizers plus the dequantise-then-matmul
reference in its tests (``tests/test_mxfp4_kernel.py:57-77``), not through its
kernels.
"""

from . import quant, lm_head, sampler  # noqa: F401
