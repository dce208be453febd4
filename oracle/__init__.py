"""CPU oracle for the attention hot path -- TEST INFRASTRUCTURE, not product code.

Only the test suite, the smoke check and the benchmark's CPU-baseline leg may
import this package.  The shipped path (``machinelearning_b200``) never does: it
runs on the CUDA library or raises.

Parity status: PINNED.  ``attention_f64`` is checked against golden vectors that
were produced by importing the reference's own float64 brute force
(``nanolab/csrc/flash_attn_sim.py:193-212`` differentiated by autograd) and its
sliding-window definitions (``nanolab/mixers.py:96-135``, ``:168-200``); the
generating script and the vectors live in ``tests/golden``.  ``build_ref`` compiles the
reference's own CUDA kernel into ``oracle/_ref/`` as a second checker on the GPU.
"""
