"""CPU oracle for the GGUF-block quantized-matmul path.  TEST INFRASTRUCTURE ONLY.

Only the tests, the smoke check and the CPU-baseline / reference legs of the
benchmark may import this package; the shipped library never does.

Parity is UNPINNED: the upstream project has no implementation, test or golden
vector for Q8_0 / Q8_1 / Q4_K / Q6_K blocks (gpu-core/tests/suite/
prove_quantized.rs:15-20 lists them as backlog), so this restatement is checked
only against itself in two independent forms (C in ``qmm_oracle.c``, numpy in
``npref.py``) and against hand-built known-answer blocks.
"""
from .cref import *  # noqa: F401,F403
