"""CPU oracle for the QVB8 / QVB8R decode-in-matmul path -- TEST INFRASTRUCTURE ONLY.

A plain-C restatement (``qvb8_oracle.c``) of the reference's pack decoders with
numpy wrappers.  Only the test-suite, the smoke check and the CPU-baseline leg
of the benchmark may import this package; the shipped library never does.

Parity pin: the reference ships no tests or golden vectors for this path, so
the oracle is pinned against the reference's own Python / C++ decoders run on
seeded packs (``tests/golden``, produced by ``tests/golden/make_golden.py``).
"""
from .oracle import *  # noqa: F401,F403
