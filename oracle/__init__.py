"""CPU oracle of the sparse feature-transformer hot path.

TEST INFRASTRUCTURE ONLY.  Nothing under this directory is part of the
product: only tests/, `__graft_entry__.smoke()` and the CPU-baseline /
`--impl reference` legs of bench.py may import it, and there only as the
checker.  The product package never imports it and has no CPU path.

Parity status: pinned.  Every function here is checked (tests/test_oracle_*)
against fixtures under tests/golden/ that were produced by importing the
reference project's own Python code (tests/golden/make_golden.py).
"""
