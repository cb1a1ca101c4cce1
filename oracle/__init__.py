"""CPU restatement of CommunityKV's sparse-decode hot path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package may import this
directory: it is used by the tests, by the smoke check and by the CPU-baseline
leg of the benchmark as the checker / the timed CPU arm, never as a product
code path.

Parity pin: every function here is checked in ``tests/test_oracle_golden.py``
against (a) the known answers held by the reference's own unit tests and
(b) fixtures under ``tests/golden/`` that were produced by importing the
reference package and its test helpers (see ``tests/golden/make_golden.py``).
"""
