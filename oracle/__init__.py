"""CPU oracle for the quantised-GEMM path.  TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package may import this: only tests/, the smoke check
and the benchmark's CPU-baseline leg use it, and only as the checker.
"""
