"""CPU oracle for the sparse entmax attention hot path.

TEST INFRASTRUCTURE ONLY.  Nothing under this package is part of the product:
only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
import it, and only as the checker.  The shipped path is the CUDA library.
"""
