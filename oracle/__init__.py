"""CPU oracle for the sparse top-k global-attention path.  TEST INFRASTRUCTURE ONLY.

Nothing in the product package imports this directory; only the test-suite, the smoke check
and the CPU-baseline legs of the benchmark do, and only as the checker / the timed CPU arm.
"""
