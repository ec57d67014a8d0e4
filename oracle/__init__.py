"""CPU oracle for the Tucker-MoE layer forward.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
directory; it is used by the tests, by the smoke check and by the CPU-baseline
leg of the benchmark, always as the checker and never as the product path.
"""
