"""CPU oracle for the MoE-layer forward path. TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package imports this directory. Only the tests, the
smoke entry and the CPU-baseline leg of the benchmark may use it, and there
only as the checker / timed baseline, never as the product path.
"""
