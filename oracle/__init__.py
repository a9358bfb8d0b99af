"""TEST INFRASTRUCTURE: CPU restatement of the reference's sparse-attention path.

Nothing in the shipped package imports this; it exists so that tests, the smoke
check and the benchmark's CPU-baseline leg can check and time the algorithm.
"""
