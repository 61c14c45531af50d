"""CPU oracle of the l4-parakeet-rs encoder / decoder hot path.

TEST INFRASTRUCTURE ONLY: imported by tests/, the smoke check and the CPU-baseline
legs of the benchmark.  Nothing under l4-parakeet-rs_b200/ may import it.
"""
