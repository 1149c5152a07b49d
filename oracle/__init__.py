"""CPU oracle for the Qwen3-0.6B greedy prefill+decode path.

TEST INFRASTRUCTURE ONLY.  Nothing under this directory is part of the
product: only the tests, the smoke check and the benchmark's CPU-baseline /
reference arm may import it, and only as the checker or the timed baseline.
"""
