"""CPU oracle for the trellis codec: TEST INFRASTRUCTURE, not a product path.

Only the test-suite, the smoke check and the benchmark's CPU-baseline / reference
legs may import this package.
"""
