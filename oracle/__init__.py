"""CPU oracle for the attention path. TEST INFRASTRUCTURE ONLY.

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
import this package. The shipped library (``ember_b200``) never does.
"""
