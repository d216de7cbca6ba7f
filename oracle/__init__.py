"""CPU oracle for the GQA decode-attention path.

TEST INFRASTRUCTURE ONLY.  Nothing under this directory is part of the shipped
library: it is imported by the test-suite, by the smoke check and by the CPU
baseline leg of the benchmark, always as the checker and never as the thing
that is measured or shipped.
"""
