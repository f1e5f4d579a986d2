"""CPU oracle (numpy + a little C) for the 4-bit dequant-GEMV path.

Test infrastructure only: imported by tests/, the smoke check and the
benchmark's CPU-baseline leg; never by the product package.
"""
