"""CPU oracle for the int8 quantized-linear path -- test infrastructure only.

Only the tests, the smoke check and the benchmark's CPU-baseline leg import
this package; the product library never does.
"""
