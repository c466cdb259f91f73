"""CPU oracle for the Based hot path (TEST INFRASTRUCTURE, not product code).

Only the tests, the smoke check and the CPU-baseline leg of the benchmark may
import this package.  Nothing under ``based_b200`` imports it: the product path
is the CUDA library and fails loudly when that library is missing.
"""
