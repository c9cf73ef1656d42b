"""CPU oracle for the LLVQ archive-code dequant-GEMV path (test infrastructure only).

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this
package. The shipped library never does.
"""
