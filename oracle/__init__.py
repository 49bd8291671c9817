"""CPU oracle for the Lumen decode path — TEST INFRASTRUCTURE, parity unpinned.

Only the test-suite, the GPU smoke test and the benchmark's CPU-baseline leg may import this
package.  The product package never does.
"""
