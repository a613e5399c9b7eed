"""TEST INFRASTRUCTURE: CPU restatements of the reference algorithm.

Nothing in the shipped package imports this directory.  It is loaded only by
the tests, by the smoke check and by the CPU-baseline / reference arm of the
benchmark, and there only as the checker or as the timed CPU baseline.
"""
