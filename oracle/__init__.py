"""CPU oracle for the SquareQ weight-streaming path.

Test infrastructure: only ``tests/``, the smoke check and the benchmark's CPU
baseline / reference legs import this package, and only as the checker or as
the timed CPU baseline.  The product (``stagehand_b200``) never does.
"""
