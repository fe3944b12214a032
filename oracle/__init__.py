"""CPU oracle for the five hot-path kernels.  TEST INFRASTRUCTURE ONLY: imported by tests/,
__graft_entry__.smoke() and bench.py's CPU-baseline legs; never by the product package."""
