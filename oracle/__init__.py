"""CPU oracle for the fast-weight recurrences: test infrastructure only.

Nothing in the shipped library imports this package.  It is used by the tests, by the smoke
check and by the benchmark's CPU-baseline leg as the checker / the timed baseline.
"""
