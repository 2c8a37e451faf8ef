"""Test-only CPU checkers.  Nothing under xsched_b200/ may import this package."""
