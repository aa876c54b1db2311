"""CPU oracle for the Linear path: test infrastructure, never the product path.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs import
this package.
"""
