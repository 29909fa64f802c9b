"""CPU oracle for the gated-MLP hot path. TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package imports this directory. It may be imported only by
tests/, by __graft_entry__.smoke() and by bench.py's cpu_baseline / reference
arm, and there only as the checker or the timed CPU baseline.
"""
