"""CPU restatement of the reference's routed-expert hot path.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this; only
``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py``
do, and there only as the checker or the timed CPU baseline.
"""
