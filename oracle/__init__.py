"""TEST INFRASTRUCTURE ONLY - CPU restatement of the reference's operators.

Nothing under this package is part of the product path.  It may be imported by
``tests/``, by ``__graft_entry__.smoke()`` and by the CPU-baseline legs of ``bench.py``,
as the checker or as the timed CPU baseline - never by ``flextensor_b200``.
"""
