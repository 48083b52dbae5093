"""CPU restatement of the reference's paged-attention semantics.

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, ``__graft_entry__.smoke()``
and the CPU-baseline / reference legs of ``bench.py`` as the checker or the
timed CPU baseline; the product package never imports it.
"""
