"""CPU oracle for the ragged paged-attention path.  TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Imported only by ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of
``bench.py``.  The shipped package ``easymlx_b200`` never imports it.
"""
