"""CPU oracle for the SparseDrop hot path.  TEST INFRASTRUCTURE ONLY.

Nothing in the product (the ``flash_dropout`` package, the C ABI) imports this package.  It is
used by ``tests/``, by ``__graft_entry__.smoke()`` as the checker, and by ``bench.py`` for the
``cpu_baseline`` leg / ``--impl reference`` arm, where it is the thing timed on the host cores.
"""
