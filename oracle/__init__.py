"""CPU oracle for the v2x2ssd hot path -- TEST INFRASTRUCTURE ONLY.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline / reference
legs of ``bench.py`` may import this package.  The shipped library
(``slinoss_b200``) never does.
"""
