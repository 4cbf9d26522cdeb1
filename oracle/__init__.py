"""CPU oracle of the SLAYER hot path -- test infrastructure, not product code.

Only ``tests/``, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` /
``--impl reference`` legs of ``bench.py`` may import this package.
"""
