"""Seeded synthetic KV and the benchmark configurations built from it.

Input generators for ``bench.py``, ``__graft_entry__.smoke()`` and the tests;
nothing in ``fragpack_b200`` imports this package.
"""
