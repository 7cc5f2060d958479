"""Test infrastructure: CPU oracles for the hot path.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` may
import this package.  The product package never does.
"""
