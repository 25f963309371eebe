"""TEST INFRASTRUCTURE ONLY — the CPU oracle for the flash-attention path.

Nothing under ``oracle/`` may be imported by the product package
(``torch_mojo_backend_b200``).  Only ``tests/``, ``__graft_entry__.smoke()`` and the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` use it, and only as the checker
or as the timed CPU baseline.
"""
