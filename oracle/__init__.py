"""CPU oracle for the contextual-sparsity MLP path — TEST INFRASTRUCTURE ONLY.

Nothing under ``oracle/`` is product code: the package ``sparse_transformers_b200`` never
imports it.  Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline / reference
legs of ``bench.py`` may use it, and there only as the checker or the timed CPU baseline.
"""
