"""Stand-in for the ``nki`` package, used only by ``tests/golden/make_golden.py``: the reference's CPU
goldens import ``nki.language`` for dtype names and nothing else."""
