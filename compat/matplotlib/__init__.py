"""Minimal stand-in for matplotlib, which the reference's bench.py imports (bench.py:4) for its
error heat map (bench.py:105-116) and which is not installed in this image.  Only used when this
directory is put on PYTHONPATH to run the reference's harness unchanged."""
