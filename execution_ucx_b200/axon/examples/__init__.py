"""Runnable examples of the Python API (``python -m execution_ucx_b200.axon.examples.<name>``)."""
