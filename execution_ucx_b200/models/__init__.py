"""Flagship workloads: the named benchmark configurations as reusable classes."""
