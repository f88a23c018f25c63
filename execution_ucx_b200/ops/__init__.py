"""Data-plane kernels (sm_100a) as Python ops."""
