"""Timing, clock sampling and roofline helpers."""
