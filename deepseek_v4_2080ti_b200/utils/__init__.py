"""Timing, clock sampling and NVTX helpers."""
