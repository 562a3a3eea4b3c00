"""Timing, tracing, checkpoint and clock-sampling helpers."""
