"""Timing, clock sampling and logging helpers."""
