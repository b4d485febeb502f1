"""Utilities: checkpoints, metrics, timing / roofline, watchdog."""
