"""Harness that runs the unmodified reference (installed under baseline/_ref) for comparison numbers."""
