"""Harness that drives the unmodified reference implementation (installed under ``baseline/_ref``)."""
