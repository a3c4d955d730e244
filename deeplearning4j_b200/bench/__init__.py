"""Benchmark runners for the five baseline configurations (used by the repository-level bench.py)."""
