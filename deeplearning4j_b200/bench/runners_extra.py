"""Runners for the remaining baseline configurations (filled in as the model families land)."""
TABLE = {}
