"""Worked example: a new compression algorithm from DSL source to training."""
