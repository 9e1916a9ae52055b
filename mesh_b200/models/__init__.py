"""Example / benchmark models."""
