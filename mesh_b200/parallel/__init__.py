"""TP / SP / DP / EP / CP / PP layer library and placement helpers."""
