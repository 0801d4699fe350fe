"""Shared pieces of the benchmark scripts: the timer, the result document and its provenance
block, and the operator case tables."""
