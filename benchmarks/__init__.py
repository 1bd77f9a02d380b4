"""Benchmark scripts of moonep_b200 (run as files; this package marker lets bench.py import the reference arm)."""
