"""Benchmark programs (run with `python -m ...benchmarks.<name>` under torchrun)."""
