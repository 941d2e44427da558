"""Micro-benchmarks on the shapes the reference benchmarks (megablocks/ops/*_benchmark.py).

Each module is runnable: ``python -m megablocks_b200.benchmarks.<name>``.
"""
