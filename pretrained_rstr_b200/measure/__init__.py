"""Measurement code: what ``bench.py`` (beside the package) times and how, the workloads it
runs, and the small single-kernel workloads that profiler captures are taken from."""
