"""Workloads and helpers of bench.py (measurement code: not part of the tscale_b200 package, which holds only the path)."""
