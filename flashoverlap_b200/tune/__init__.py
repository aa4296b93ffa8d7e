"""Tuner: GEMM tile profiling, bandwidth curves, tile-order hints, exhaustive
and predictive search (reference: tune/*.py)."""
