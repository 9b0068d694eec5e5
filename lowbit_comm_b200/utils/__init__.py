"""Benchmark and diagnostics helpers (timing, result schema, gates, roofline, tracing)."""
