"""Command-line tools: `python -m luatorch_b200.tools.benchmark` (kernel micro-benchmarks)."""
