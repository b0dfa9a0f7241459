"""Test infrastructure only: CPU restatement of the reference's torch
implementation of the Qwen3 dense-decode path.  Nothing in the shipped package
imports this directory; only tests, the smoke check and the CPU-baseline /
reference legs of the benchmark do, and there only as the checker or as the
CPU arm being timed."""
