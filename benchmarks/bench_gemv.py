#!/usr/bin/env python
"""GEMV kernel benchmark (ezops benchmarks/bench_gemv.py): ``-h`` lists backends, ``-k <backends>`` selects them."""

from _per_op import main

if __name__ == "__main__":
    main("gemv", "gemv", "GEMV kernel benchmark (ezops benchmarks/bench_gemv.py)")
