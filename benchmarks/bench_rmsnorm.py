#!/usr/bin/env python
"""RMSNorm kernel benchmark (ezops benchmarks/bench_rmsnorm.py): ``-h`` lists backends, ``-k <backends>`` selects them."""

from _per_op import main

if __name__ == "__main__":
    main("rmsnorm", "rmsnorm", "RMSNorm kernel benchmark (ezops benchmarks/bench_rmsnorm.py)")
