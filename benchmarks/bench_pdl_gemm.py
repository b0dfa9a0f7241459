#!/usr/bin/env python
"""Chained GEMMs with and without programmatic dependent launch (ezops benchmarks/bench_pdl_gemm.py): ``-h`` lists backends, ``-k <backends>`` selects them."""

from _per_op import main

if __name__ == "__main__":
    main("pdl_gemm", "pdl_gemm", "Chained GEMMs with and without programmatic dependent launch (ezops benchmarks/bench_pdl_gemm.py)")
