#!/usr/bin/env python
"""Fused Qwen3 dense decode layer benchmark (ezops benchmarks/bench_qwen3_dense_decode.py): ``-h`` lists backends, ``-k <backends>`` selects them."""

from _per_op import main

if __name__ == "__main__":
    main("qwen3_dense_decode", "layer", "Fused Qwen3 dense decode layer benchmark (ezops benchmarks/bench_qwen3_dense_decode.py)")
