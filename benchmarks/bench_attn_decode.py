#!/usr/bin/env python
"""Decode attention benchmark (ezops benchmarks/bench_attn_decode.py): ``-h`` lists backends, ``-k <backends>`` selects them."""

from _per_op import main

if __name__ == "__main__":
    main("attn_decode", "attn", "Decode attention benchmark (ezops benchmarks/bench_attn_decode.py)")
