#!/usr/bin/env python
"""Fused o_proj + FFN benchmark (ezops benchmarks/bench_fused_o_proj_ffn.py): ``-h`` lists backends, ``-k <backends>`` selects them."""

from _per_op import main

if __name__ == "__main__":
    main("fused_o_proj_ffn", "ffn", "Fused o_proj + FFN benchmark (ezops benchmarks/bench_fused_o_proj_ffn.py)")
