#!/usr/bin/env python
"""Fused q/k-norm + RoPE + cache write benchmark (ezops benchmarks/bench_fused_qk_norm_rope.py): ``-h`` lists backends, ``-k <backends>`` selects them."""

from _per_op import main

if __name__ == "__main__":
    main("fused_qk_norm_rope", "rope", "Fused q/k-norm + RoPE + cache write benchmark (ezops benchmarks/bench_fused_qk_norm_rope.py)")
