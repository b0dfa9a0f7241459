#!/usr/bin/env python
"""Device-side timeline of the tensor-parallel batch-1 decode layer (one persistent kernel per rank, both sums over
ranks inside it).  Launch one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        benchmarks/tp_layer_timeline.py [--layers 6] [--seq-len 4096]

Every rank replays a CUDA graph of ``--layers`` layer calls over rotating weight sets; rank 0 records, per CTA and
phase of the kernel, %globaltimer at the start of the phase, when its activations are staged, when its first weight
(or K/V) stage has landed and at its end (``ezb_trace_enable``), and prints min / median / max over the CTAs in
microseconds since the first record, for two layers in the middle of the graph.  Phases: qkv, attn (the slice of a
kv head a CTA streams, then the fold by the last CTA of the head; ``attn_d`` = q ready | V landed | P.V done |
record + ticket), oproj (ends after the gather of the CTA's own rows), gateup, down, final (gather of the second sum).
"""

from __future__ import annotations

import argparse
import os
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--layers", type=int, default=6)
    ap.add_argument("--seq-len", type=int, default=4096)
    args = ap.parse_args()

    from ezops_b200 import _lib, tp as tpm, workloads as wl

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    lib, dev = _lib.load(), torch.device("cuda")
    sh, B, S, NL = wl.QWEN3_8B, 1, args.seq_len, args.layers
    hidden, K0, V0, Wqkv, Wo, Wgu, Wd = wl.decode_layer_inputs(sh, B, S)
    heads = (sh.num_heads, sh.num_kv_heads, sh.head_dim)
    lay = tpm.TensorParallelDecodeLayer(B, S, sh.hidden, sh.inter, sh.num_heads, sh.head_dim, sh.num_kv_heads, exchange="fused")
    sets = []
    for _ in range(3):
        shards = tuple(t.cuda().clone() for t in tpm.shard_layer_weights(Wqkv, Wo, Wgu, Wd, *heads, world, rank))
        sets.append((tpm.shard_kv_cache(K0, world, rank).cuda(), tpm.shard_kv_cache(V0, world, rank).cuda()) + shards)
    hid, out = hidden.cuda(), torch.empty(B, sh.hidden, dtype=torch.bfloat16, device=dev)
    _lib.set_tuning(pdl_across_calls=1)

    def run():
        for i in range(NL):
            lay(hid, *sets[i % len(sets)], out=out)

    side = torch.cuda.Stream()
    cap = NL * 148 * 9 + 100
    rec = torch.zeros(cap * 6, dtype=torch.int64, device=dev)
    cur = torch.zeros(1, dtype=torch.int32, device=dev)
    with torch.cuda.stream(side):
        run()
        run()
        torch.cuda.synchronize()
        dist.barrier()
        if rank == 0:
            lib.ezb_trace_enable(rec.data_ptr(), cur.data_ptr(), cap)  # kernel parameters are fixed at capture
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            run()
    for _ in range(2):
        torch.cuda.synchronize()
        dist.barrier()
        cur.zero_()
        torch.cuda.synchronize()
        dist.barrier()
        graph.replay()
    torch.cuda.synchronize()
    dist.barrier()
    if rank == 0:
        lib.ezb_trace_enable(None, None, 0)
        n = int(cur.item())
        r = rec.cpu().numpy().reshape(-1, 6)[:min(n, cap)]
        print(f"world {world}: {n} records, device status {_lib.device_status()}")
        t0 = r[:, 2].min()
        names = {20: "qkv", 21: "attn", 25: "attn_d", 22: "oproj", 23: "gateup", 24: "down", 26: "final"}
        for kid, name in names.items():
            a = r[r[:, 0] == kid]
            a = a[np.argsort(a[:, 2])]
            per = len(a) // NL
            if per == 0:
                continue
            for L in (NL // 2 - 1, NL // 2):
                blk = a[L * per:(L + 1) * per]

                def stat(col):
                    v = (blk[:, col][blk[:, col] > 0] - t0) / 1e3
                    return (v.min(), float(np.median(v)), v.max()) if len(v) else (-1.0, -1.0, -1.0)

                print(f"layer {L} {name:7s} ctas {per:4d} | start %7.2f %7.2f %7.2f | staged %7.2f %7.2f %7.2f | first stage %7.2f %7.2f %7.2f | end %7.2f %7.2f %7.2f"
                      % (stat(2) + stat(3) + stat(4) + stat(5)))
    torch.cuda.synchronize()
    dist.barrier()
    lay.close()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
