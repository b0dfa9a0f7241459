"""One rank of the multi-GPU check of the tensor-parallel decode layer (launched by
tests/test_tp_multi_gpu.py through torch.distributed.run, one process per GPU).

Every rank runs the layer with the exchange fused into the kernels and with NCCL in between the
three parts; rank 0 compares both with the CPU oracle on the unsharded weights.  Prints one line
per case and exits 0 when every check held.
"""

import os
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from ezops_b200 import _lib, tp as tpm, workloads as wl  # noqa: E402
from oracle import ezops_oracle as orc  # noqa: E402


def main() -> int:
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ok = True
    # batch 1: the rank-local layer and both exchanges in one persistent kernel (and, with that switched off, in the
    # small-batch kernels); batch 3: gather and push inside the small-batch kernel; batch 16: row kernel + tensor-core
    # kernel; the last case is the benchmark's tensor-parallel configuration (Qwen3-32B shapes, batch 64) at a shorter cache
    for sh, B, S in [(wl.QWEN3_VL_2B, 1, 700), (wl.QWEN3_8B, 1, 2100), (wl.QWEN3_8B, 3, 1025), (wl.QWEN3_VL_2B, 16, 400),
                     (wl.QWEN3_32B, 64, 1536)]:
        hidden, K0, V0, Wqkv, Wo, Wgu, Wd = wl.decode_layer_inputs(sh, B, S)
        heads = (sh.num_heads, sh.num_kv_heads, sh.head_dim)
        ref = (orc.qwen3_dense_decode_ref(hidden, K0.clone(), V0.clone(), Wqkv, Wo, Wgu, Wd, *heads, lean_attention=B >= 32)
               if rank == 0 else None)
        args = (B, S, sh.hidden, sh.inter, sh.num_heads, sh.head_dim, sh.num_kv_heads)
        nccl = tpm.TensorParallelDecodeLayer(*args)
        fused = tpm.TensorParallelDecodeLayer(*args, exchange="fused")
        peer = tpm.TensorParallelDecodeLayer(*args, exchange="peer")  # the three parts with the library's own all-reduce
        shards = tuple(t.cuda() for t in tpm.shard_layer_weights(Wqkv, Wo, Wgu, Wd, *heads, world, rank))
        Kl, Vl = tpm.shard_kv_cache(K0, world, rank).cuda(), tpm.shard_kv_cache(V0, world, rank).cuda()
        hid = hidden.cuda()
        a = nccl(hid, Kl.clone(), Vl.clone(), *shards)
        torch.cuda.synchronize()
        dist.barrier()
        outs = [fused(hid, Kl, Vl, *shards) for _ in range(6)]  # several epochs of the exchange
        torch.cuda.synchronize()
        chained = outs[0]
        if B == 1:  # the same exchange through the chained kernels: their arithmetic is the NCCL form's
            _lib.set_tuning(mega=0)
            chained = fused(hid, Kl, Vl, *shards)
            torch.cuda.synchronize()
            _lib.set_tuning(mega=1)
        pouts = [peer(hid, Kl.clone(), Vl.clone(), *shards) for _ in range(4)]  # several epochs of its flags
        torch.cuda.synchronize()
        status = _lib.device_status()
        gathered = [torch.empty_like(a) for _ in range(world)]
        dist.all_gather(gathered, outs[-1])
        same_on_all_ranks = all(torch.equal(g, outs[-1]) for g in gathered)
        dist.all_gather(gathered, pouts[-1])
        same_on_all_ranks = same_on_all_ranks and all(torch.equal(g, pouts[-1]) for g in gathered)
        repeatable = all(torch.equal(o, outs[0]) for o in outs) and all(torch.equal(o, pouts[0]) for o in pouts)
        verdict = torch.tensor([int(same_on_all_ranks and repeatable and status == 0)], device="cuda")
        if rank == 0:
            err_fused = ((outs[0].cpu().float() - ref.float()).norm() / ref.float().norm()).item()
            err_nccl = ((a.cpu().float() - ref.float()).norm() / ref.float().norm()).item()
            err_chained = ((chained.cpu().float() - ref.float()).norm() / ref.float().norm()).item()
            err_peer = ((pouts[0].cpu().float() - ref.float()).norm() / ref.float().norm()).item()
            # two ranks: a + b has one order, so every form of the exchange gives NCCL's bits
            good = (err_fused < 1e-2 and err_nccl < 1e-2 and err_chained < 1e-2 and err_peer < 1e-2
                    and (world != 2 or (torch.equal(a, chained) and torch.equal(a, pouts[0]))))
            verdict *= int(good)
            print(f"tp={world} {sh.name} B={B} S={S}: rel_fro fused {err_fused:.3e} nccl {err_nccl:.3e} peer {err_peer:.3e} "
                  f"identical_across_ranks={same_on_all_ranks} repeatable={repeatable} status={status}", flush=True)
        dist.all_reduce(verdict, op=dist.ReduceOp.MIN)
        ok = ok and bool(verdict.item())
        torch.cuda.synchronize()
        dist.barrier()
        fused.close()
        peer.close()
    # the whole stack: three layers with norm weights and RoPE; batch 2: second sums folded into the next layer's
    # first kernel; batch 1: one persistent kernel per layer
    for B in (2, 1):
        ok = run_stack_case(rank, world, B) and ok
    dist.barrier()
    sys.stdout.flush()
    os._exit(0 if ok else 1)  # a test worker: every check is done and flushed; skip the NCCL teardown and its ordering across ranks


def run_stack_case(rank: int, world: int, B: int) -> bool:
    import copy

    sh, S, NL = wl.QWEN3_VL_2B, 300, 3
    hid, layers, cos, sin = wl.decode_stack_inputs(sh, B, S, NL)
    ref = orc.qwen3_decode_stack_ref(hid, copy.deepcopy(layers), sh.num_heads, sh.num_kv_heads, sh.head_dim, cos, sin) if rank == 0 else None
    local = [{k: (None if v is None else v.cuda()) for k, v in L.items()}
             for L in tpm.shard_stack(layers, sh.num_heads, sh.num_kv_heads, sh.head_dim, world, rank)]
    stack = tpm.TensorParallelDecodeStack(B, S, sh.hidden, sh.inter, sh.num_heads, sh.head_dim, sh.num_kv_heads, NL)
    outs = [stack(hid.cuda(), local, cos.cuda(), sin.cuda()) for _ in range(3)]
    torch.cuda.synchronize()
    status = _lib.device_status()
    gathered = [torch.empty_like(outs[0]) for _ in range(world)]
    dist.all_gather(gathered, outs[-1])
    good = all(torch.equal(g, outs[-1]) for g in gathered) and all(torch.equal(o, outs[0]) for o in outs) and status == 0
    verdict = torch.tensor([int(good)], device="cuda")
    if rank == 0:
        err = ((outs[0].cpu().float() - ref.float()).norm() / ref.float().norm()).item()
        verdict *= int(err < 1e-2)
        print(f"tp={world} stack of {NL} layers B={B} S={S}: rel_fro {err:.3e} identical_across_ranks={good} status={status}", flush=True)
    dist.all_reduce(verdict, op=dist.ReduceOp.MIN)
    torch.cuda.synchronize()
    dist.barrier()
    stack.close()
    return bool(verdict.item())


if __name__ == "__main__":
    main()
