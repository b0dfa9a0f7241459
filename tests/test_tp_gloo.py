"""World-size-2 test of the tensor-parallel orchestration on CPU ranks (gloo).

The per-rank compute entry points of ``TensorParallelDecodeLayer`` are CUDA
only, so this test replaces those three methods -- inside the test processes
only -- by torch-CPU emulations of what each part computes, and checks what the
host logic is responsible for: contiguous head / column sharding, the order
part -> sum over ranks -> part, and that every rank ends with the same full
output equal to the unsharded oracle.
"""

import os
import socket
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, result_dir: str):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    from ezops_b200 import tp as tpm
    from ezops_b200 import workloads as wl
    from oracle import ezops_oracle as orc

    sh = wl.LayerShape("tiny", 128, 256, 4, 2, 32)
    B, S = 2, 19
    hidden, K0, V0, Wqkv, Wo, Wgu, Wd = wl.decode_layer_inputs(sh, B, S, seed=5)
    heads = (sh.num_heads, sh.num_kv_heads, sh.head_dim)

    lay = tpm.TensorParallelDecodeLayer(B, S, sh.hidden, sh.inter, *heads[:1], sh.head_dim, sh.num_kv_heads)
    assert lay.tp == world and lay.rank == rank
    Wqkv_l, Wo_l, Wgu_l, Wd_l = tpm.shard_layer_weights(Wqkv, Wo, Wgu, Wd, *heads, world, rank)
    K_l, V_l = tpm.shard_kv_cache(K0, world, rank), tpm.shard_kv_cache(V0, world, rank)
    assert torch.equal(Wqkv_l, orc.shard_layer_weights(Wqkv, Wo, Wgu, Wd, *heads, world, rank)[0])

    calls = []
    bufs = dict(partial_o=torch.empty(B, sh.hidden), partial_d=torch.empty(B, sh.hidden),
                x2=torch.empty(B, sh.hidden, dtype=torch.bfloat16))
    lay._buffers = lambda device: bufs
    NH_l, NKV_l, D = lay.NH_l, lay.NKV_l, sh.head_dim

    def part_attn(hid, K, V, Wq, Wo_, b):
        calls.append("attn")
        x = orc.rmsnorm_bf16_ref(hid)
        qkv = x @ Wq.T
        q = orc.rmsnorm_bf16_ref(qkv[:, : NH_l * D].view(B, NH_l, D))
        k = orc.rmsnorm_bf16_ref(qkv[:, NH_l * D : (NH_l + NKV_l) * D].view(B, NKV_l, D))
        K[:, :, -1], V[:, :, -1] = k, qkv[:, (NH_l + NKV_l) * D :].view(B, NKV_l, D)
        attn = orc.attn_decode_ref(q.unsqueeze(2), K, V).squeeze(2).reshape(B, NH_l * D)
        b["partial_o"].copy_(attn.float() @ Wo_.float().T)

    def part_ffn(hid, Wgu_, Wd_, b):
        calls.append("ffn")
        x2 = hid + b["partial_o"].to(torch.bfloat16)
        b["x2"].copy_(x2)
        gu = orc.rmsnorm_bf16_ref(x2) @ Wgu_.T
        il = Wgu_.shape[0] // 2
        h = torch.nn.functional.silu(gu[:, :il]) * gu[:, il:]
        b["partial_d"].copy_(h.float() @ Wd_.float().T)

    def part_out(out, b):
        calls.append("out")
        out.copy_(b["x2"] + b["partial_d"].to(torch.bfloat16))

    lay._part_attn, lay._part_ffn, lay._part_out = part_attn, part_ffn, part_out
    out = lay(hidden, K_l, V_l, Wqkv_l, Wo_l, Wgu_l, Wd_l)
    assert calls == ["attn", "ffn", "out"]

    ref = orc.qwen3_dense_decode_ref(hidden, K0.clone(), V0.clone(), Wqkv, Wo, Wgu, Wd, *heads)
    err = ((out.float() - ref.float()).norm() / ref.float().norm()).item()
    gathered = [torch.empty_like(out) for _ in range(world)]
    dist.all_gather(gathered, out)
    same = all(torch.equal(g, out) for g in gathered)
    Path(result_dir, f"rank{rank}.txt").write_text(f"{err} {int(same)}")
    dist.destroy_process_group()


def test_two_rank_tensor_parallel_layer_on_gloo(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        err, same = Path(tmp_path, f"rank{r}.txt").read_text().split()
        assert float(err) < 1e-2 and same == "1"


def test_exchange_names_are_checked():
    import pytest

    from ezops_b200 import tp as tpm

    for name in ("nccl", "fused", "peer"):
        assert tpm.TensorParallelDecodeLayer(1, 64, 256, 512, 4, 64, 2, exchange=name).exchange == name
    with pytest.raises(ValueError, match="exchange"):
        tpm.TensorParallelDecodeLayer(1, 64, 256, 512, 4, 64, 2, exchange="mpi")


def test_shard_shapes_and_errors():
    sys.path.insert(0, str(ROOT))
    import pytest

    from ezops_b200 import tp as tpm

    Wqkv, Wo, Wgu, Wd = torch.zeros(6144, 64), torch.zeros(64, 4096), torch.zeros(2 * 1024, 64), torch.zeros(64, 1024)
    a, b, c, d = tpm.shard_layer_weights(Wqkv, Wo, Wgu, Wd, 32, 8, 128, 8, 3)
    assert a.shape == (768, 64) and b.shape == (64, 512) and c.shape == (256, 64) and d.shape == (64, 128)
    assert all(t.is_contiguous() for t in (a, b, c, d))
    with pytest.raises(ValueError):
        tpm.shard_layer_weights(Wqkv, Wo, Wgu, Wd, 32, 8, 128, 3, 0)
    with pytest.raises(ValueError):
        tpm.shard_kv_cache(torch.zeros(1, 8, 4, 128), 3, 0)
