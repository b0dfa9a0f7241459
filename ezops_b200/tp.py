"""Tensor-parallel form of the Qwen3 decode layer: one process per GPU, heads
and FFN columns split across ranks, one sum over ranks after o_proj and one
after down_proj (the reference is single-GPU and has no counterpart).

Sharding (``tp`` ranks, rank ``r``):
    Wqkv rows : q heads [r*NH/tp, (r+1)*NH/tp), the matching k heads and v heads
    KV cache  : the rank's kv heads                    -> attention is rank-local
    Wo        : the columns of the rank's q heads      -> partial [B, H], summed
    Wgu rows  : gate rows and up rows [r*I/tp, (r+1)*I/tp)
    Wd        : the same columns                       -> partial [B, H], summed
Hidden states, residuals and norms are replicated.  Partials are exchanged in
fp32, either with ``torch.distributed.all_reduce`` (NCCL over NVLink on GPUs;
``exchange="nccl"``) or inside the projection kernels themselves, which store
their partial into an inbox on every rank over NVLink peer memory and publish an
epoch flag that the consuming kernel waits for (``exchange="fused"``: one C call
and six kernels per layer, no collective launch in between).
"""

from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from . import _lib


def shard_layer_weights(Wqkv, Wo, Wgu, Wd, num_heads: int, num_kv_heads: int, head_dim: int, tp: int, rank: int):
    """Contiguous per-rank copies of one layer's weights (see module docstring)."""
    if num_heads % tp or num_kv_heads % tp:
        raise ValueError(f"tp ({tp}) must divide num_heads ({num_heads}) and num_kv_heads ({num_kv_heads})")
    inter = Wgu.shape[0] // 2
    if inter % tp or (inter // tp) % 16:
        raise ValueError(f"intermediate_size / tp ({inter}/{tp}) must be a multiple of 16")
    q_rows, kv_rows = num_heads * head_dim, num_kv_heads * head_dim
    ql, kl, il = q_rows // tp, kv_rows // tp, inter // tp
    Wqkv_r = torch.cat(
        [
            Wqkv[rank * ql : (rank + 1) * ql],
            Wqkv[q_rows + rank * kl : q_rows + (rank + 1) * kl],
            Wqkv[q_rows + kv_rows + rank * kl : q_rows + kv_rows + (rank + 1) * kl],
        ]
    ).contiguous()
    Wo_r = Wo[:, rank * ql : (rank + 1) * ql].contiguous()
    Wgu_r = torch.cat([Wgu[rank * il : (rank + 1) * il], Wgu[inter + rank * il : inter + (rank + 1) * il]]).contiguous()
    Wd_r = Wd[:, rank * il : (rank + 1) * il].contiguous()
    return Wqkv_r, Wo_r, Wgu_r, Wd_r


def shard_kv_cache(cache: torch.Tensor, tp: int, rank: int) -> torch.Tensor:
    nkv = cache.shape[1]
    if nkv % tp:
        raise ValueError(f"tp ({tp}) must divide num_kv_heads ({nkv})")
    n = nkv // tp
    return cache[:, rank * n : (rank + 1) * n].contiguous()


class TensorParallelDecodeLayer:
    """Per-rank executor.  ``__call__(hidden, K_local, V_local, Wqkv_l, Wo_l, Wgu_l, Wd_l)``
    returns the full [B, H] layer output (identical on every rank)."""

    rms_eps = 1e-6

    def __init__(self, batch, seq_len, hidden_size, intermediate_size, num_heads, head_dim, num_kv_heads, group=None,
                 exchange: str = "nccl"):
        if exchange not in ("nccl", "fused", "peer"):
            raise ValueError(f"exchange must be 'nccl', 'fused' or 'peer', got {exchange!r}")
        self.exchange = exchange
        self._comm = None
        self.group = group
        self.tp = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        tp = self.tp
        if num_heads % tp or num_kv_heads % tp or intermediate_size % tp:
            raise ValueError(f"tp ({tp}) must divide num_heads, num_kv_heads and intermediate_size")
        self.B, self.S, self.H, self.D = batch, seq_len, hidden_size, head_dim
        self.NH_l, self.NKV_l, self.I_l = num_heads // tp, num_kv_heads // tp, intermediate_size // tp
        if self.I_l % 16 or hidden_size % 16:
            raise ValueError("hidden_size and intermediate_size / tp must be divisible by 16")
        self._bufs = None

    # -- buffers ------------------------------------------------------------
    def _buffers(self, device):
        if self._bufs is None or self._bufs["partial_o"].device != device:
            lib = _lib.load()
            ws1 = lib.ezb_qwen3_decode_layer_workspace_bytes(self.B, self.S, self.H, self.I_l, self.NH_l, self.NKV_l, self.D)
            ws2 = lib.ezb_o_proj_ffn_workspace_bytes(self.B, self.H, self.I_l, 16)
            self._bufs = dict(
                ws1=torch.zeros(max(ws1, 256), dtype=torch.uint8, device=device),
                ws2=torch.zeros(max(ws2, 256), dtype=torch.uint8, device=device),
                partial_o=torch.empty(self.B, self.H, dtype=torch.float32, device=device),
                partial_d=torch.empty(self.B, self.H, dtype=torch.float32, device=device),
                x2=torch.empty(self.B, self.H, dtype=torch.bfloat16, device=device),
            )
        return self._bufs

    # -- the three local parts (C ABI) and the exchange in between ------------
    # ``po`` / ``so`` / ``pd`` / ``sd``: device addresses of the o_proj partial and its sum over ranks, and of the
    # down partial and its sum; by default the buffers of ``bufs``, where NCCL sums a partial in place
    def _part_attn(self, hidden, K_l, V_l, Wqkv_l, Wo_l, bufs, po=None):
        lib = _lib.load()
        po = bufs["partial_o"].data_ptr() if po is None else po
        s = torch.cuda.current_stream().cuda_stream
        _lib.check(lib.ezb_qwen3_decode_layer_tp_attn(
            hidden.data_ptr(), K_l.data_ptr(), V_l.data_ptr(), Wqkv_l.data_ptr(), Wo_l.data_ptr(),
            po, bufs["ws1"].data_ptr(), bufs["ws1"].numel(),
            self.B, self.S, self.H, self.NH_l, self.NKV_l, self.D, self.rms_eps, s))

    def _part_ffn(self, hidden, Wgu_l, Wd_l, bufs, so=None, pd=None):
        lib = _lib.load()
        so = bufs["partial_o"].data_ptr() if so is None else so
        pd = bufs["partial_d"].data_ptr() if pd is None else pd
        s = torch.cuda.current_stream().cuda_stream
        _lib.check(lib.ezb_qwen3_decode_layer_tp_ffn(
            hidden.data_ptr(), so, Wgu_l.data_ptr(), Wd_l.data_ptr(), bufs["x2"].data_ptr(),
            pd, bufs["ws2"].data_ptr(), bufs["ws2"].numel(),
            self.B, self.H, self.I_l, self.rms_eps, s))

    def _part_out(self, out, bufs, sd=None):
        lib = _lib.load()
        sd = bufs["partial_d"].data_ptr() if sd is None else sd
        s = torch.cuda.current_stream().cuda_stream
        _lib.check(lib.ezb_residual_add_f32(bufs["x2"].data_ptr(), sd, out.data_ptr(), self.B, self.H, s))

    def _call_peer(self, hidden, K_l, V_l, Wqkv_l, Wo_l, Wgu_l, Wd_l, out, bufs):
        """The three parts with this library's own in-place sum over ranks in between (``ezb_tp_allreduce_f32``:
        two-shot over peer memory, epoch-tagged cells) instead of NCCL's all-reduce."""
        lib = _lib.load()
        comm = self._fused_comm(hidden.device)
        s = torch.cuda.current_stream().cuda_stream
        self._part_attn(hidden, K_l, V_l, Wqkv_l, Wo_l, bufs)
        _lib.check(lib.ezb_tp_allreduce_f32(bufs["partial_o"].data_ptr(), comm["bases"], self.tp, self.rank, 0, self.B, self.H, s))
        self._part_ffn(hidden, Wgu_l, Wd_l, bufs)
        _lib.check(lib.ezb_tp_allreduce_f32(bufs["partial_d"].data_ptr(), comm["bases"], self.tp, self.rank, 1, self.B, self.H, s))
        self._part_out(out, bufs)

    def _sum_over_ranks(self, t: torch.Tensor) -> None:
        if self.tp > 1:
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)

    # -- fused exchange: peer-mapped inboxes ------------------------------------
    def _fused_comm(self, device):
        """Allocates this rank's communication buffer, exchanges IPC handles over the
        process group and maps every peer's buffer.  Collective: all ranks call it
        together (it happens inside the first ``__call__``)."""
        if self._comm is not None:
            return self._comm
        lib = _lib.load()
        nbytes = lib.ezb_tp_comm_bytes(self.B, self.H)
        own = ctypes.c_void_p()
        _lib.check(lib.ezb_tp_comm_alloc(nbytes, ctypes.byref(own)))
        handle = ctypes.create_string_buffer(64)
        _lib.check(lib.ezb_ipc_export(own, handle))
        handles = [None] * self.tp
        if self.tp > 1:
            dist.all_gather_object(handles, handle.raw, group=self.group)
        bases = (ctypes.c_void_p * self.tp)()
        mapped = []
        for r in range(self.tp):
            if r == self.rank:
                bases[r] = own.value
                continue
            peer = ctypes.c_void_p()
            _lib.check(lib.ezb_ipc_open(ctypes.create_string_buffer(handles[r], 64), ctypes.byref(peer)))
            bases[r] = peer.value
            mapped.append(peer)
        torch.cuda.synchronize(device)
        if self.tp > 1:
            dist.barrier(group=self.group)  # every inbox is zeroed and mapped before anyone pushes
        self._comm = dict(own=own, bases=bases, mapped=mapped)
        return self._comm

    def close(self):
        """Unmaps the peers' buffers and frees this rank's (call on every rank, after a device sync)."""
        if self._comm is None:
            return
        lib = _lib.load()
        for peer in self._comm["mapped"]:
            lib.ezb_ipc_close(peer)
        if self.tp > 1:
            dist.barrier(group=self.group)
        lib.ezb_tp_comm_free(self._comm["own"])
        self._comm = None

    def _call_fused(self, hidden, K_l, V_l, Wqkv_l, Wo_l, Wgu_l, Wd_l, out, bufs):
        lib = _lib.load()
        comm = self._fused_comm(hidden.device)
        s = torch.cuda.current_stream().cuda_stream
        _lib.check(lib.ezb_qwen3_decode_layer_tp_fused(
            hidden.data_ptr(), K_l.data_ptr(), V_l.data_ptr(), Wqkv_l.data_ptr(), Wo_l.data_ptr(), Wgu_l.data_ptr(),
            Wd_l.data_ptr(), out.data_ptr(), bufs["ws1"].data_ptr(), bufs["ws1"].numel(), comm["bases"], self.tp,
            self.rank, self.B, self.S, self.H, self.I_l, self.NH_l, self.NKV_l, self.D, self.rms_eps, s))

    def __call__(self, hidden, K_local, V_local, Wqkv_l, Wo_l, Wgu_l, Wd_l, out=None):
        bufs = self._buffers(hidden.device)
        if out is None:
            out = torch.empty_like(hidden)
        if self.exchange == "fused":
            self._call_fused(hidden, K_local, V_local, Wqkv_l, Wo_l, Wgu_l, Wd_l, out, bufs)
            return out
        if self.exchange == "peer":
            self._call_peer(hidden, K_local, V_local, Wqkv_l, Wo_l, Wgu_l, Wd_l, out, bufs)
            return out
        self._part_attn(hidden, K_local, V_local, Wqkv_l, Wo_l, bufs)
        self._sum_over_ranks(bufs["partial_o"])
        self._part_ffn(hidden, Wgu_l, Wd_l, bufs)
        self._sum_over_ranks(bufs["partial_d"])
        self._part_out(out, bufs)
        return out


def shard_stack(layers, num_heads: int, num_kv_heads: int, head_dim: int, tp: int, rank: int):
    """Per-rank copy of a stack's layers (dicts as ``Qwen3DecodeStackOp.gen_data`` returns them):
    weights and caches sharded as for one layer, norm weights replicated."""
    out = []
    for L in layers:
        Wqkv, Wo, Wgu, Wd = shard_layer_weights(L["Wqkv"], L["Wo"], L["Wgu"], L["Wd"], num_heads, num_kv_heads, head_dim, tp, rank)
        local = {"K_cache": shard_kv_cache(L["K_cache"], tp, rank), "V_cache": shard_kv_cache(L["V_cache"], tp, rank),
                 "Wqkv": Wqkv, "Wo": Wo, "Wgu": Wgu, "Wd": Wd}
        for key in ("input_norm_w", "post_norm_w", "q_norm_w", "k_norm_w"):
            local[key] = L.get(key)
        out.append(local)
    return out


class TensorParallelDecodeStack(TensorParallelDecodeLayer):
    """All layers of a decoder stack on this rank's shards in one call, the sums over ranks fused
    into the kernels (``ezb_qwen3_decode_stack_tp_fused``).  ``__call__(hidden, layers_local, cos,
    sin)``; every rank returns the same [B, H] output."""

    def __init__(self, batch, seq_len, hidden_size, intermediate_size, num_heads, head_dim, num_kv_heads, num_layers, group=None):
        super().__init__(batch, seq_len, hidden_size, intermediate_size, num_heads, head_dim, num_kv_heads, group=group,
                         exchange="fused")
        self.L = num_layers
        self._table, self._table_key, self._stack_ws = None, None, None

    def _layer_table(self, layers):
        names = ("K_cache", "V_cache", "Wqkv", "Wo", "Wgu", "Wd", "input_norm_w", "post_norm_w", "q_norm_w", "k_norm_w")
        key = tuple(0 if L.get(n) is None else L[n].data_ptr() for L in layers for n in names)
        if key != self._table_key:
            table = (_lib.LayerStruct * len(layers))()
            for i, L in enumerate(layers):
                for n in names:
                    t = L.get(n)
                    if t is None and not n.endswith("_norm_w"):
                        raise ValueError(f"layer {i}: {n} is required")
                    if t is not None and (not t.is_cuda or t.dtype != torch.bfloat16 or not t.is_contiguous()):
                        raise ValueError(f"layer {i}: {n} must be a contiguous bf16 CUDA tensor")
                    setattr(table[i], n, None if t is None else t.data_ptr())
            self._table, self._table_key = table, key
        return self._table

    def __call__(self, hidden, layers_local, cos=None, sin=None, out=None, seq_lens=None):
        if len(layers_local) != self.L:
            raise ValueError(f"expected {self.L} layers, got {len(layers_local)}")
        lib = _lib.load()
        if self._stack_ws is None or self._stack_ws.device != hidden.device:
            need = lib.ezb_qwen3_decode_stack_tp_fused_workspace_bytes(self.B, self.S, self.H, self.I_l, self.NH_l, self.NKV_l, self.D)
            self._stack_ws = torch.zeros(max(need, 256), dtype=torch.uint8, device=hidden.device)
        comm = self._fused_comm(hidden.device)
        table = self._layer_table(layers_local)
        if out is None:
            out = torch.empty_like(hidden)
        _lib.check(lib.ezb_qwen3_decode_stack_tp_fused(
            hidden.data_ptr(), out.data_ptr(), table, self.L, None if cos is None else cos.data_ptr(),
            None if sin is None else sin.data_ptr(), self.S - 1, None if seq_lens is None else seq_lens.data_ptr(),
            self._stack_ws.data_ptr(), self._stack_ws.numel(), comm["bases"],
            self.tp, self.rank, self.B, self.S, self.H, self.I_l, self.NH_l, self.NKV_l, self.D, self.rms_eps,
            torch.cuda.current_stream().cuda_stream))
        return out

