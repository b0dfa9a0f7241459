"""The multi-layer oracle is a composition of pieces that the golden fixtures pin one by one;
these checks tie the composition back to those pieces (no GPU)."""

import copy

import torch

from oracle import ezops_oracle as orc

from ezops_b200 import workloads as wl

SH = wl.QWEN3_0_6B
HEADS = (SH.num_heads, SH.num_kv_heads, SH.head_dim)


def test_one_plain_layer_is_the_layer_oracle_bit_for_bit():
    hid, layers, _, _ = wl.decode_stack_inputs(SH, 3, 33, 1, rope=False, norm_weights=False)
    a, b = copy.deepcopy(layers[0]), copy.deepcopy(layers[0])
    got = orc.qwen3_decode_stack_ref(hid, [a], *HEADS)
    want = orc.qwen3_dense_decode_ref(hid, b["K_cache"], b["V_cache"], b["Wqkv"], b["Wo"], b["Wgu"], b["Wd"], *HEADS)
    assert torch.equal(got, want)
    assert torch.equal(a["K_cache"], b["K_cache"]) and torch.equal(a["V_cache"], b["V_cache"])


def test_layers_chain_through_the_residual_stream():
    hid, layers, cos, sin = wl.decode_stack_inputs(SH, 2, 20, 3)
    whole = orc.qwen3_decode_stack_ref(hid, copy.deepcopy(layers), *HEADS, cos, sin)
    x = hid
    for L in copy.deepcopy(layers):
        x = orc.qwen3_decode_stack_ref(x, [L], *HEADS, cos, sin)
    assert torch.equal(whole, x)


def test_new_token_k_is_the_rope_operators_k():
    """Slot S-1 of the K cache after a layer with RoPE equals what the stand-alone
    q/k-norm + RoPE oracle (pinned by tests/golden/qk_norm_rope*.npz) writes for the same qkv."""
    B, S = 2, 25
    hid, layers, cos, sin = wl.decode_stack_inputs(SH, B, S, 1)
    L = copy.deepcopy(layers[0])
    orc.qwen3_decode_stack_ref(hid, [L], *HEADS, cos, sin)
    qkv = orc.rmsnorm_bf16_ref(hid, layers[0]["input_norm_w"]) @ layers[0]["Wqkv"].T
    q = qkv[:, :SH.q_rows].view(B, SH.num_heads, SH.head_dim)
    k = qkv[:, SH.q_rows:SH.q_rows + SH.kv_rows].view(B, SH.num_kv_heads, SH.head_dim)
    v = qkv[:, SH.q_rows + SH.kv_rows:].view(B, SH.num_kv_heads, SH.head_dim)
    Kc, Vc = layers[0]["K_cache"].clone(), layers[0]["V_cache"].clone()
    _, k_out = orc.qk_norm_rope_ref(q, k, v, layers[0]["q_norm_w"], layers[0]["k_norm_w"], cos, sin, Kc, Vc, S - 1)
    assert torch.equal(L["K_cache"][:, :, -1], k_out)
    assert torch.equal(L["K_cache"], Kc) and torch.equal(L["V_cache"], Vc)


def test_operator_reference_matches_the_oracle():
    import ezops_b200 as ez

    hid, layers, cos, sin = wl.decode_stack_inputs(SH, 2, 17, 2)
    op = ez.Qwen3DecodeStackOp(2, 17, SH.hidden, SH.inter, SH.num_heads, SH.head_dim, 2, backend="ref", num_kv_heads=SH.num_kv_heads)
    got = op._ref_forward(hid, copy.deepcopy(layers), cos, sin)
    want = orc.qwen3_decode_stack_ref(hid, copy.deepcopy(layers), *HEADS, cos, sin)
    assert torch.equal(got, want)
    assert op.check(got, want)


def test_shard_stack_splits_every_layer_like_one_layer():
    from ezops_b200 import tp as tpm

    _, layers, _, _ = wl.decode_stack_inputs(SH, 2, 12, 2)
    world = 4
    shards = [tpm.shard_stack(layers, *HEADS, world, r) for r in range(world)]
    for l, L in enumerate(layers):
        for r in range(world):
            want = tpm.shard_layer_weights(L["Wqkv"], L["Wo"], L["Wgu"], L["Wd"], *HEADS, world, r)
            got = shards[r][l]
            for name, w in zip(("Wqkv", "Wo", "Wgu", "Wd"), want):
                assert torch.equal(got[name], w)
            assert got["input_norm_w"] is L["input_norm_w"] and got["q_norm_w"] is L["q_norm_w"]  # replicated
        assert torch.equal(torch.cat([shards[r][l]["K_cache"] for r in range(world)], dim=1), L["K_cache"])
        assert torch.equal(torch.cat([shards[r][l]["Wo"] for r in range(world)], dim=1), L["Wo"])


def test_per_row_lengths_reduce_to_the_uniform_case_and_match_the_operator_reference():
    import ezops_b200 as ez

    B, S, NL = 3, 21, 2
    hid, layers, cos, sin = wl.decode_stack_inputs(SH, B, S, NL)
    full = orc.qwen3_decode_stack_ref(hid, copy.deepcopy(layers), *HEADS, cos, sin)
    same = orc.qwen3_decode_stack_ref(hid, copy.deepcopy(layers), *HEADS, cos, sin, seq_lens=[S] * B)
    assert torch.equal(full, same)
    lens = [S, 5, 13]
    la, lb = copy.deepcopy(layers), copy.deepcopy(layers)
    want = orc.qwen3_decode_stack_ref(hid, la, *HEADS, cos, sin, seq_lens=lens)
    op = ez.Qwen3DecodeStackOp(B, S, SH.hidden, SH.inter, SH.num_heads, SH.head_dim, NL, backend="ref",
                               num_kv_heads=SH.num_kv_heads, seq_lens=lens)
    got = op(hid, lb, cos, sin)
    assert torch.equal(got, want)
    for L0, L1 in zip(layers, la):
        for b, n in enumerate(lens):  # only slot len-1 of each row changed
            keep = [i for i in range(S) if i != n - 1]
            assert torch.equal(L1["K_cache"][b][:, keep], L0["K_cache"][b][:, keep])
            assert not torch.equal(L1["K_cache"][b][:, n - 1], L0["K_cache"][b][:, n - 1])
    # a row with a shorter prefix must not depend on the keys behind it
    lc = copy.deepcopy(layers)
    for L in lc:
        L["K_cache"][1, :, 5:] = 7.0
        L["V_cache"][1, :, 5:] = -3.0
    again = orc.qwen3_decode_stack_ref(hid, lc, *HEADS, cos, sin, seq_lens=lens)
    assert torch.equal(again[1], want[1])
    import pytest

    with pytest.raises(ValueError):
        ez.Qwen3DecodeStackOp(B, S, SH.hidden, SH.inter, SH.num_heads, SH.head_dim, NL, seq_lens=[S, 0, 3])
