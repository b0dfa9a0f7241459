"""Generate the golden fixtures that pin ``oracle/ezops_oracle.py``.

Run once, in a container where the reference project is mounted::

    TILELANG_CACHE_DIR=/tmp/ezops_tl python tests/golden/make_golden.py /path/to/reference

It imports the reference's ``ezops`` package, builds small seeded CPU tensors
(the reference's own ``gen_data`` hard-codes ``device="cuda"``, so the tensors
are built here with the same shapes and scalings), calls the reference's
``_ref_forward`` methods on them and stores inputs and outputs, bf16 as raw
uint16, in ``tests/golden/*.npz``.  The one exception is stand-alone decode
attention: the reference method pins the cuDNN SDPA backend, which cannot run
on CPU, so that fixture calls the same ``F.scaled_dot_product_attention(Q, K,
V, enable_gqa=True)`` expression without the pin; the layer fixtures exercise
SDPA through the reference's own layer method.
"""

import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def pack(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.uint16).numpy().copy()
    return t.contiguous().numpy().copy()


def save(name: str, **tensors):
    np.savez(HERE / f"{name}.npz", **{k: pack(v) if isinstance(v, torch.Tensor) else np.asarray(v) for k, v in tensors.items()})
    print("wrote", name, {k: tuple(v.shape) if hasattr(v, "shape") else v for k, v in tensors.items()})


def main(ref_root: str):
    os.environ.setdefault("TILELANG_CACHE_DIR", "/tmp/ezops_tl")
    sys.path.insert(0, ref_root)
    import ezops  # the reference package
    import torch.nn.functional as F

    bf = torch.bfloat16
    g = torch.Generator().manual_seed(42)

    def randn(*shape, dtype=bf, scale=1.0):
        return (torch.randn(*shape, generator=g, dtype=torch.float32) * scale).to(dtype)

    # ---- gemv (reference "ref" layout: B is [K, N]) -------------------------
    N, K = 192, 320
    A, Wnk = randn(K), randn(N, K)
    C = torch.empty(N, dtype=bf)
    ezops.GemvOp(N, K, backend="ref")._ref_forward(A, Wnk.T.contiguous(), C)
    save("gemv", x=A, W=Wnk, y=C)

    # ---- rmsnorm fp32 -------------------------------------------------------
    X = randn(5, 1025, dtype=torch.float32)
    Out = torch.empty_like(X)
    ezops.RmsNormOp(5, 1025, backend="ref", eps=1e-6)._ref_forward(X, Out)
    save("rmsnorm_f32", X=X, Out=Out, eps=1e-6)

    # ---- fused qk-norm + rope ----------------------------------------------
    for tag, (B, NQ, NKV, D, S, pos) in {"a": (2, 4, 2, 64, 33, 17), "b": (1, 16, 8, 128, 40, 0)}.items():
        op = ezops.FusedQkNormRopeOp(B, NQ, D, S, pos, backend="ref", num_kv_heads=NKV)
        q, k, v = randn(B, NQ, D), randn(B, NKV, D), randn(B, NKV, D)
        qw, kw = randn(D), randn(D)
        inv = 1.0 / (op.rope_theta ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
        ang = torch.arange(S, dtype=torch.float32)[:, None] * inv[None, :]
        cos = torch.cat([ang.cos(), ang.cos()], -1).to(bf)
        sin = torch.cat([ang.sin(), ang.sin()], -1).to(bf)
        Kc, Vc = randn(B, NKV, S, D), randn(B, NKV, S, D)
        K0, V0 = Kc.clone(), Vc.clone()
        q_out, k_out = op._ref_forward(q, k, v, qw, kw, cos, sin, Kc, Vc)
        save(f"qk_norm_rope_{tag}", q=q, k=k, v=v, qw=qw, kw=kw, cos=cos, sin=sin, K0=K0, V0=V0,
             q_out=q_out, k_out=k_out, K1=Kc, V1=Vc, position=pos)

    # ---- stand-alone decode attention (see module docstring) ---------------
    B, H, NKV, S, D = 2, 8, 2, 77, 64
    Q, Kt, Vt = randn(B, H, 1, D), randn(B, NKV, S, D), randn(B, NKV, S, D)
    out = F.scaled_dot_product_attention(Q, Kt, Vt, enable_gqa=True)
    save("attn_decode", Q=Q, K=Kt, V=Vt, out=out)

    # ---- fused o_proj + ffn --------------------------------------------------
    for tag, (B, H, I, NH, D) in {"a": (2, 128, 384, 4, 32), "b": (1, 64, 192, 4, 32)}.items():
        op = ezops.FusedOProjFfnOp(B, H, I, NH, D, backend="ref")
        Qr = NH * D
        attn, res = randn(B, Qr), randn(B, H)
        Wo, pw = randn(H, Qr, scale=Qr**-0.5), randn(H)
        Wg, Wu, Wd = randn(I, H, scale=H**-0.5), randn(I, H, scale=H**-0.5), randn(H, I, scale=I**-0.5)
        out = op._ref_forward(attn, res, Wo, pw, Wg, Wu, Wd)
        save(f"o_proj_ffn_{tag}", attn=attn, residual=res, Wo=Wo, post_norm_w=pw, Wg=Wg, Wu=Wu, Wd=Wd, out=out)

    # ---- whole decode layer --------------------------------------------------
    for tag, (B, S, H, I, NH, D, NKV) in {"a": (2, 19, 128, 256, 4, 32, 2), "b": (1, 1, 128, 256, 4, 32, 4)}.items():
        op = ezops.Qwen3DenseDecodeOp(B, S, H, I, NH, D, backend="ref", num_kv_heads=NKV)
        Qr, KVr = NH * D, NKV * D
        hidden = randn(B, H)
        Kc, Vc = randn(B, NKV, S, D), randn(B, NKV, S, D)
        K0, V0 = Kc.clone(), Vc.clone()
        Wqkv = randn(Qr + 2 * KVr, H, scale=H**-0.5)
        Wo = randn(H, Qr, scale=Qr**-0.5)
        Wgu = randn(2 * I, H, scale=H**-0.5)
        Wd = randn(H, I, scale=I**-0.5)
        out = op._ref_forward(hidden, Kc, Vc, Wqkv, Wo, Wgu, Wd)
        save(f"decode_layer_{tag}", hidden=hidden, K0=K0, V0=V0, Wqkv=Wqkv, Wo=Wo, Wgu=Wgu, Wd=Wd,
             out=out, K1=Kc, V1=Vc, num_heads=NH, num_kv_heads=NKV, head_dim=D)

    (HERE / "VERSIONS.txt").write_text(
        f"generated with torch {torch.__version__}, numpy {np.__version__}, "
        f"threads {torch.get_num_threads()}\nreference package: ezops (imported from a read-only mount)\n"
    )


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path of an ez-ops checkout>")
    main(sys.argv[1])
