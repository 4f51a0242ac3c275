"""Small Galupel models for the tests: configurations that differ in every size and constant, and random weights.

The writer here knows the tensor names and shapes of the design by itself (it does not ask the engine), draws matrices
as N(0, gain / sqrt(inputs)) so that every layer changes the residual stream noticeably, and lets a test overwrite any
tensor before the folder is written.
"""
from __future__ import annotations

import functools
import json
import os
import tempfile

import torch
from safetensors.torch import save_file


def attn(heads, kv_heads, dim, vdim, size, pool=None, kv_from=None, scale=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5 if scale is None else scale,
         "mask": {"size": size}}
    if pool is not None:
        m["mask"]["pool"] = pool
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": mlp}


def latent(heads, dim, rot_dim, vdim, kv_rank, size=None, rot=None, base=10000.0, scale=None, mlp=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
         "scale": (dim + rot_dim) ** -0.5 if scale is None else scale}
    if rot is not None:
        m["rot"] = {"base": base, "dims": rot}
    if size is not None:
        m["mask"] = {"size": size}
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def moe(experts, top, ff, groups=None):
    r = {"experts": experts, "top": top}
    if groups is not None:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "router": r, "expert": {"ff": ff}}


def config(vocab, width, layers, eps=1e-5, groups=1, scale=1.0, cap=None):
    c = {"architecture": "Galupel", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": groups}, "logit_scale": scale,
         "layers": layers}
    if cap is not None:
        c["logit_softcap"] = cap
    return c


# A: windows narrower and wider than a page run; blocks of 5 (no divisor of the page); the borrower has a window and blocks of
#    its own (7 and 3 against the lender's 20 and 5); a latent layer whose rotation covers half of the rotated part; groups
#    of experts of which two of three are kept; three norm groups
A = config(101, 48, [
    attn(4, 2, 16, 24, size=20, pool=5, mlp=moe(6, 2, 40, groups=(3, 2))),
    latent(3, 8, 8, 16, 24, size=33, rot=4, base=500.0, mlp=moe(4, 1, 32)),
    attn(2, 2, 16, 24, size=7, pool=3, kv_from=0, mlp=None),
    latent(2, 16, 16, 8, 40, size=9, rot=16, base=50.0, mlp=moe(8, 3, 24, groups=(4, 2))),
    attn(4, 2, 16, 24, size=11, pool=16, kv_from=0, mlp=moe(4, 4, 16, groups=(2, 2))),
], eps=1e-6, groups=3, scale=0.7, cap=9.0)
# B: no size a multiple of 8; one norm group (the plain RMS norm); a window of ONE token with blocks of ONE token (every
#    earlier token is seen as a block of its own); a block longer than the window; an attention without blocks; a latent
#    layer without window and one without rotation; groups of one expert; uncapped, unscaled logits
B = config(75, 52, [
    attn(3, 1, 10, 9, size=1, pool=1, mlp=moe(5, 2, 22, groups=(5, 3))),
    latent(2, 6, 4, 7, 10, rot=4, base=77.0, mlp=None),
    attn(6, 3, 6, 5, size=4, pool=9, mlp=moe(3, 3, 18)),
    attn(3, 3, 6, 5, size=13, kv_from=2, mlp=moe(6, 1, 14, groups=(2, 1))),
    latent(3, 5, 6, 3, 12, size=6, mlp=moe(4, 2, 10, groups=(1, 1))),
], eps=2e-5, groups=1)
# C: heads of 64 (the sizes tensor-core kernels take), eight query heads on two kv heads, blocks of 16 (a page) and of 32,
#    a latent of 128 + 64, sixteen experts in four groups
C = config(130, 128, [
    attn(8, 2, 64, 64, size=128, pool=16, mlp=moe(16, 2, 64, groups=(4, 2))),
    latent(4, 32, 64, 32, 128, size=100, rot=64, base=1e6, mlp=moe(8, 4, 48, groups=(2, 1))),
    attn(8, 2, 64, 64, size=48, pool=32, kv_from=0, mlp=moe(8, 2, 32)),
], eps=1e-5, groups=4, scale=0.5, cap=20.0)

# D: a latent layer first; two lenders and a borrower behind each; heads of 128 on one kv head and heads of 32 with values of 64;
#    windows of several pages; every expert in one group and one chosen; a latent of 64 + 32 (the tensor-core sizes) and one of
#    40 + 24 with half of it rotated; pages of 32
D = config(300, 256, [
    latent(4, 32, 32, 48, 64, size=70, rot=32, base=20000.0, mlp=moe(4, 1, 64)),
    attn(4, 1, 128, 128, size=90, pool=10, mlp=moe(6, 3, 32, groups=(2, 1))),
    attn(6, 2, 32, 64, size=40, pool=24, mlp=None),
    attn(8, 1, 128, 128, size=33, pool=32, kv_from=1, mlp=moe(4, 2, 48, groups=(4, 2))),
    latent(5, 24, 24, 16, 40, size=50, rot=12, base=300.0, mlp=moe(8, 2, 40, groups=(2, 2))),
    attn(2, 2, 32, 64, size=100, pool=7, kv_from=2, mlp=moe(5, 5, 24)),
], eps=1e-5, groups=2, scale=0.3, cap=15.0)

ALL = {"A": (A, 1, 16), "B": (B, 2, 8), "C": (C, 3, 16), "D": (D, 4, 32)}        # config, seed, page size


def tensors(cfg: dict, seed: int, gain: float = 1.2) -> dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]

    def mat(rows, cols, k=gain):
        return torch.randn(rows, cols, generator=g) * (k / cols ** 0.5)

    def around(n, mean, std):
        return mean + std * torch.randn(n, generator=g)
    t = {"embed": torch.randn(cfg["vocab"], W, generator=g) * 0.6, "embed.norm": around(W, 1.0, 0.3), "final.norm": around(W, 1.5, 0.4)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        t[p + "norm1"] = around(W, 0.7, 0.2)
        H, Dk, Dv = m["heads"], m["dim"], m["vdim"]
        if layer["type"] == "attention":
            G = m["kv_heads"]
            t[p + "mix.q"], t[p + "mix.o"] = mat(H * Dk, W, 1.5), mat(W, H * Dv, 1.2)
            t[p + "mix.q.norm"], t[p + "mix.temp"] = around(Dk, 1.5, 0.4), around(H, 1.0, 0.4)
            if "kv_from" not in m:
                t[p + "mix.k"], t[p + "mix.v"], t[p + "mix.k.norm"] = mat(G * Dk, W, 1.5), mat(G * Dv, W, 1.5), around(Dk, 1.5, 0.4)
        else:
            R, C = m["rot_dim"], m["kv_rank"]
            t[p + "mix.q"], t[p + "mix.dkv"], t[p + "mix.dkv.norm"] = mat(H * (Dk + R), W, 2.0), mat(C + R, W, 2.0), around(C, 1.0, 0.3)
            t[p + "mix.uk"], t[p + "mix.uv"], t[p + "mix.o"] = mat(H * Dk, C, 2.0), mat(H * Dv, C, 1.5), mat(W, H * Dv, 1.2)
        mlp = layer["mlp"]
        if mlp is not None:
            E = mlp["router"]["experts"]
            t[p + "norm2"] = around(W, 0.7, 0.2)
            t[p + "mlp.router"], t[p + "mlp.correction"] = mat(E, W, 2.0), around(E, 0.0, 0.3)
            for e in range(E):
                t[p + f"mlp.e{e}.up"], t[p + f"mlp.e{e}.down"] = mat(mlp["expert"]["ff"], W, 1.6), mat(W, mlp["expert"]["ff"], 1.0)
    return {k: v.to(torch.bfloat16).contiguous() for k, v in t.items()}


def write_folder(cfg: dict, weights: dict[str, torch.Tensor]) -> str:
    d = tempfile.mkdtemp(prefix="me_galupel_")
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous() for k, v in weights.items()}, os.path.join(d, "model.safetensors"))
    return d


@functools.lru_cache(maxsize=None)
def folder(name: str) -> str:
    cfg, seed, _ = ALL[name]
    return write_folder(cfg, tensors(cfg, seed))
