"""Small Gevulorn models for the tests: configurations that differ in every size and constant, and random weights.

The writer here knows the tensor names and shapes of the design by itself (it does not ask the engine), draws matrices
as N(0, gain / sqrt(inputs)) so that every layer changes the residual stream noticeably, and lets a test overwrite any
tensor before the folder is written.  config.json does not say the rank of a gla layer's decay projection: the engine has
to read it from the weights (``RANKS`` below is the writer's own business).
"""
from __future__ import annotations

import functools
import json
import os
import tempfile

import torch
from safetensors.torch import save_file


def gla(heads, dim, vdim, tau, mlp=None):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}, "mlp": mlp}


def attn(heads, kv_heads, dim, vdim, rot=None, base=10000.0, size=None, keep_first=None, scale=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5 if scale is None else scale}
    if rot is not None:
        m["rot"] = {"base": base, "dims": rot}
    if size is not None:
        m["mask"] = {"size": size}
        if keep_first is not None:
            m["mask"]["keep_first"] = keep_first
    return {"type": "attention", "mixer": m, "mlp": mlp}


def attn2(heads, kv_heads, dim, vdim, rot=None, base=10000.0, scaling=None, size=None, softcap=None, scale=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5 if scale is None else scale}
    if rot is not None:
        m["rot"] = {"base": base, "dims": rot}
        if scaling is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    if size is not None:
        m["mask"] = {"size": size}
    if softcap is not None:
        m["softcap"] = softcap
    return {"type": "attention_2", "mixer": m, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=None):
    out = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


def config(vocab, width, layers, eps=1e-5, emb=1.0, cap=None, loop=None):
    c = {"architecture": "Gevulorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": emb}, "layers": layers}
    if cap is not None:
        c["logit_softcap"] = cap
    if loop is not None:
        c["loop"] = dict(zip(("start", "stop", "times"), loop))
    return c


# A: the loop sits in the middle and holds all three mixers; a window narrower than a page run with two kept tokens; chunks
#    of 24; the frequencies' scaling cuts through the rotated range; two kv heads of four
A = config(101, 64, [
    gla(2, 16, 24, 8.0, mlp=dense(96)),
    attn(4, 2, 16, 24, rot=8, base=5000.0, size=20, keep_first=2, mlp=moe(6, 2, 40, shared=48)),
    gla(4, 8, 8, 2.0, mlp=moe(4, 1, 32)),
    attn2(4, 2, 16, 8, rot=16, base=100.0, scaling=(4.0, 1.0, 4.0, 64), size=24, softcap=5.0, mlp=dense(80)),
    attn(2, 1, 24, 16, rot=12, base=300.0, size=33, mlp=None),
], eps=1e-6, emb=3.0, cap=8.0, loop=(1, 4, 2))
# B: no size a multiple of 8; odd value sizes; the loop covers the last layers and runs three times; a window without kept
#    tokens and one whose kept tokens exceed a page; an attention_2 without chunks, cap or scaling; every expert chosen;
#    uncapped logits
B = config(75, 52, [
    attn(3, 1, 10, 9, rot=6, base=300.0, size=17, mlp=dense(70)),
    attn2(6, 3, 6, 5, rot=6, base=50.0, mlp=moe(3, 3, 22)),
    gla(3, 10, 7, 1.0, mlp=None),
    attn(2, 2, 12, 12, rot=4, base=77.0, size=9, keep_first=11, mlp=moe(5, 3, 18, shared=14)),
], eps=2e-5, emb=0.7, loop=(2, 4, 3))
# C: heads of 64 (the sizes tensor-core kernels take), eight query heads on two kv heads, no loop at all, chunks of 64 and a
#    window of 128 with 16 kept tokens, 16 experts
C = config(130, 128, [
    attn(8, 2, 64, 64, rot=64, size=128, keep_first=16, mlp=dense(256)),
    gla(2, 64, 64, 16.0, mlp=moe(16, 2, 64, shared=64)),
    attn2(8, 2, 64, 64, rot=32, base=1e6, scaling=(8.0, 1.0, 4.0, 512), size=64, softcap=30.0, mlp=moe(8, 4, 48)),
], eps=1e-5, emb=11.0, cap=20.0)
# D: one layer looped four times; a window of ONE token (a query sees itself, the kept first token and the sink); chunks of
#    one page; one head everywhere
D = config(64, 40, [
    attn(1, 1, 8, 8, rot=8, base=50.0, size=1, keep_first=1, mlp=dense(56)),
    attn2(1, 1, 8, 16, rot=4, base=50.0, size=32, softcap=2.0, mlp=None),
    gla(1, 4, 40, 4.0, mlp=dense(24)),
], eps=1e-5, emb=2.0, cap=3.0, loop=(2, 3, 4))

ALL = {"A": (A, 1, 16), "B": (B, 2, 8), "C": (C, 3, 16), "D": (D, 4, 32)}        # config, seed, page size
RANKS = {"A": 6, "B": 3, "C": 16, "D": 1}                                        # of the decay's low-rank projection


def tensors(cfg: dict, seed: int, rank: int, gain: float = 1.2) -> dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]

    def mat(rows, cols, k=gain):
        return torch.randn(rows, cols, generator=g) * (k / cols ** 0.5)

    def around(n, mean, std):
        return mean + std * torch.randn(n, generator=g)

    def glu(prefix, ff):
        t[prefix + "gate"], t[prefix + "up"], t[prefix + "down"] = mat(ff, W, 1.6), mat(ff, W, 1.6), mat(W, ff, 1.0)
    t = {"embed": torch.randn(cfg["vocab"], W, generator=g) * 0.6, "final.norm": around(W, 1.0, 0.3), "final.norm.b": around(W, 0.0, 0.2),
         "head": mat(cfg["vocab"], W, 2.0)}
    if cfg.get("loop"):
        t["loop.step"] = torch.randn(cfg["loop"]["times"], W, generator=g) * 0.8
    for i, layer in enumerate(cfg["layers"]):
        p, m, kind = f"l{i}.", layer["mixer"], layer["type"]
        for n in ("norm1", "norm2"):
            t[p + n], t[p + n + ".b"] = around(W, 1.0, 0.3), around(W, 0.0, 0.3)
        H, Dk, Dv = m["heads"], m["dim"], m["vdim"]
        if kind == "gla":
            t[p + "mix.q"], t[p + "mix.k"] = mat(H * Dk, W, 2.0), mat(H * Dk, W, 2.0)
            t[p + "mix.v"], t[p + "mix.g"], t[p + "mix.o"] = mat(H * Dv, W, 1.5), mat(H * Dv, W, 1.5), mat(W, H * Dv, 1.2)
            t[p + "mix.norm"] = around(Dv, 1.0, 0.3)
            t[p + "mix.a1"], t[p + "mix.a2"] = mat(rank, W, 1.5), mat(H * Dk, rank, 3.0)
            t[p + "mix.a2.b"] = around(H * Dk, 1.0, 2.0)
        else:
            G = m["kv_heads"]
            t[p + "mix.q"], t[p + "mix.k"], t[p + "mix.v"] = mat(H * Dk, W, 1.5), mat(G * Dk, W, 1.5), mat(G * Dv, W, 1.5)
            t[p + "mix.o"] = mat(W, H * Dv, 1.2)
            t[p + "mix.sink"] = around(H, 0.5, 1.0)
            if kind == "attention_2":
                for n, rows in (("q", H * Dk), ("k", G * Dk), ("v", G * Dv), ("o", W)):
                    t[p + f"mix.{n}.b"] = around(rows, 0.0, 0.4)
                t[p + "mix.q.norm"], t[p + "mix.k.norm"] = around(Dk, 1.0, 0.3), around(Dk, 1.0, 0.3)
        mlp = layer["mlp"]
        if mlp is None:
            del t[p + "norm2"], t[p + "norm2.b"]
        elif mlp["kind"] == "dense":
            t[p + "mlp.up"], t[p + "mlp.down"] = mat(mlp["ff"], W, 1.6), mat(W, mlp["ff"], 1.0)
        else:
            E = mlp["router"]["experts"]
            t[p + "mlp.router"] = mat(E, W, 2.0)
            for e in range(E):
                glu(p + f"mlp.e{e}.", mlp["expert"]["ff"])
            if "shared" in mlp:
                glu(p + "mlp.shared.", mlp["shared"]["ff"])
    return {k: v.to(torch.bfloat16).contiguous() for k, v in t.items()}


def write_folder(cfg: dict, weights: dict[str, torch.Tensor]) -> str:
    d = tempfile.mkdtemp(prefix="me_gevulorn_")
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous() for k, v in weights.items()}, os.path.join(d, "model.safetensors"))
    return d


@functools.lru_cache(maxsize=None)
def folder(name: str) -> str:
    cfg, seed, _ = ALL[name]
    return write_folder(cfg, tensors(cfg, seed, RANKS[name]))
