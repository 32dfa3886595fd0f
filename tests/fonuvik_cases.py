"""Small Fonuvik configurations for the tests, and random weights for them under the checkpoint's names.

The cases differ from one another in every size and option: the order of the layer kinds (a parallel layer first, two of
a kind in a row, one kind only), heads and kv heads (also equal, also one), key and value widths (unequal, equal, not
multiples of 8), the part of a head that is turned and whether its frequencies are rescaled (or no rotation at all), the
block of positions a query sees (smaller than a page, not a multiple of one, larger than any prompt, none), the inner
widths of the two narrow projections (multiples of 8, which run as products, and others), tau, the number of experts and
how many a token runs (one, some, all), a shared expert or none, a layer without a feed-forward, and the two branch
weights (also 1, which a fault that drops them would hide at other values only).
"""
from __future__ import annotations

import copy
import os
from typing import Dict

import torch


def moe(experts, top, ff, shared=None):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}, "shared": {"ff": shared} if shared else None}


def wkv(heads, dim, mlp):
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim}, "mlp": mlp}


def parallel(left, right, mlp, left_scale=1.3, right_scale=0.7, rot=None, block=None, scale=None):
    lh, lg, ld, lv = left
    rh, rd, rv, tau = right
    l = {"heads": lh, "kv_heads": lg, "dim": ld, "vdim": lv, "scale": scale or ld ** -0.5 * 4.0}
    if rot:
        l["rot"] = rot
    if block:
        l["mask"] = {"size": block}
    return {"type": "parallel", "mixer": {"left": l, "right": {"heads": rh, "dim": rd, "vdim": rv, "tau": tau},
                                           "left_scale": left_scale, "right_scale": right_scale}, "mlp": mlp}


SLOW = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 48}
CASES = {
    # a parallel layer first, then the recurrence, a layer without a feed-forward; unequal widths everywhere; a block of
    # positions that is no multiple of a page; inner widths that run inside the kernels
    "a": {"architecture": "Fonuvik", "vocab": 210, "width": 64, "norm": {"eps": 1e-5},
          "layers": [parallel((4, 2, 16, 24), (3, 8, 12, 7.0), moe(5, 2, 24, 40), rot={"base": 5000.0, "dims": 12, "scaling": SLOW}, block=21),
                     wkv(3, 24, moe(5, 2, 24, 40)),
                     parallel((4, 2, 16, 24), (3, 8, 12, 7.0), None, rot={"base": 5000.0, "dims": 12, "scaling": SLOW}, block=21)],
          "ranks": (5, 6)},
    # sizes that are not multiples of 8; one kv head for three query heads; equal key and value widths on the left; both
    # branch weights 1; plain frequencies over the whole head; a block smaller than a page; one expert a token, none shared;
    # two recurrence layers in a row
    "b": {"architecture": "Fonuvik", "vocab": 333, "width": 72, "norm": {"eps": 1e-3},
          "layers": [wkv(2, 20, moe(3, 1, 36)),
                     wkv(2, 20, moe(3, 1, 36)),
                     parallel((3, 1, 12, 12), (1, 20, 10, 1.0), moe(3, 1, 36), left_scale=1.0, right_scale=1.0,
                              rot={"base": 100.0, "dims": 12, "scaling": None}, block=5)],
          "ranks": (3, 9)},
    # sizes the tensor-core kernels like (heads of 64 on the left, 64 / 64 on the right); inner widths that run as products;
    # every expert runs for every token; a block of several pages
    "c": {"architecture": "Fonuvik", "vocab": 256, "width": 128, "norm": {"eps": 2e-6},
          "layers": [wkv(2, 64, moe(4, 4, 64, 128)),
                     parallel((4, 2, 64, 64), (2, 64, 64, 16.0), moe(4, 4, 64, 128), left_scale=0.8, right_scale=1.1,
                              rot={"base": 5e5, "dims": 32, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 128}}, block=96),
                     parallel((4, 2, 64, 64), (2, 64, 64, 16.0), moe(4, 4, 64, 128), left_scale=0.8, right_scale=1.1,
                              rot={"base": 5e5, "dims": 32, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 128}}, block=96)],
          "ranks": (16, 8)},
    # parallel layers only; one head each side; no rotation; no block (plain causal attention); wide keys on the right
    # (several registers a lane)
    "d": {"architecture": "Fonuvik", "vocab": 150, "width": 48, "norm": {"eps": 1e-5},
          "layers": [parallel((1, 1, 40, 16), (1, 136, 40, 30.0), moe(2, 2, 16, 24), left_scale=2.0, right_scale=0.25),
                     parallel((1, 1, 40, 16), (1, 136, 40, 30.0), moe(2, 2, 16, 24), left_scale=2.0, right_scale=0.25)],
          "ranks": (7, 4)},
    # recurrence layers only, heads times dim wider than the stream; many experts
    "e": {"architecture": "Fonuvik", "vocab": 120, "width": 40, "norm": {"eps": 1e-5},
          "layers": [wkv(5, 16, moe(9, 3, 16, 8)), wkv(5, 16, None)],
          "ranks": (8, 24)},
    # wide heads: keys of 80 beside values of 160 on the left (stored at 256 on the tensor-core kernels), all of a head
    # turned; a block larger than any prompt of the tests
    "f": {"architecture": "Fonuvik", "vocab": 130, "width": 96, "norm": {"eps": 1e-6},
          "layers": [parallel((2, 1, 80, 160), (2, 24, 48, 4.0), moe(4, 2, 32, 64), left_scale=0.9, right_scale=0.8,
                              rot={"base": 2000.0, "dims": 80, "scaling": None}, block=4096),
                     wkv(3, 32, moe(4, 2, 32, 64))],
          "ranks": (8, 16)},
}


def raw_config(key: str) -> dict:
    raw = copy.deepcopy(CASES[key])
    raw.pop("ranks")
    return raw


def random_weights(raw: dict, seed: int, ranks=(5, 6)) -> Dict[str, torch.Tensor]:
    """Random float32 tensors under the checkpoint's names; `ranks` = inner widths of (the decay of the linear attention,
    the decay of the token-shift recurrence)."""
    g = torch.Generator().manual_seed(seed)
    W = raw["width"]
    normal = lambda *shape, std=1.0: torch.randn(*shape, generator=g) * std
    proj = lambda rows, cols=W: normal(rows, cols, std=cols ** -0.5)
    out = {"embed": normal(raw["vocab"], W), "embed.norm": 1 + normal(W, std=0.1), "final.norm": 1 + normal(W, std=0.1)}
    for i, layer in enumerate(raw["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        out[p + "norm1"], out[p + "norm1b"] = 1 + normal(W, std=0.1), 1 + normal(W, std=0.1)
        if layer["type"] == "parallel":
            l, q = m["left"], p + "mix.left."
            H, G, dk, dv = l["heads"], l["kv_heads"], l["dim"], l["vdim"]
            out[q + "q"], out[q + "k"], out[q + "v"], out[q + "o"] = proj(H * dk), proj(G * dk), proj(G * dv), proj(W, H * dv)
            r, q = m["right"], p + "mix.right."
            H, dk, dv, rank = r["heads"], r["dim"], r["vdim"], r.get("a_rank", ranks[0])
            out[q + "q"], out[q + "k"], out[q + "v"], out[q + "g"] = proj(H * dk), proj(H * dk), proj(H * dv), proj(H * dv)
            out[q + "a1"], out[q + "a2"], out[q + "a2.b"] = proj(rank), proj(H * dk, rank) * 2.0, normal(H * dk, std=1.0) + 2.0
            out[q + "norm"], out[q + "o"] = 1 + normal(dv, std=0.1), proj(W, H * dv)
        else:
            q, H, d, rank = p + "mix.", m["heads"], m["dim"], m.get("w_rank", ranks[1])
            for s in "rkvgw":
                out[q + "mu." + s] = torch.rand(W, generator=g)
            for s in "rkvg":
                out[q + s] = proj(H * d)
            out[q + "w1"], out[q + "w2"], out[q + "w0"] = proj(rank), proj(H * d, rank) * 2.0, normal(H * d, std=1.0) - 2.0
            out[q + "u"], out[q + "norm"], out[q + "o"] = normal(H, d, std=0.5), 1 + normal(H * d, std=0.1), proj(W, H * d)
        mlp = layer.get("mlp")
        if mlp:
            q, ff = p + "mlp.", mlp["expert"]["ff"]
            out[p + "norm2"], out[p + "norm2b"] = 1 + normal(W, std=0.1), 1 + normal(W, std=0.1)
            out[q + "router"], out[q + "router.b"] = proj(mlp["router"]["experts"]) * 2.0, normal(mlp["router"]["experts"], std=0.5)
            for e in range(mlp["router"]["experts"]):
                out[f"{q}e{e}.gate"], out[f"{q}e{e}.up"], out[f"{q}e{e}.down"] = proj(ff), proj(ff), proj(W, ff)
            if mlp.get("shared"):
                sf = mlp["shared"]["ff"]
                out[q + "shared.gate"], out[q + "shared.up"], out[q + "shared.down"] = proj(sf), proj(sf), proj(W, sf)
    return out


def case(key: str, seed: int = 0, sharp: float = 1.0):
    """(raw config as config.json holds it, weights).  `sharp` multiplies the scale of every softmax, which makes it
    peaky: single keys, far back or at an edge, then carry a position's output."""
    raw = raw_config(key)
    for layer in raw["layers"]:
        if layer["type"] == "parallel":
            layer["mixer"]["left"]["scale"] *= sharp
    return raw, random_weights(raw, seed or (len(key) + ord(key[0])), CASES[key]["ranks"])


def with_ranks(raw: dict, weights: Dict[str, torch.Tensor]) -> dict:
    from microllm_rocm_b200.config.fonuvik import sizes_from_tensors
    return sizes_from_tensors(raw, {n: tuple(t.shape) for n, t in weights.items()})


def write_folder(folder: str, raw: dict, weights: Dict[str, torch.Tensor], storage: torch.dtype = torch.float32) -> str:
    import json

    from microllm_rocm_b200.weights.safetensors import save_file
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(raw, f)
    save_file({n: t.to(storage).contiguous() for n, t in weights.items()}, os.path.join(folder, "model.safetensors"), metadata={"format": "pt"})
    return folder
