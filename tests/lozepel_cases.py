"""Small Lozepel configurations for the tests, and random weights for them under the checkpoint's names.

The cases differ from one another in every size and option: the order of the layer kinds (each kind first somewhere, two of
a kind in a row), heads and kv heads (also equal, also one), key and value widths (unequal, equal, not multiples of 8,
wider than 128), the part of a head that is turned (a part, all, none), a cap on the scores or none, a layer that reads
another layer's keys and values (one reader, two readers, none), decays (also exactly 1), branch weights (also 1), the
clamp of the dense feed-forward (tight enough to bite, and so wide that it never does), the number of experts, how many
a token runs (one, some, all outputs) and how many router outputs pass the input on (none, one, several), a layer without
a feed-forward, the pair table's size and multipliers, a cap on the logits or none, eps from 1e-3 to 1e-6.
"""
from __future__ import annotations

import copy
import os
from typing import Dict

import torch


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts, top, ff, identity=0):
    return {"kind": "moe", "router": {"experts": experts, "top": top, "identity": identity}, "expert": {"ff": ff}}


def attention(heads, kv_heads, dim, mlp, rot=None, scale=None):
    return {"type": "attention", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale or dim ** -0.5 * 3.0, "rot": rot}}


def capped(heads, kv_heads, dim, vdim, mlp, rot=None, scale=None, softcap=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or 6.0, "softcap": softcap, "rot": rot}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention_2", "mixer": m, "mlp": mlp}


def parallel(left, right, mlp, left_scale=1.3, right_scale=0.7, scale=None):
    lh, lg, ld, lv = left
    rh, rd, rv, decay = right
    return {"type": "parallel", "mlp": mlp,
            "mixer": {"left": {"heads": lh, "kv_heads": lg, "dim": ld, "vdim": lv, "scale": scale or 4.0 * ld ** -0.5},
                      "right": {"heads": rh, "dim": rd, "vdim": rv, "decay": list(decay)}, "left_scale": left_scale, "right_scale": right_scale}}


def model(vocab, width, eps, layers, bigram, cap):
    raw = {"architecture": "Lozepel", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers, "logit_softcap": cap}
    if bigram:
        raw["embedding"] = {"bigram": {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}}
    return raw


CASES = {
    # every kind once and a reader of another layer's keys and values without a feed-forward; part of a head turned;
    # unequal widths everywhere; a clamp that bites; one pass-through output
    "a": model(210, 64, 1e-5, [attention(4, 2, 16, dense(40, 0.4), rot={"base": 5000.0, "dims": 12}),
                               parallel((4, 2, 16, 24), (3, 8, 12, (0.5, 0.9, 0.99)), moe(5, 2, 24, identity=1)),
                               capped(3, 1, 24, 16, moe(5, 2, 24, identity=1), rot={"base": 300.0, "dims": 24}, softcap=5.0),
                               capped(3, 1, 24, 16, None, rot={"base": 300.0, "dims": 24}, softcap=5.0, kv_from=2)], (97, 13, 5), 8.0),
    # a parallel layer first; sizes that are not multiples of 8; one head; no rotation anywhere; no cap on scores or logits;
    # a decay of exactly 1; branch weights 1; a clamp that never bites; every router output runs (top = experts + identity);
    # one expert a token in the last layer, nothing passes through there
    "b": model(333, 72, 1e-3, [parallel((3, 1, 12, 12), (1, 20, 10, (1.0,)), moe(2, 4, 36, identity=2), left_scale=1.0, right_scale=1.0),
                               capped(1, 1, 20, 28, dense(30, 1e4)),
                               attention(3, 3, 12, moe(3, 1, 36))], (11, 7, 3), None),
    # sizes the tensor-core kernels like (heads of 64); two readers of one layer's keys and values, with layers of other kinds
    # between; all of a head turned; two of a kind in a row
    "c": model(256, 128, 2e-6, [capped(4, 2, 64, 64, moe(4, 2, 64, identity=2), rot={"base": 2e5, "dims": 64}, softcap=12.0),
                                attention(4, 1, 64, dense(96, 1.0), rot={"base": 1e4, "dims": 32}),
                                capped(4, 2, 64, 64, moe(4, 2, 64, identity=2), rot={"base": 2e5, "dims": 64}, softcap=12.0, kv_from=0),
                                parallel((4, 2, 64, 64), (2, 64, 64, (0.9, 0.999)), moe(4, 2, 64, identity=2), left_scale=0.8, right_scale=1.1),
                                capped(4, 2, 64, 64, None, rot={"base": 2e5, "dims": 64}, softcap=12.0, kv_from=0)], (251, 17, 9), 25.0),
    # wide heads: keys of 40 beside values of 136, an attention layer of 80; wide keys in the linear attention; no pair table
    "d": model(150, 48, 1e-6, [attention(2, 1, 80, None, rot={"base": 2000.0, "dims": 80}),
                               capped(2, 2, 40, 136, dense(24, 2.0), softcap=3.0),
                               parallel((1, 1, 40, 16), (1, 136, 40, (0.95,)), moe(2, 1, 16, identity=1), left_scale=2.0, right_scale=0.25)],
               None, 15.0),
}


def raw_config(key: str) -> dict:
    return copy.deepcopy(CASES[key])


def random_weights(raw: dict, seed: int, sink: float = 1.0) -> Dict[str, torch.Tensor]:
    """Random float32 tensors under the checkpoint's names.  Sinks are drawn around `sink`: large enough that leaving one
    out, scaling it or capping it shows in the logits."""
    g = torch.Generator().manual_seed(seed)
    W = raw["width"]
    normal = lambda *shape, std=1.0: torch.randn(*shape, generator=g) * std
    proj = lambda rows, cols=W: normal(rows, cols, std=cols ** -0.5)
    out = {"embed": normal(raw["vocab"], W), "final.norm": normal(W, std=0.1), "head": proj(raw["vocab"]) * 3.0}
    bg = (raw.get("embedding") or {}).get("bigram")
    if bg:
        out["bigram"] = normal(bg["buckets"] + 1, W)
    for i, layer in enumerate(raw["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        out[p + "norm1"], out[p + "norm1b"] = normal(W, std=0.1), normal(W, std=0.1)
        if layer["type"] == "attention":
            q, H, G, d = p + "mix.", m["heads"], m["kv_heads"], m["dim"]
            out[q + "q"], out[q + "k"], out[q + "q.b"], out[q + "k.b"] = proj(H * d), proj(G * d), normal(H * d, std=0.5), normal(G * d, std=0.5)
            out[q + "g"], out[q + "o"] = proj(H) * 2.0, proj(W, H * d)
        elif layer["type"] == "attention_2":
            q, H, G, dk, dv = p + "mix.", m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out[q + "q"], out[q + "sink"], out[q + "o"] = proj(H * dk), normal(H, std=1.0) + sink, proj(W, H * dv)
            if m.get("kv_from") is None:
                out[q + "k"], out[q + "v"] = proj(G * dk), proj(G * dv)
        else:
            l, q = m["left"], p + "mix.left."
            H, G, dk, dv = l["heads"], l["kv_heads"], l["dim"], l["vdim"]
            out[q + "q"], out[q + "k"], out[q + "v"], out[q + "o"] = proj(H * dk), proj(G * dk), proj(G * dv), proj(W, H * dv)
            out[q + "q.norm"], out[q + "k.norm"] = 1 + normal(H * dk, std=0.2), 1 + normal(G * dk, std=0.2)
            out[q + "sink"], out[q + "g"] = normal(H, std=1.0) + sink, proj(H) * 2.0
            r, q = m["right"], p + "mix.right."
            H, dk, dv = r["heads"], r["dim"], r["vdim"]
            out[q + "q"], out[q + "k"], out[q + "v"], out[q + "g"] = proj(H * dk), proj(H * dk), proj(H * dv), proj(H * dv)
            out[q + "norm"], out[q + "o"] = 1 + normal(H * dv, std=0.1), proj(W, H * dv)
        mlp = layer.get("mlp")
        if not mlp:
            continue
        q = p + "mlp."
        out[p + "norm2"], out[p + "norm2b"] = normal(W, std=0.1), normal(W, std=0.1)
        if mlp["kind"] == "dense":
            out[q + "gate"], out[q + "up"], out[q + "down"] = proj(mlp["ff"]), proj(mlp["ff"]), proj(W, mlp["ff"])
        else:
            E, N, ff = mlp["router"]["experts"], mlp["router"]["experts"] + mlp["router"].get("identity", 0), mlp["expert"]["ff"]
            out[q + "router"], out[q + "correction"] = proj(N) * 2.0, normal(N, std=0.3)
            for e in range(E):
                out[f"{q}e{e}.gate"], out[f"{q}e{e}.up"], out[f"{q}e{e}.down"] = proj(ff), proj(ff), proj(W, ff)
    return out


def case(key: str, seed: int = 0, sharp: float = 1.0, sink: float = 1.0):
    """(raw config as config.json holds it, weights).  `sharp` multiplies the scale of every softmax, which makes it
    peaky: single keys, far back or at a page's border, then carry a position's output."""
    raw = raw_config(key)
    for layer in raw["layers"]:
        m = layer["mixer"]
        for part in ([m["left"]] if layer["type"] == "parallel" else [m]):
            part["scale"] *= sharp
            if part.get("softcap"):
                part["softcap"] *= sharp
    return raw, random_weights(raw, seed or (len(key) + ord(key[0])), sink)


def write_folder(folder: str, raw: dict, weights: Dict[str, torch.Tensor], storage: torch.dtype = torch.float32) -> str:
    import json

    from microllm_rocm_b200.weights.safetensors import save_file
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(raw, f)
    save_file({n: t.to(storage).contiguous() for n, t in weights.items()}, os.path.join(folder, "model.safetensors"), metadata={"format": "pt"})
    return folder
