"""Small Zuzelorn configurations with random weights, written as model folders.

The sizes differ from one configuration to the next in everything: width, heads
and groups, key and value head sizes (equal and unequal, multiples of 16 and
not), layers with and without a feed-forward, layers that read an earlier
layer's keys and values, scale, eps, logit scale (also exactly 1).  The weights
are drawn here, on the host, so that the sinks, the heads' factors, the gates and
the norms' alphas all matter: a part that is left out changes the logits by far
more than any tolerance.
"""
import json
import os
import tempfile

import torch


def attn(heads, kv_heads, dim, vdim, scale, kv_from=None, ff=None):
    m = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "scale": scale, "vdim": vdim}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": {"ff": ff, "kind": "dense"} if ff else None}


def config(width, vocab, max_positions, layers, eps=1e-5, logit_scale=1.0):
    return {"architecture": "Zuzelorn", "layers": layers, "logit_scale": logit_scale,
            "max_positions": max_positions, "norm": {"eps": eps}, "vocab": vocab, "width": width}


# unequal key and value sizes, a layer without a feed-forward, two readers of other layers
ZA = config(64, 130, 400, [attn(4, 2, 16, 32, 0.3, ff=96), attn(4, 2, 16, 32, 0.3, kv_from=0, ff=80),
                           attn(4, 2, 16, 32, 0.25), attn(4, 2, 16, 32, 0.25, kv_from=2, ff=96)],
            eps=1e-6, logit_scale=0.7)
# heads of 64: the tensor-core prefill kernel and the one-chunk decode kernel; one KV head;
# two layers read the same layer's keys and values
ZB = config(128, 300, 700, [attn(4, 1, 64, 64, 0.11, ff=200), attn(4, 1, 64, 64, 0.13, ff=136),
                            attn(4, 1, 64, 64, 0.13, kv_from=1, ff=200), attn(4, 1, 64, 64, 0.2, kv_from=1)],
            eps=1e-5, logit_scale=1.0)
# heads of 128, as many KV heads as heads: the decode kernel that makes q, k and v itself
ZC = config(96, 211, 1100, [attn(2, 2, 128, 128, 0.08, ff=136), attn(2, 2, 128, 128, 0.08, kv_from=0, ff=72)],
            eps=3e-6, logit_scale=1.9)
# multiples of nothing: width 50, heads of 24 keys and 40 values, groups of 3
ZD = config(50, 101, 260, [attn(6, 2, 24, 40, 0.2, ff=70), attn(3, 3, 8, 8, 0.4, ff=30),
                           attn(6, 2, 24, 40, 0.2, kv_from=0)], eps=1e-4, logit_scale=0.5)
# heads of 128 values in groups of 4, keys of 64: unequal sizes at the tensor-core kernels' sizes
ZE = config(128, 257, 600, [attn(8, 2, 64, 128, 0.1, ff=192), attn(8, 2, 128, 128, 0.09, ff=192),
                            attn(8, 2, 128, 128, 0.09, kv_from=1, ff=64)], eps=1e-5, logit_scale=0.8)

CONFIGS = {"ZA": ZA, "ZB": ZB, "ZC": ZC, "ZD": ZD, "ZE": ZE}
SEEDS = {"ZA": 11, "ZB": 12, "ZC": 13, "ZD": 14, "ZE": 15}


def tensor_shapes(c):
    W, V = c["width"], c["vocab"]
    t = {"embed": (V, W), "pos": (c["max_positions"], W), "head": (V, W)}

    def norm(name):
        t[name] = (W,)
        t[name + ".b"] = (W,)
        t[name + ".alpha"] = ()

    for i, layer in enumerate(c["layers"]):
        L, m = f"l{i}", layer["mixer"]
        norm(L + ".norm1")
        norm(L + ".norm1b")
        H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        mats = {"q": (H * D, W), "o": (W, H * Dv)}
        if "kv_from" not in m:
            mats.update({"k": (G * D, W), "v": (G * Dv, W)})
        for n, s in mats.items():
            t[f"{L}.mix.{n}"] = s
            t[f"{L}.mix.{n}.b"] = (s[0],)
        t[L + ".mix.temp"] = (H,)
        t[L + ".mix.sink"] = (H,)
        t[L + ".rg1"] = (W, W)
        t[L + ".rg1.b"] = (W,)
        if layer["mlp"] is not None:
            norm(L + ".norm2")
            norm(L + ".norm2b")
            t[L + ".mlp.up"] = (layer["mlp"]["ff"], W)
            t[L + ".mlp.down"] = (W, layer["mlp"]["ff"])
            t[L + ".mlp.act"] = (4,)
            t[L + ".rg2"] = (W, W)
            t[L + ".rg2.b"] = (W,)
    norm("final.norm")
    return t


def random_weights(c, seed):
    """bfloat16 weights whose every part shows in the logits."""
    g = torch.Generator().manual_seed(seed)
    W = c["width"]
    out = {}
    for name, shape in tensor_shapes(c).items():
        r = torch.randn(shape, generator=g)
        leaf = name.split(".")[-1]
        if name.endswith(".alpha"):
            v = 0.6 + 0.2 * r
        elif leaf == "b" and ".norm" in name:
            v = 0.1 * r
        elif leaf == "b":
            v = 0.3 * r
        elif ".norm" in name:
            v = 1.0 + 0.2 * r
        elif leaf == "temp":
            v = 1.0 + 0.3 * r.abs()
        elif leaf == "sink":
            v = 0.5 + r
        elif leaf == "act":
            v = 0.4 + 0.3 * r
        elif name in ("embed", "pos"):
            v = r
        else:
            v = r * (2.0 / (shape[1] ** 0.5))
        out[name] = v.to(torch.bfloat16)
    return out


_FOLDERS = {}


def write_model(c, weights, prefix="zuzelorn_"):
    from safetensors.torch import save_file
    d = tempfile.mkdtemp(prefix=prefix)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(c, f)
    save_file({k: v.contiguous() for k, v in weights.items()}, os.path.join(d, "model.safetensors"))
    return d


def model(name):
    """(folder, config, float32 weights) of the named configuration, made once."""
    if name not in _FOLDERS:
        c = CONFIGS[name]
        w = random_weights(c, SEEDS[name])
        _FOLDERS[name] = (write_model(c, w, f"zuzelorn_{name}_"), c, {k: v.float() for k, v in w.items()})
    return _FOLDERS[name]
