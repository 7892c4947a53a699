"""Small Dunavik configurations with random weights, written as model folders.

The sizes differ from one configuration to the next in everything: width, heads and
groups, plain and rotated key sizes, value sizes (multiples of 16 and not), latent
sizes, windows (shorter than a page, a page, longer than a chunk), caps, query
temperatures, layers with and without a feed-forward, the latent mixer first, in the
middle of a repeated pass or last, passes that start at layer 0, a model with no
repeated pass, a residual factor that is exactly 1.  The weights are drawn here so
that every part shows in the logits: a part left out changes them by far more than
any tolerance.
"""
import json
import os
import tempfile

import torch


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base=10000.0, dims=None, ff=None):
    m = {"dim": dim, "heads": heads, "kv_rank": kv_rank, "q_rank": q_rank,
         "rot": {"base": base, "dims": rot_dim if dims is None else dims}, "rot_dim": rot_dim,
         "scale": scale, "vdim": vdim}
    return {"type": "latent_attention", "mixer": m, "mlp": {"ff": ff, "kind": "dense"} if ff else None}


def attn(heads, kv_heads, dim, vdim, scale, window=None, softcap=None, q_temp=None, ff=None):
    m = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "scale": scale, "vdim": vdim}
    if window:
        m["mask"] = {"size": window}
    if softcap:
        m["softcap"] = softcap
    if q_temp:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return {"type": "attention", "mixer": m, "mlp": {"ff": ff, "kind": "dense"} if ff else None}


def config(width, vocab, layers, loop, eps=1e-5, mult=1.0):
    c = {"architecture": "Dunavik", "layers": layers, "norm": {"eps": eps}, "residual_mult": mult,
         "vocab": vocab, "width": width}
    if loop is not None:
        c["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return c


# the latent mixer first and last, a window shorter than a page, a layer without a feed-forward
DA = config(64, 130, [latent(4, 16, 8, 24, 40, 24, 0.2, ff=96),
                      attn(4, 2, 16, 32, 0.3, window=37, softcap=20.0, q_temp=(0.25, 16), ff=80),
                      attn(4, 2, 16, 32, 0.3, window=37, softcap=20.0, q_temp=(0.25, 16)),
                      latent(2, 8, 4, 8, 24, 16, 0.35, base=500.0, ff=64)],
            (1, 3, 2), eps=1e-6, mult=0.5)
# multiples of nothing; fewer rotated dimensions than the rotated part is long; passes that start at
# layer 0 with the latent mixer inside them; no cap and no temperature; a residual factor of 1
DB = config(50, 101, [latent(3, 10, 6, 6, 22, 14, 0.3, base=77.0, dims=4, ff=70),
                      attn(6, 2, 24, 40, 0.2, window=200, ff=30),
                      attn(3, 3, 8, 8, 0.4)],
            (0, 2, 3), eps=1e-4, mult=1.0)
# heads of 64 in one group, a window longer than a chunk; the latent mixer in the middle of the pass,
# its plain and rotated parts together as long as its values (64: whole prompts in bfloat16 then form
# keys and values per head for the tensor-core kernel)
DC = config(128, 300, [attn(4, 1, 64, 64, 0.11, window=130, softcap=50.0, q_temp=(0.4, 64), ff=200),
                       latent(2, 32, 32, 64, 96, 48, 0.09, base=100000.0, ff=136),
                       attn(4, 1, 64, 64, 0.13, window=130, softcap=50.0, q_temp=(0.4, 64), ff=72)],
            (1, 2, 2), eps=1e-5, mult=0.8)
# heads of 128, as many key/value heads as heads, a window of exactly a page, a temperature that
# grows with every position, one latent head, no window on one layer, no repeated pass at all
DD = config(96, 211, [attn(2, 2, 128, 128, 0.08, window=64, softcap=8.0, q_temp=(0.1, 1), ff=136),
                      latent(1, 24, 16, 40, 64, 32, 0.15, ff=72),
                      attn(2, 2, 128, 128, 0.08, softcap=25.0, ff=40)],
            None, eps=3e-6, mult=1.3)

CONFIGS = {"DA": DA, "DB": DB, "DC": DC, "DD": DD}
SEEDS = {"DA": 21, "DB": 22, "DC": 23, "DD": 24}


def tensor_shapes(c):
    W, V = c["width"], c["vocab"]
    t = {"embed": (V, W), "head": (V, W)}

    def norm(name):
        t[name] = (W,)
        t[name + ".b"] = (W,)

    norm("embed.norm")
    for i, layer in enumerate(c["layers"]):
        L, m = f"l{i}", layer["mixer"]
        norm(L + ".norm1")
        H, D, Dv = m["heads"], m["dim"], m["vdim"]
        if layer["type"] == "latent_attention":
            R, C, Cq = m["rot_dim"], m["kv_rank"], m["q_rank"]
            t.update({f"{L}.mix.dq": (Cq, W), f"{L}.mix.dq.norm": (Cq,), f"{L}.mix.uq": (H * (D + R), Cq),
                      f"{L}.mix.dkv": (C + R, W), f"{L}.mix.dkv.norm": (C,), f"{L}.mix.uk": (H * D, C),
                      f"{L}.mix.uv": (H * Dv, C), f"{L}.mix.g": (H * Dv, W), f"{L}.mix.o": (W, H * Dv)})
        else:
            G = m["kv_heads"]
            t.update({f"{L}.mix.q": (H * D, W), f"{L}.mix.k": (G * D, W), f"{L}.mix.v": (G * Dv, W),
                      f"{L}.mix.o": (W, H * Dv)})
        if layer["mlp"] is not None:
            t[L + ".mlp.up"] = (layer["mlp"]["ff"], W)
            t[L + ".mlp.down"] = (W, layer["mlp"]["ff"])
    norm("final.norm")
    return t


def random_weights(c, seed):
    """bfloat16 weights whose every part shows in the logits."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(c).items():
        r = torch.randn(shape, generator=g)
        leaf = name.split(".")[-1]
        if leaf == "b":
            v = 0.2 * r
        elif leaf.startswith("norm"):
            v = 1.0 + 0.2 * r
        elif name == "embed":
            v = r
        elif leaf in ("q", "k", "uq", "uk"):
            v = r * (3.0 / (shape[1] ** 0.5))          # scores that differ from key to key
        else:
            v = r * (1.5 / (shape[1] ** 0.5))
        out[name] = v.to(torch.bfloat16)
    return out


_FOLDERS = {}


def write_model(c, weights, prefix="dunavik_"):
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
        _FOLDERS[name] = (write_model(c, w, f"dunavik_{name}_"), c, {k: v.float() for k, v in w.items()})
    return _FOLDERS[name]
