"""Small Tazulix configurations for the tests, as config.json dictionaries, and a writer of model folders with
random weights that the tests may tune.

T1 mixes everything: attention with values wider than keys and two query heads per key head, a partly rotated
head with ramp-scaled frequencies, lightning layers with three heads of unequal decay, a dense unit, routed units
with and without a shared unit, a layer without feed-forward, a looped span in the middle.
T2 has sizes the tensor-core attention kernels take (heads of 64 and 128, values of the keys' size, four query
heads per key head), a span of two layers that starts the model and runs three times, a lightning layer of 64 x 64.
T3 has values that are 1 or absent elsewhere: one head, no rotation or a full one without scaling, no loop, no
embedding scale, top 1 without a shared unit, one lightning head that never decays, a value size of one page row.
T4 has sizes that are no multiple of 8 anywhere, a span that ends the model, and a top that takes every expert.
"""
import json
import os

import torch


def rot(dims, base, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling is not None:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def attention(heads, kv_heads, dim, vdim, rotation, scale, mlp):
    return {"type": "attention", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": rotation, "scale": scale}}


def lightning(heads, dim, vdim, decay, mlp):
    return {"type": "lightning", "mlp": mlp, "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, limit, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        m["shared"] = {"ff": shared[0], "limit": shared[1]}
    return m


T1 = {"architecture": "Tazulix", "vocab": 300, "width": 96, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0},
      "loop": {"start": 1, "stop": 4, "times": 2},
      "layers": [attention(4, 2, 24, 40, rot(12, 10000.0, (4.0, 64, 16.0, 2.0)), 0.3, dense(136)),
                 lightning(3, 20, 12, (0.8, 0.97, 0.999), moe(5, 2, 40, 0.8, (24, 1.2))),
                 attention(6, 3, 16, 8, rot(16, 50000.0), 0.25, None),
                 attention(2, 1, 40, 40, rot(8, 100.0, (2.0, 32, 8.0, 1.0)), 0.2, moe(6, 3, 24, 1.5)),
                 lightning(2, 8, 24, (0.5, 0.9), dense(72))]}
T2 = {"architecture": "Tazulix", "vocab": 260, "width": 128, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.5},
      "loop": {"start": 0, "stop": 2, "times": 3},
      "layers": [attention(8, 2, 64, 64, rot(32, 500000.0, (8.0, 128, 4.0, 1.0)), 0.18, moe(8, 3, 64, 1.0, (64, 2.0))),
                 lightning(2, 64, 64, (0.9, 0.995), dense(192)),
                 attention(4, 1, 128, 128, rot(128, 10000.0), 0.09, dense(128))]}
T3 = {"architecture": "Tazulix", "vocab": 200, "width": 64, "norm": {"eps": 1e-6},
      "layers": [attention(1, 1, 16, 16, None, 0.4, moe(4, 1, 32, 0.7)),
                 lightning(1, 32, 16, (1.0,), None),
                 attention(2, 1, 32, 16, rot(32, 3.0), 0.2, dense(64))]}
T4 = {"architecture": "Tazulix", "vocab": 173, "width": 76, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
      "loop": {"start": 1, "stop": 3, "times": 2},
      "layers": [lightning(5, 9, 7, (0.6, 0.7, 0.8, 0.9, 0.99), moe(3, 3, 12, 0.9, (20, 0.5))),
                 attention(5, 5, 20, 12, rot(10, 777.0, (3.0, 40, 6.0, 1.5)), 0.33, moe(3, 2, 12, 1.1)),
                 attention(3, 1, 36, 36, rot(36, 10000.0), 0.2, dense(52))]}

# Standard deviations that make every mechanism matter in a random model: projections whose results are of order
# one, biases that count, routers that choose firmly (so that few choices hang on a rounding), output projections
# that weigh as much as the stream.
LIVELY = {"weight": 0.5, "q": 0.12, "k": 0.12, "v": 0.12, "g": 0.15, "o": 0.1, "q.b": 0.3, "k.b": 0.3, "v.b": 0.3,
          "up": 0.12, "gate": 0.12, "down": 0.1, "router": 0.4, "shared.gate": 0.12, "shared.up": 0.12, "shared.down": 0.1}


def tune_norms(tensors):
    """Gains that differ from one, so that a norm left out, or the wrong gain, shows."""
    for name, t in tensors.items():
        if name.split(".")[-1] in ("norm1", "norm2", "norm") and t.dim() == 1:
            g = torch.Generator().manual_seed(len(name) * 131 + t.numel())
            t.copy_((1.0 + 0.3 * torch.randn(t.shape, generator=g)).to(t.dtype))
        if name == "loop.in":
            f = t.float()
            t.copy_((f / f.std() * 1.4 / t.shape[1] ** 0.5).to(t.dtype))          # an output of the inputs' size


def write_model(model_dir, raw, seed, slot_std=None, tune=None, dtype=torch.bfloat16):
    """config.json + model.safetensors with random weights (the package's own generator and writer);
    ``tune(tensors)`` may change them before they are written.  Returns {name: tensor}."""
    from nanoinfer_b200.config import config_from_dict
    from nanoinfer_b200.weights.plan import tensor_plan
    from nanoinfer_b200.weights.random_init import random_tensors
    from nanoinfer_b200.weights.safetensors_io import write_safetensors
    cfg = config_from_dict(raw)
    std = dict(LIVELY if slot_std is None else slot_std)
    for p in tensor_plan(cfg):
        leaf = p.slot.split(".")[-1]                      # an expert's "e3.gate" is drawn like "gate"
        if p.slot not in std and leaf in std and p.slot[0] == "e":
            std[p.slot] = std[leaf]
    tensors = dict(random_tensors(cfg, seed, 0.05, dtype, std))
    tune_norms(tensors)
    if tune is not None:
        tune(tensors)
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(raw, f)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors.items())
    return tensors
