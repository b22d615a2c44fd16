"""Small Mobatar configurations for the tests, as config.json dictionaries, and a writer of model folders with
random weights that the tests may tune.

M1 mixes everything: attention with a sink whose values are wider than its keys, a side-by-side layer (chunks of 24
positions beside retention with three unequal decays), latent attention with a window of 20 and a rotated part, a
layer without feed-forward, and layers that run with earlier layers' weights - one of them in the middle.
M2 has sizes the tensor-core attention kernels take (heads of 64 and 128, values of the keys' size), a latent row of
128, retention heads of 64 x 64, chunks and a window that are whole pages.
M3 has values that are 1 or absent elsewhere: one head, one key head per query head, no pair-hash table, no frequency
scaling, a rotation of the whole head or none, scales of 1, a window of one position and a chunk of two, a latent
without a rotated part, a retention head that never decays.
M4 has sizes that are no multiple of 8 anywhere, a chunk and a window that are no multiple of the page, and a first
layer that runs with the weights of a later one.
"""
import json
import os

import torch


def rot(dims, base, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling is not None:
        r["scaling"] = scaling
    return r


def llama3(factor, original, low, high):
    return {"factor": factor, "original": original, "low": low, "high": high}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def attention(heads, kv_heads, dim, vdim, rotation, scale, mlp):
    return {"type": "attention", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": rotation, "scale": scale}}


def latent(heads, dim, rot_dim, vdim, rank, window, base, scale, mlp):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale,
         "rot": rot(rot_dim, base), "mask": {"size": window}}
    return {"type": "latent_attention", "mlp": mlp, "mixer": m}


def side_by_side(left, right, left_scale, right_scale, mlp):
    return {"type": "parallel", "mlp": mlp,
            "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}}


def chunked(heads, kv_heads, dim, vdim, rotation, scale, chunk):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": rotation, "scale": scale,
            "mask": {"size": chunk}}


def retention(heads, dim, vdim, decay, rotation):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay), "rot": rotation}


def again(layer, j):
    """The entry of a layer that runs with layer j's weights: the same sizes, and ``weights_of``."""
    out = json.loads(json.dumps(layer))
    out["weights_of"] = j
    return out


def _m1():
    a = attention(4, 2, 24, 40, rot(24, 10000.0, llama3(5.0, 64, 1.0, 3.0)), 0.15, dense(136, 1.5))
    p = side_by_side(chunked(6, 3, 16, 8, rot(16, 50000.0, {"factor": 2.0}), 0.25, 24),
                     retention(3, 20, 12, (0.8, 0.97, 0.999), rot(12, 1000.0)), 1.3, 0.7, dense(72, 2.0))
    la = latent(3, 12, 8, 20, 24, 20, 3000.0, 0.22, None)
    return {"architecture": "Mobatar", "vocab": 300, "width": 96, "norm": {"eps": 1e-5},
            "embedding": {"bigram": {"buckets": 101, "mul_prev": 31, "mul_cur": 7}},
            "layers": [a, p, again(a, 0), la, again(p, 1), again(la, 3)]}


def _m2():
    a = attention(8, 2, 64, 64, rot(64, 500000.0, llama3(8.0, 128, 1.0, 4.0)), 0.18, dense(192, 2.0))
    p = side_by_side(chunked(4, 1, 128, 128, rot(128, 10000.0, {"factor": 4.0}), 0.09, 48),
                     retention(2, 64, 64, (0.9, 0.995), rot(64, 100000.0)), 1.25, 0.85, dense(128, 1.0))
    la = latent(4, 32, 16, 48, 112, 32, 200000.0, 0.15, dense(128, 2.5))
    return {"architecture": "Mobatar", "vocab": 260, "width": 128, "norm": {"eps": 1e-6},
            "embedding": {"bigram": {"buckets": 64, "mul_prev": 5, "mul_cur": 3}},
            "layers": [p, a, la, again(p, 0)]}


def _m3():
    a = attention(1, 1, 16, 16, rot(16, 7.0), 0.4, dense(32, 0.7))
    p = side_by_side(chunked(2, 2, 32, 16, None, 0.2, 2), retention(1, 32, 16, (1.0,), None), 1.0, 1.0, None)
    la = latent(1, 16, 0, 16, 8, 1, 10.0, 0.3, dense(64, 3.0))
    la["mixer"]["rot"] = None
    return {"architecture": "Mobatar", "vocab": 200, "width": 64, "norm": {"eps": 1e-6}, "layers": [a, p, la]}


def _m4():
    a = attention(5, 5, 18, 11, rot(10, 777.0, llama3(3.0, 40, 1.5, 6.0)), 0.33, dense(52, 1.1))
    p = side_by_side(chunked(3, 1, 22, 36, rot(6, 123.0, {"factor": 3.0}), 0.2, 19),
                     retention(5, 9, 7, (0.6, 0.7, 0.8, 0.9, 0.99), rot(4, 50.0)), 0.6, 1.7, dense(20, 0.9))
    la = latent(5, 10, 6, 9, 13, 27, 999.0, 0.27, dense(12, 2.0))
    return {"architecture": "Mobatar", "vocab": 173, "width": 76, "norm": {"eps": 1e-5},
            "embedding": {"bigram": {"buckets": 17, "mul_prev": 1, "mul_cur": 1}},
            "layers": [again(la, 2), a, la, p]}                  # the first entry borrows from a LATER layer


M1, M2, M3, M4 = _m1(), _m2(), _m3(), _m4()

# Standard deviations (by the last part of a tensor's slot) that make every mechanism matter in a random model:
# projections whose results are of order one, biases that reach the caps, output projections that weigh as much as
# the stream, a second embedding table as large as the first.
LIVELY = {"weight": 0.5, "pairs": 0.5, "q": 0.12, "k": 0.12, "v": 0.12, "g": 0.15, "o": 0.1, "dkv": 0.12, "uk": 0.2, "uv": 0.2,
          "up": 0.12, "gate": 0.12, "down": 0.1, "b": 0.4}


def tune_norms(tensors):
    """Weights that differ from their neutral value, so that a norm left out, or a gain of w instead of 1 + w, shows."""
    for name, t in tensors.items():
        leaf = name.split(".")[-1]
        if leaf in ("norm1", "norm2") or name == "final.norm":                 # stored around zero
            g = torch.Generator().manual_seed(len(name) * 131 + t.numel())
            t.copy_((0.3 * torch.randn(t.shape, generator=g)).to(t.dtype))
        elif leaf == "norm" and t.dim() == 1:                                  # plain weights
            g = torch.Generator().manual_seed(len(name) * 137 + t.numel())
            t.copy_((1.0 + 0.3 * torch.randn(t.shape, generator=g)).to(t.dtype))


def write_model(model_dir, raw, seed, tune=None, dtype=torch.bfloat16):
    """config.json + model.safetensors with random weights (the package's own generator and writer);
    ``tune(tensors)`` may change them before they are written.  Returns {name: tensor}."""
    from nanoinfer_b200.config import config_from_dict
    from nanoinfer_b200.weights.plan import tensor_plan
    from nanoinfer_b200.weights.random_init import random_tensors
    from nanoinfer_b200.weights.safetensors_io import write_safetensors
    cfg = config_from_dict(raw)
    std = {p.slot: LIVELY[p.slot.split(".")[-1]] for p in tensor_plan(cfg) if p.slot.split(".")[-1] in LIVELY}
    tensors = dict(random_tensors(cfg, seed, 0.05, dtype, std))
    tune_norms(tensors)
    if tune is not None:
        tune(tensors)
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(raw, f)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors.items())
    return tensors
