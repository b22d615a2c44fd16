"""A plain, slow implementation of the Mobatar design in FP64: one function per mechanism, token by token, with Python
lists as caches.  It shares no code with the package and knows nothing of pages, slots or steps; the tests compare
the engine with it.

Notation: x is the stream, h a sublayer's input (the stream itself), w the dictionary of tensors by name.  Weights
are [out, in] and applied as W h.
"""
import math

import torch

F64 = torch.float64


def unit_rms(x, eps):
    """x divided by its root mean square, eps under the root."""
    return x / torch.sqrt((x * x).mean() + eps)


def shifted_norm(x, weight, eps):
    """RMS norm whose stored weight lies around zero: the gain is 1 + weight."""
    return unit_rms(x, eps) * (1.0 + weight)


def frequencies(rot):
    """f_i = base^(-2 i / dims); `scaling` with `original`: the three-band rule by wavelength; with a factor alone:
    all divided by it."""
    n = rot["dims"]
    f = torch.tensor([rot["base"] ** (-2.0 * i / n) for i in range(n // 2)], dtype=F64)
    sc = rot.get("scaling")
    if not sc:
        return f
    if "original" not in sc:
        return f / sc["factor"]
    out = []
    for fi in f.tolist():
        wave = 2.0 * math.pi / fi
        if wave < sc["original"] / sc["high"]:
            out.append(fi)
        elif wave > sc["original"] / sc["low"]:
            out.append(fi / sc["factor"])
        else:
            s = (sc["original"] / wave - sc["low"]) / (sc["high"] - sc["low"])
            out.append((1.0 - s) * fi / sc["factor"] + s * fi)
    return torch.tensor(out, dtype=F64)


def rotate(v, pos, freq, adjacent):
    """Rotate the first 2 len(freq) entries of the vector v by pos * freq: entry i with i + half, or 2i with 2i + 1."""
    half = len(freq)
    first = torch.arange(half) * 2 if adjacent else torch.arange(half)
    second = first + 1 if adjacent else first + half
    c, s = torch.cos(pos * freq), torch.sin(pos * freq)
    out = v.clone()
    out[first] = v[first] * c - v[second] * s
    out[second] = v[second] * c + v[first] * s
    return out


def softmax_read(scores, values, sink):
    """sum_j p_j values_j with p = softmax(scores); with `sink` the denominator has one more term, exp(0)."""
    s = torch.stack(scores)
    top = max(s.max().item(), 0.0) if sink else s.max().item()
    e = torch.exp(s - top)
    denom = e.sum() + (math.exp(-top) if sink else 0.0)
    return sum(p * v for p, v in zip((e / denom), values))


def visible(pos, j, chunk=None, window=None):
    """Whether the query at pos sees the key at j <= pos."""
    if chunk is not None and pos // chunk != j // chunk:
        return False
    if window is not None and pos - j >= window:
        return False
    return True


def sink_attention(w, pre, m, h, pos, cache, eps):
    """Grouped-query attention: rotate, then every head of q and k to unit root mean square; all earlier keys; a
    softmax with a sink."""
    H, G, D, V = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m.get("vdim", m["dim"])
    f = frequencies(m["rot"]) if m.get("rot") and m["rot"]["dims"] else None
    q, k, v = (w[pre + "q"] @ h).view(H, D), (w[pre + "k"] @ h).view(G, D), (w[pre + "v"] @ h).view(G, V)
    if f is not None:
        q = torch.stack([rotate(x, pos, f, False) for x in q])
        k = torch.stack([rotate(x, pos, f, False) for x in k])
    q = torch.stack([unit_rms(x, eps) for x in q])
    k = torch.stack([unit_rms(x, eps) for x in k])
    cache.append((k, v))
    heads = []
    for a in range(H):
        g = a // (H // G)
        heads.append(softmax_read([(q[a] @ kk[g]) * m["scale"] for kk, _ in cache], [vv[g] for _, vv in cache], True))
    return w[pre + "o"] @ torch.cat(heads)


def chunked_attention(w, pre, m, h, pos, cache, eps):
    """Grouped-query attention whose whole q and whole k pass an RMS norm with a plain weight before the rotation;
    keys of the query's own chunk only; every head's output times a sigmoid gate of the input."""
    H, G, D, V = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m.get("vdim", m["dim"])
    f = frequencies(m["rot"]) if m.get("rot") and m["rot"]["dims"] else None
    q = (unit_rms(w[pre + "q"] @ h, eps) * w[pre + "q.norm"]).view(H, D)
    k = (unit_rms(w[pre + "k"] @ h, eps) * w[pre + "k.norm"]).view(G, D)
    v = (w[pre + "v"] @ h).view(G, V)
    if f is not None:
        q = torch.stack([rotate(x, pos, f, False) for x in q])
        k = torch.stack([rotate(x, pos, f, False) for x in k])
    cache.append((k, v))
    chunk = m["mask"]["size"] if m.get("mask") else None
    seen = [j for j in range(pos + 1) if visible(pos, j, chunk=chunk)]
    gate = torch.sigmoid(w[pre + "g"] @ h)
    heads = []
    for a in range(H):
        g = a // (H // G)
        heads.append(gate[a] * softmax_read([(q[a] @ cache[j][0][g]) * m["scale"] for j in seen],
                                            [cache[j][1][g] for j in seen], False))
    return w[pre + "o"] @ torch.cat(heads)


def retention(w, pre, m, h, pos, state, eps):
    """S <- decay S + k v^T, o = S^T q per head, with rotated q and k and k / sqrt(dim); every head's o to unit root
    mean square; times silu of a gate projection.  `state` is a list with one [dim, vdim] matrix per head."""
    H, D, V = m["heads"], m["dim"], m.get("vdim", m["dim"])
    f = frequencies(m["rot"]) if m.get("rot") and m["rot"]["dims"] else None
    q, k, v = (w[pre + "q"] @ h).view(H, D), (w[pre + "k"] @ h).view(H, D), (w[pre + "v"] @ h).view(H, V)
    outs = []
    for a in range(H):
        qa, ka = (rotate(q[a], pos, f, False), rotate(k[a], pos, f, False)) if f is not None else (q[a], k[a])
        ka = ka * D ** -0.5
        state[a] = m["decay"][a] * state[a] + torch.outer(ka, v[a])
        outs.append(unit_rms(state[a].T @ qa, eps))
    z = w[pre + "g"] @ h
    return w[pre + "o"] @ (torch.cat(outs) * z * torch.sigmoid(z))


def latent_attention(w, pre, m, h, pos, cache, eps):
    """Only a normed latent c and one rotated key part are kept per token; a head's key is [W_uk c | that part], its
    value W_uv c; the last mask.size keys are visible."""
    H, D, R, V, C = m["heads"], m["dim"], m["rot_dim"], m.get("vdim", m["dim"]), m["kv_rank"]
    f = frequencies(m["rot"]) if R else None
    q = (w[pre + "q"] @ h).view(H, D + R)
    down = w[pre + "dkv"] @ h
    c = unit_rms(down[:C], eps) * w[pre + "dkv.norm"]
    shared = rotate(down[C:], pos, f, True) if R else down[C:]
    cache.append((c, shared))
    window = m["mask"]["size"] if m.get("mask") else None
    seen = [j for j in range(pos + 1) if visible(pos, j, window=window)]
    uk, uv = w[pre + "uk"].view(H, D, C), w[pre + "uv"].view(H, V, C)
    heads = []
    for a in range(H):
        qa = torch.cat([q[a, :D], rotate(q[a, D:], pos, f, True)]) if R else q[a]
        scores = [(qa @ torch.cat([uk[a] @ cache[j][0], cache[j][1]])) * m["scale"] for j in seen]
        heads.append(softmax_read(scores, [uv[a] @ cache[j][0] for j in seen], False))
    return w[pre + "o"] @ torch.cat(heads)


def capped_unit(w, pre, mlp, h):
    """Biased gate, up and down projections; the gate capped from above, up from both sides."""
    lim = mlp["limit"]
    g = torch.clamp(w[pre + "gate"] @ h + w[pre + "gate.b"], max=lim)
    u = torch.clamp(w[pre + "up"] @ h + w[pre + "up.b"], -lim, lim)
    return w[pre + "down"] @ (g * torch.sigmoid(1.702 * g) * (u + 1.0)) + w[pre + "down.b"]


def pair_row(bigram, prev, tok):
    """Row of the second embedding table: a hash of the token and its predecessor, or the last row at a sequence's start."""
    if prev is None:
        return bigram["buckets"]
    return (prev * bigram["mul_prev"] + tok * bigram["mul_cur"]) % bigram["buckets"]


class PlainMobatar:
    def __init__(self, cfg, weights):
        self.cfg = cfg
        self.w = {k: v.to(F64) for k, v in weights.items()}
        self.eps = cfg["norm"]["eps"]
        self.bigram = (cfg.get("embedding") or {}).get("bigram")
        self.owner = []
        for i in range(len(cfg["layers"])):
            j = i
            while cfg["layers"][j].get("weights_of") is not None:
                j = cfg["layers"][j]["weights_of"]
            self.owner.append(j)

    def new_state(self):
        st = {"pos": 0, "prev": None, "layers": []}
        for layer in self.cfg["layers"]:
            if layer["type"] == "parallel":
                r = layer["mixer"]["right"]
                st["layers"].append(([], [torch.zeros(r["dim"], r.get("vdim", r["dim"]), dtype=F64) for _ in range(r["heads"])]))
            else:
                st["layers"].append([])
        return st

    def mixer(self, i, h, pos, kept):
        layer, pre = self.cfg["layers"][i], f"l{self.owner[i]}.mix."
        m = layer["mixer"]
        if layer["type"] == "attention":
            return sink_attention(self.w, pre, m, h, pos, kept, self.eps)
        if layer["type"] == "latent_attention":
            return latent_attention(self.w, pre, m, h, pos, kept, self.eps)
        left = chunked_attention(self.w, pre + "left.", m["left"], h, pos, kept[0], self.eps)
        right = retention(self.w, pre + "right.", m["right"], h, pos, kept[1], self.eps)
        return m["left_scale"] * left + m["right_scale"] * right

    def token(self, tok, st, leave_out=None):
        """Logits after one more token of the sequence whose state is st.  ``leave_out``: a mechanism that is skipped
        (for tests that show it matters)."""
        w, pos = self.w, st["pos"]
        x = w["embed"][tok].clone()
        if self.bigram and leave_out != "bigram":
            x = x + w["bigram"][pair_row(self.bigram, st["prev"], tok)]
        for i, layer in enumerate(self.cfg["layers"]):
            p = f"l{self.owner[i]}."
            y = self.mixer(i, x, pos, st["layers"][i])
            x = x + (y if leave_out == "norm1" else shifted_norm(y, w[p + "norm1"], self.eps))
            if layer.get("mlp"):
                x = x + shifted_norm(capped_unit(w, p + "mlp.", layer["mlp"], x), w[p + "norm2"], self.eps)
        st["pos"], st["prev"] = pos + 1, tok
        return w["head"] @ shifted_norm(x, w["final.norm"], self.eps)

    def run(self, tokens, st):
        return torch.stack([self.token(int(t), st) for t in tokens])


def whole_sequence(cfg, weights, tokens):
    """Logits [T, vocab] of one sequence from its start."""
    plain = PlainMobatar(cfg, weights)
    return plain.run(tokens, plain.new_state())
