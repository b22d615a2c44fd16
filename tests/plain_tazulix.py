"""A plain, slow implementation of the Tazulix design, written from its equations: one function per mechanism,
float64, one token after the other, lists and matrices for caches and states.  It shares no code with the package.

Notation: x the stream [width]; h a sublayer's input; N(v, w) = v / sqrt(mean(v^2) + eps) * w.

  embedding      x = E[token] * embedding.scale;  x0 = that x
  loop           layers start .. stop-1 run `times` times with the same weights; before the first layer of every
                 pass x = W_in [x; x0]; every pass has caches and states of its own
  layer          x += mixer(N(x, norm1));  x += ff(N(x, norm2))  (ff may be absent)
  lightning      per head (H heads): q = silu(W_q h), k = silu(W_k h) of size D, v = silu(W_v h) of size V;
                 S <- decay_head * S + k v^T (S [D, V], zero at the start);  o = S^T q;
                 y = W_o (N(all heads' o side by side, norm) * sigmoid(W_g h))
  attention      q = W_q h + b_q, k = W_k h + b_k, v = W_v h + b_v;  q = N(q, q.norm), k = N(k, k.norm) over ALL heads
                 at once;  the first rot.dims dimensions of every head rotated, dimension i with i + dims/2, by the
                 angle p * f_i, cos and sin both times m;  s = (q . k) * scale;  softmax over keys 0 .. p;  head h
                 reads key head h // (H / G);  W_o on the heads side by side
  frequencies    f_i = base^(-2i / dims), or with scaling (factor, original, fast, slow):
                 c(t) = dims * ln(original / (2 pi t)) / (2 ln base), lo = max(floor(c(fast)), 0),
                 hi = min(ceil(c(slow)), dims - 1), r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1),
                 f_i <- f_i / factor * r_i + f_i * (1 - r_i),  m = 0.1 ln(factor) + 1  (m = 1 without scaling)
  dense ff       W_down relu(W_up h)^2
  unit           g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit);  W_down (g * sigmoid(1.702 g) * (u + 1))
  routed ff      s = sigmoid(W_router h);  the `top` experts with the largest s are chosen;
                 sum over the chosen e of unit_e(s_e * h), plus the shared unit(h) if there is one
  output         logits = W_head N(x, final.norm)
"""
import math

import torch

F64 = torch.float64


def rms_norm(v, w, eps):
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps) * w


def silu(z):
    return z * torch.sigmoid(z)


def rotary_frequencies(rot):
    """(frequencies [dims / 2], the factor on cos and sin)."""
    dims, base = rot["dims"], rot["base"]
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0

    def corr(t):
        return dims * math.log(sc["original"] / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(corr(sc["fast"])), 0)
    hi = min(math.ceil(corr(sc["slow"])), dims - 1)
    out = []
    for i, fi in enumerate(f):
        r = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / sc["factor"] * r + fi * (1.0 - r))
    return out, 0.1 * math.log(sc["factor"]) + 1.0


def rotate_half(v, position, rot):
    """v [heads, D]: dimension i of the first ``dims`` is paired with dimension i + dims / 2."""
    if not rot or not rot["dims"]:
        return v
    f, m = rotary_frequencies(rot)
    half = rot["dims"] // 2
    out = v.clone()
    for i in range(half):
        a = position * f[i]
        c, s = math.cos(a) * m, math.sin(a) * m
        out[:, i] = v[:, i] * c - v[:, i + half] * s
        out[:, i + half] = v[:, i + half] * c + v[:, i] * s
    return out


def attend(q, keys, values, scale):
    """q [H, D]; keys [n, G, D], values [n, G, V] (all visible keys): returns [H, V]."""
    n_heads, n_kv = q.shape[0], keys.shape[1]
    out = []
    for h in range(n_heads):
        g = h // (n_heads // n_kv)
        p = torch.softmax((keys[:, g] @ q[h]) * scale, 0)
        out.append(p @ values[:, g])
    return torch.stack(out)


def lightning_token(S, q, k, v, decay):
    """S [H, D, V], q and k [H, D], v [H, V], decay [H]: the new S and the read-out [H, V]."""
    S = decay[:, None, None] * S + k[:, :, None] * v[:, None, :]
    return S, torch.einsum("hdv,hd->hv", S, q)


def relu2_unit(h, w_up, w_down):
    return w_down @ torch.relu(w_up @ h) ** 2


def capped_unit(h, w_gate, w_up, w_down, limit):
    g = torch.clamp(w_gate @ h, max=limit)
    u = torch.clamp(w_up @ h, -limit, limit)
    return w_down @ (g * torch.sigmoid(1.702 * g) * (u + 1.0))


def route(h, w_router, top):
    """(chosen experts, all scores)."""
    s = torch.sigmoid(w_router @ h)
    return torch.topk(s, top).indices.tolist(), s


def routed_unit(h, w_router, experts, top, limit, shared=None):
    """experts: list of (w_gate, w_up, w_down); shared: (w_gate, w_up, w_down, limit) or None.  The score
    multiplies the expert's input."""
    chosen, s = route(h, w_router, top)
    out = torch.zeros_like(h)
    for e in chosen:
        out = out + capped_unit(s[e] * h, *experts[e], limit)
    if shared is not None:
        out = out + capped_unit(h, *shared)
    return out


def layer_runs(cfg):
    """[(layer, first of its pass)] in the order of execution."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    runs = [(i, False) for i in range(loop["start"])]
    for _ in range(loop["times"]):
        runs += [(i, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, False) for i in range(loop["stop"], n)]


class PlainTazulix:
    def __init__(self, cfg, weights):
        self.cfg = cfg
        self.w = {k: v.to(F64) for k, v in weights.items()}
        self.eps = cfg["norm"]["eps"]
        self.runs = layer_runs(cfg)

    def new_state(self):
        """Per run: keys and values so far, or the lightning state; and the position."""
        return {"pos": 0, "runs": [{"k": [], "v": [], "S": None} for _ in self.runs]}

    def attention(self, i, h, position, st):
        w, m = self.w, self.cfg["layers"][i]["mixer"]
        p = f"l{i}.mix."
        n_heads, n_kv, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        q = rms_norm(w[p + "q"] @ h + w[p + "q.b"], w[p + "q.norm"], self.eps).view(n_heads, dim)
        k = rms_norm(w[p + "k"] @ h + w[p + "k.b"], w[p + "k.norm"], self.eps).view(n_kv, dim)
        v = (w[p + "v"] @ h + w[p + "v.b"]).view(n_kv, vdim)
        st["k"].append(rotate_half(k, position, m.get("rot")))
        st["v"].append(v)
        out = attend(rotate_half(q, position, m.get("rot")), torch.stack(st["k"]), torch.stack(st["v"]), m["scale"])
        return w[p + "o"] @ out.reshape(-1)

    def lightning(self, i, h, st):
        w, m = self.w, self.cfg["layers"][i]["mixer"]
        p = f"l{i}.mix."
        n_heads, dim, vdim = m["heads"], m["dim"], m["vdim"]
        if st["S"] is None:
            st["S"] = torch.zeros(n_heads, dim, vdim, dtype=F64)
        q, k = silu(w[p + "q"] @ h).view(n_heads, dim), silu(w[p + "k"] @ h).view(n_heads, dim)
        v = silu(w[p + "v"] @ h).view(n_heads, vdim)
        st["S"], o = lightning_token(st["S"], q, k, v, torch.tensor(m["decay"], dtype=F64))
        return w[p + "o"] @ (rms_norm(o.reshape(-1), w[p + "norm"], self.eps) * torch.sigmoid(w[p + "g"] @ h))

    def feed_forward(self, i, h):
        w, mlp = self.w, self.cfg["layers"][i]["mlp"]
        p = f"l{i}.mlp."
        if mlp["kind"] == "dense":
            return relu2_unit(h, w[p + "up"], w[p + "down"])
        r = mlp["router"]
        experts = [(w[f"{p}e{e}.gate"], w[f"{p}e{e}.up"], w[f"{p}e{e}.down"]) for e in range(r["experts"])]
        shared = None
        if mlp.get("shared"):
            shared = (w[p + "shared.gate"], w[p + "shared.up"], w[p + "shared.down"], mlp["shared"]["limit"])
        return routed_unit(h, w[p + "router"], experts, r["top"], mlp["expert"]["limit"], shared)

    def token(self, tok, state, streams=None, leave_out=()):
        cfg, w, eps = self.cfg, self.w, self.eps
        x0 = w["embed"][tok] * (cfg.get("embedding") or {}).get("scale", 1.0)
        x = x0
        for r, (i, first) in enumerate(self.runs):
            if first and "loop.in" not in leave_out:
                x = w["loop.in"] @ torch.cat([x, x0])
            p = f"l{i}."
            h = rms_norm(x, w[p + "norm1"], eps)
            if cfg["layers"][i]["type"] == "lightning":
                x = x + self.lightning(i, h, state["runs"][r])
            else:
                x = x + self.attention(i, h, state["pos"], state["runs"][r])
            if cfg["layers"][i].get("mlp") is not None:
                x = x + self.feed_forward(i, rms_norm(x, w[p + "norm2"], eps))
            if streams is not None:
                streams.append(x.clone())
        state["pos"] += 1
        return w["head"] @ rms_norm(x, w["final.norm"], eps)

    def run(self, tokens, state):
        """Logits [len(tokens), vocab] of the next tokens of the sequence that ``state`` holds."""
        return torch.stack([self.token(int(t), state) for t in tokens])


def whole_sequence(cfg, weights, tokens):
    """The same design once more, for a whole sequence at once in matrices (no caches, no state; the lightning
    mixer as a decayed causal product): what the token-by-token form must agree with.  Returns logits [T, vocab]."""
    w = {k: v.to(F64) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    n = len(tokens)
    x0 = w["embed"][torch.tensor(tokens)] * (cfg.get("embedding") or {}).get("scale", 1.0)
    x = x0
    causal = torch.tril(torch.ones(n, n, dtype=torch.bool))
    steps = torch.arange(n, dtype=F64)
    apart = (steps[:, None] - steps[None, :]).clamp(min=0)            # t - j where the key is visible

    def rotate(v, rot):
        if not rot or not rot["dims"]:
            return v
        f, m = rotary_frequencies(rot)
        half = rot["dims"] // 2
        ang = steps[:, None] * torch.tensor(f, dtype=F64)
        c, s = (torch.cos(ang) * m)[:, None], (torch.sin(ang) * m)[:, None]
        out = v.clone()
        a, b = v[..., :half], v[..., half:2 * half]
        out[..., :half], out[..., half:2 * half] = a * c - b * s, b * c + a * s
        return out

    for i, first in layer_runs(cfg):
        if first:
            x = torch.cat([x, x0], -1) @ w["loop.in"].T
        layer, p = cfg["layers"][i], f"l{i}."
        m = layer["mixer"]
        h = rms_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "lightning":
            n_heads, dim, vdim = m["heads"], m["dim"], m["vdim"]
            q, k = silu(h @ w[p + "mix.q"].T).view(n, n_heads, dim), silu(h @ w[p + "mix.k"].T).view(n, n_heads, dim)
            v = silu(h @ w[p + "mix.v"].T).view(n, n_heads, vdim)
            heads = []
            for hd in range(n_heads):
                a = (q[:, hd] @ k[:, hd].T) * torch.pow(torch.tensor(m["decay"][hd], dtype=F64), apart)
                heads.append(a.masked_fill(~causal, 0.0) @ v[:, hd])
            o = rms_norm(torch.cat(heads, -1), w[p + "mix.norm"], eps) * torch.sigmoid(h @ w[p + "mix.g"].T)
            x = x + o @ w[p + "mix.o"].T
        else:
            n_heads, n_kv, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            q = rms_norm(h @ w[p + "mix.q"].T + w[p + "mix.q.b"], w[p + "mix.q.norm"], eps).view(n, n_heads, dim)
            k = rms_norm(h @ w[p + "mix.k"].T + w[p + "mix.k.b"], w[p + "mix.k.norm"], eps).view(n, n_kv, dim)
            v = (h @ w[p + "mix.v"].T + w[p + "mix.v.b"]).view(n, n_kv, vdim)
            q, k = rotate(q, m.get("rot")), rotate(k, m.get("rot"))
            heads = []
            for hd in range(n_heads):
                g = hd // (n_heads // n_kv)
                s = ((q[:, hd] @ k[:, g].T) * m["scale"]).masked_fill(~causal, -math.inf)
                heads.append(torch.softmax(s, -1) @ v[:, g])
            x = x + torch.cat(heads, -1) @ w[p + "mix.o"].T
        mlp = layer.get("mlp")
        if mlp is not None:
            h = rms_norm(x, w[p + "norm2"], eps)
            if mlp["kind"] == "dense":
                y = torch.relu(h @ w[p + "mlp.up"].T) ** 2 @ w[p + "mlp.down"].T
            else:
                r_ = mlp["router"]
                experts = [(w[f"{p}mlp.e{e}.gate"], w[f"{p}mlp.e{e}.up"], w[f"{p}mlp.e{e}.down"]) for e in range(r_["experts"])]
                shared = None
                if mlp.get("shared"):
                    shared = (w[p + "mlp.shared.gate"], w[p + "mlp.shared.up"], w[p + "mlp.shared.down"], mlp["shared"]["limit"])
                y = torch.stack([routed_unit(r, w[p + "mlp.router"], experts, r_["top"], mlp["expert"]["limit"], shared) for r in h])
            x = x + y
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T
