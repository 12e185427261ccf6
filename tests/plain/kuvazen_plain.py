"""Plain, slow Kuvazen: one function per mechanism, written from the design's equations.

Everything runs on the CPU in one dtype (float64 by default), token by token or with explicit loops over the keys;
nothing of the engine is imported.  Notation: h [T, width] is a sublayer's input, rows are tokens of ONE sequence in
order.  A sequence's carried state is a plain dict, so that a prompt may be fed in pieces.

    embedding   x_t = LN(E[id_t]) * w
    layer       x <- x + s1 * mixer(LN1(x));  x <- x + s2 * ff(LN2(x));  x <- x + RMS(P (gelu(G x) * e_t)) * w_side
                (s1, s2: a scale per channel; e_t: this layer's slice of a second embedding row of the token)
    mingru      S_t = (1 - z_t) S_{t-1} + z_t c_t;  c = u + 1/2 (u >= 0), sigmoid(u) (u < 0);  y = W_o (S * silu(g))
    attention   rotated q, k (neighbouring pairs) AND rotated values; key j is seen by i if 0 <= i - j < W; a whole
                block of P tokens that lies behind the window is seen as ONE key/value, the block's mean; one
                softmax over both; the summed values are turned back by the query's position
    dense ff    W_d [g~ sigmoid(1.702 g~) (u~ + 1)],  g~ = min(g, L), u~ = clamp(u, +-L)
    moe         s = sigmoid(W_r h); the `top` largest are chosen; y = sum_e expert_e(s_e h), expert = W_d (silu(W_g .) * (W_u .))
"""
from __future__ import annotations

import json
import math
import os

import torch


# --------------------------------------------------------------------------- small pieces
def layer_norm(x, w, eps):
    d = x - x.mean(-1, keepdim=True)
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * w


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def turn_pairs(x, pos, base, dims):
    """Rotate the first `dims` columns of every row of x [..., n]: column 2i with column 2i + 1 by the angle
    pos * base^(-2i / dims).  `pos` may be negative (turning back)."""
    out = x.clone()
    if dims == 0:
        return out
    a = pos * torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
    c, s = torch.cos(a).to(x.dtype), torch.sin(a).to(x.dtype)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


# --------------------------------------------------------------------------- token side input
def side_input(x, ids, layer, E_side, W, dim, eps):
    """x + RMS(proj (gelu(gate x) * e)) * norm, e = columns [layer * dim, (layer + 1) * dim) of the tokens' side rows."""
    e = E_side[torch.as_tensor(list(ids))][:, layer * dim:(layer + 1) * dim]
    g = gelu_tanh(x @ W["gate"].T) * e
    y = g @ W["proj"].T
    return x + rms_norm(y, W["norm"], eps)


# --------------------------------------------------------------------------- minGRU
def mingru(h, W, state):
    """W: z, z.b, x, x.b, g, o.  `state`: {"S": [width]} or {} (zeros)."""
    z = torch.sigmoid(h @ W["z"].T + W["z.b"])
    u = h @ W["x"].T + W["x.b"]
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    gate = silu(h @ W["g"].T)
    S = state.get("S")
    if S is None:
        S = torch.zeros(z.shape[1], dtype=h.dtype)
    rows = []
    for t in range(h.shape[0]):
        S = (1.0 - z[t]) * S + z[t] * cand[t]
        rows.append(S * gate[t])
    state["S"] = S
    return torch.stack(rows) @ W["o"].T


# --------------------------------------------------------------------------- attention over a window and pooled blocks
def pooled_window_attention(h, W, state, *, heads, kv_heads, dim, vdim, scale, window, pool, base, rot_dims):
    """W: q, k, v, o.  `state`: {"k": [n, kv_heads, dim], "v": [n, kv_heads, vdim]} of all earlier tokens (rotated), or {}."""
    T = h.shape[0]
    start = 0 if "k" not in state else state["k"].shape[0]
    q = (h @ W["q"].T).view(T, heads, dim)
    k = (h @ W["k"].T).view(T, kv_heads, dim)
    v = (h @ W["v"].T).view(T, kv_heads, vdim)
    q = torch.stack([turn_pairs(q[t], start + t, base, rot_dims) for t in range(T)])
    k = torch.stack([turn_pairs(k[t], start + t, base, rot_dims) for t in range(T)])
    v = torch.stack([turn_pairs(v[t], start + t, base, vdim) for t in range(T)])
    if start:
        k, v = torch.cat([state["k"], k]), torch.cat([state["v"], v])
    state["k"], state["v"] = k, v
    per = heads // kv_heads
    out = torch.zeros(T, heads, vdim, dtype=h.dtype)
    for t in range(T):
        i = start + t
        first = max(0, i - window + 1)                       # the oldest token inside the window
        blocks = max(0, (i - window + 1) // pool)             # blocks that lie wholly behind the window
        # what position i sees: one mean per block, then the window's tokens  [n, kv_heads, .]
        keys = torch.cat([k[:blocks * pool].reshape(blocks, pool, kv_heads, dim).mean(1), k[first:i + 1]])
        vals = torch.cat([v[:blocks * pool].reshape(blocks, pool, kv_heads, vdim).mean(1), v[first:i + 1]])
        for hd in range(heads):
            g = hd // per
            p = torch.softmax(keys[:, g] @ q[t, hd] * scale, 0)
            out[t, hd] = turn_pairs(p @ vals[:, g], -i, base, vdim)
    return out.reshape(T, heads * vdim) @ W["o"].T


# --------------------------------------------------------------------------- feed-forwards
def dense_ff(h, W, limit):
    g = torch.clamp(h @ W["gate"].T, max=limit)
    u = torch.clamp(h @ W["up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W["down"].T


def moe_ff(h, W, *, experts, top, margins=None):
    """`margins` (a list): per token the gap between the last chosen score and the best one left out is appended (a
    small gap is a choice that rounding may turn)."""
    s = torch.sigmoid(h @ W["router"].T)                      # [T, experts]
    out = torch.zeros_like(h)
    if margins is not None:
        ranked = s.sort(-1, descending=True).values
        margins.append(ranked[:, top - 1] - ranked[:, top] if experts > top else torch.ones_like(s[:, 0]))
    for t in range(h.shape[0]):
        for e in torch.topk(s[t], top).indices.tolist():
            x = s[t, e] * h[t]
            out[t] += (silu(x @ W[f"e{e}.gate"].T) * (x @ W[f"e{e}.up"].T)) @ W[f"e{e}.down"].T
    return out


# --------------------------------------------------------------------------- the model
class PlainKuvazen:
    def __init__(self, cfg: dict, tensors: dict, dtype=torch.float64):
        self.cfg = cfg
        self.w = {k: (v if v.dtype in (torch.int32, torch.int64) else v.to(dtype)) for k, v in tensors.items()}
        self.dtype = dtype
        loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
        n = len(cfg["layers"])
        a, b, times = loop["start"], loop["stop"], loop["times"]
        self.runs = list(range(a)) + list(range(a, b)) * times + list(range(b, n)) if b > a else list(range(n))

    @classmethod
    def from_folder(cls, folder: str, dtype=torch.float64):
        from safetensors import safe_open
        with open(os.path.join(folder, "config.json")) as f:
            cfg = json.load(f)
        tensors = {}
        with safe_open(os.path.join(folder, "model.safetensors"), framework="pt", device="cpu") as f:
            for name in f.keys():
                tensors[name] = f.get_tensor(name)
        return cls(cfg, tensors, dtype)

    def _sub(self, prefix):
        return {k[len(prefix):]: v for k, v in self.w.items() if k.startswith(prefix)}

    def new_state(self):
        return {"runs": [dict() for _ in self.runs]}

    def forward(self, ids, state, layer_outputs=None, margins=None):
        """Logits [T, vocab] of the next `ids` of a sequence whose earlier tokens left `state`.  `margins` (a list) gets
        one tensor [T] per routed layer run: how clear the router's choice was (see `moe_ff`)."""
        cfg, eps = self.cfg, self.cfg["norm"]["eps"]
        ids = list(ids)
        x = layer_norm(self.w["embed"][torch.as_tensor(ids)], self.w["embed.norm"], eps)
        for run, i in enumerate(self.runs):
            layer, st = cfg["layers"][i], state["runs"][run]
            m = layer["mixer"]
            W = self._sub(f"l{i}.mix.")
            hin = layer_norm(x, self.w[f"l{i}.norm1"], eps)
            if layer["type"] == "mingru":
                y = mingru(hin, W, st)
            elif layer["type"] == "attention":
                y = pooled_window_attention(hin, W, st, heads=m["heads"], kv_heads=m["kv_heads"], dim=m["dim"], vdim=m["vdim"],
                                            scale=m["scale"], window=m["mask"]["size"], pool=m["mask"]["pool"],
                                            base=m["rot"]["base"], rot_dims=m["rot"]["dims"])
            else:
                raise ValueError(layer["type"])
            x = x + self.w[f"l{i}.ls1"] * y
            ff = layer.get("mlp")
            if ff is not None:
                W = self._sub(f"l{i}.mlp.")
                hin = layer_norm(x, self.w[f"l{i}.norm2"], eps)
                if ff["kind"] == "dense":
                    y = dense_ff(hin, W, ff["limit"])
                else:
                    y = moe_ff(hin, W, experts=ff["router"]["experts"], top=ff["router"]["top"], margins=margins)
                x = x + self.w[f"l{i}.ls2"] * y
            if cfg.get("token_side"):
                x = side_input(x, ids, i, self.w["side.embed"], self._sub(f"l{i}.side."), cfg["token_side"]["dim"], eps)
            if layer_outputs is not None:
                layer_outputs.append(x)
        return layer_norm(x, self.w["final.norm"], eps) @ self.w["head"].T
