"""Plain, slow Dudurax: one function per mechanism, written from the design's equations.

Everything runs on the CPU in one dtype (float64 by default), token by token or with explicit masks; nothing of
the engine is imported.  Notation: h [T, width] is a sublayer's input, rows are tokens of ONE sequence in order.
A sequence's carried state is a plain dict, so that a prompt may be fed in pieces.

    embedding     x_t = E[id_t] * scale + G[(id_{t-1} * mul_prev + id_t * mul_cur) mod buckets]   (G[buckets] at t = 0)
    layer         x <- N1(alpha x + mixer(x));  x <- N2(alpha x + ff(x))      (post-norm, alpha scales the skip path)
    gla           S_t = diag(a_t) S_{t-1} + k_t v_t^T,  o_t = S_t^T q_t,  a_t = sigmoid(z_t)^(1/tau)
    latent attn   c_t = N(W_dkv h)[:r], shared rotated key part, per-head keys / values expanded from c_t, window
    moe           softmax router, correction for the choice only, groups, identity experts, clamped gated experts
"""
from __future__ import annotations

import json
import math
import os

import torch


# --------------------------------------------------------------------------- small pieces
def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def embed(ids, prev_id, E, G, scale, buckets, mul_prev, mul_cur):
    """Rows of the token table times `scale`, plus the bigram table's row of (previous id, id); `prev_id` is the id
    before ids[0], or None at a sequence's start."""
    rows = []
    for t, tok in enumerate(ids):
        before = prev_id if t == 0 else ids[t - 1]
        g = buckets if before is None else (before * mul_prev + tok * mul_cur) % buckets
        rows.append(E[tok] * scale + G[g])
    return torch.stack(rows)


# --------------------------------------------------------------------------- gated linear attention
def gla(h, W, state, *, heads, dim, vdim, tau, eps):
    """W: q, k, v, g, o, norm, a1, a2, a2.b.  `state`: {"S": [heads, dim, vdim]} or {} (zeros)."""
    T = h.shape[0]
    q = (h @ W["q"].T).view(T, heads, dim) * dim ** -0.5
    k = (h @ W["k"].T).view(T, heads, dim)
    v = (h @ W["v"].T).view(T, heads, vdim)
    z = (h @ W["a1"].T) @ W["a2"].T + W["a2.b"]
    decay = torch.sigmoid(z).pow(1.0 / tau).view(T, heads, dim)
    S = state.get("S")
    if S is None:
        S = torch.zeros(heads, dim, vdim, dtype=h.dtype)
    out = []
    for t in range(T):
        S = decay[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hd,hdv->hv", q[t], S))
    state["S"] = S
    o = rms_norm(torch.stack(out), W["norm"], eps).reshape(T, heads * vdim)
    return (o * silu(h @ W["g"].T)) @ W["o"].T


# --------------------------------------------------------------------------- latent attention with a window
def rotate_half(x, pos, base, dims=None):
    """x [..., m] at positions pos [T] (x's first axis): among the first n = dims columns, pairs (i, i + n/2) turn by
    the angle pos * base^(-2i/n); the columns behind stay."""
    if dims is not None and dims < x.shape[-1]:
        return torch.cat([rotate_half(x[..., :dims], pos, base), x[..., dims:]], -1)
    n = x.shape[-1]
    if n == 0:
        return x
    f = base ** (-2.0 * torch.arange(n // 2, dtype=x.dtype) / n)
    a = pos.to(x.dtype)[:, None] * f
    a = a.view(a.shape[0], *([1] * (x.dim() - 2)), n // 2)
    u, v = x[..., : n // 2], x[..., n // 2:]
    return torch.cat([u * torch.cos(a) - v * torch.sin(a), v * torch.cos(a) + u * torch.sin(a)], -1)


def latent_attention(h, W, state, *, heads, dim, rot_dim, vdim, kv_rank, scale, window, base, eps, rot_dims=None):
    """W: q, dkv, dkv.norm, uk, uv, o.  `state`: {"c": [n, kv_rank], "kr": [n, rot_dim]} of the tokens before."""
    T = h.shape[0]
    n0 = 0 if "c" not in state else state["c"].shape[0]
    pos = torch.arange(n0, n0 + T)
    q = (h @ W["q"].T).view(T, heads, dim + rot_dim)
    q_plain, q_rot = q[..., :dim], rotate_half(q[..., dim:], pos, base, rot_dims)
    d = h @ W["dkv"].T
    c = rms_norm(d[:, :kv_rank], W["dkv.norm"], eps)
    kr = rotate_half(d[:, kv_rank:], pos, base, rot_dims)
    if n0:
        c, kr = torch.cat([state["c"], c]), torch.cat([state["kr"], kr])
    state["c"], state["kr"] = c, kr
    k_plain = (c @ W["uk"].T).view(-1, heads, dim)
    val = (c @ W["uv"].T).view(-1, heads, vdim)
    out = torch.zeros(T, heads, vdim, dtype=h.dtype)
    for t in range(T):
        i = n0 + t
        lo = max(0, i - window + 1)
        s = (torch.einsum("hd,jhd->hj", q_plain[t], k_plain[lo:i + 1]) + q_rot[t] @ kr[lo:i + 1].T) * scale
        out[t] = torch.einsum("hj,jhv->hv", torch.softmax(s, -1), val[lo:i + 1])
    return out.reshape(T, heads * vdim) @ W["o"].T


# --------------------------------------------------------------------------- feed-forwards
def dense_ff(h, W):
    return gelu_tanh(h @ W["up"].T) @ W["down"].T


def route(h, W_router, correction, *, top, groups, keep, scale):
    """[T, n] weights (zero where not chosen) over real and identity experts together."""
    s = torch.softmax(h @ W_router.T, -1)
    choice = s + correction
    T, n = s.shape
    best = choice.view(T, groups, n // groups).max(-1).values
    kept = torch.zeros(T, groups, dtype=torch.bool)
    kept.scatter_(1, best.topk(keep, -1).indices, True)
    choice = torch.where(kept[:, :, None].expand(T, groups, n // groups).reshape(T, n), choice,
                         torch.full_like(choice, -math.inf))
    w = torch.zeros_like(s)
    idx = choice.topk(top, -1).indices
    w.scatter_(1, idx, s.gather(1, idx) * scale)
    return w


def expert(h, gate, up, down, limit):
    g = (h @ gate.T).clamp(max=limit)
    u = (h @ up.T).clamp(-limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def moe_ff(h, W, *, experts, identity, top, groups, keep, scale, limit):
    w = route(h, W["router"], W["correction"], top=top, groups=groups, keep=keep, scale=scale)
    out = h * w[:, experts:].sum(-1, keepdim=True)
    for e in range(experts):
        out = out + w[:, e:e + 1] * expert(h, W[f"e{e}.gate"], W[f"e{e}.up"], W[f"e{e}.down"], limit)
    return out


# --------------------------------------------------------------------------- the model
class PlainDudurax:
    def __init__(self, config: dict, tensors: dict, dtype=torch.float64):
        self.cfg, self.dtype = config, dtype
        self.w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}

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
        return {"prev": None, "layers": [dict() for _ in self.cfg["layers"]]}

    def forward(self, ids, state, layer_outputs=None):
        """Logits [T, vocab] of the next `ids` of a sequence whose earlier tokens left `state`."""
        cfg, eps, alpha = self.cfg, self.cfg["norm"]["eps"], self.cfg["postln_alpha"]
        bg = cfg["embedding"]["bigram"]
        x = embed(list(ids), state["prev"], self.w["embed"], self.w["bigram"], cfg["embedding"]["scale"],
                  bg["buckets"], bg["mul_prev"], bg["mul_cur"])
        state["prev"] = ids[-1]
        for i, layer in enumerate(cfg["layers"]):
            m, st = layer["mixer"], state["layers"][i]
            W = self._sub(f"l{i}.mix.")
            if layer["type"] in ("gla", "gla_2"):
                y = gla(x, W, st, heads=m["heads"], dim=m["dim"], vdim=m["vdim"], tau=m["tau"], eps=eps)
            elif layer["type"] == "latent_attention":
                y = latent_attention(x, W, st, heads=m["heads"], dim=m["dim"], rot_dim=m["rot_dim"], vdim=m["vdim"],
                                     kv_rank=m["kv_rank"], scale=m["scale"], window=m["mask"]["size"],
                                     base=m["rot"]["base"], eps=eps, rot_dims=m["rot"]["dims"])
            else:
                raise ValueError(layer["type"])
            x = rms_norm(alpha * x + y, self.w[f"l{i}.norm1"], eps)
            ff = layer.get("mlp")
            if ff is not None:
                W = self._sub(f"l{i}.mlp.")
                if ff["kind"] == "dense":
                    y = dense_ff(x, W)
                else:
                    r = ff["router"]
                    y = moe_ff(x, W, experts=r["experts"], identity=r["identity"], top=r["top"],
                               groups=r["groups"]["count"], keep=r["groups"]["keep"], scale=r["scale"],
                               limit=ff["expert"]["limit"])
                x = rms_norm(alpha * x + y, self.w[f"l{i}.norm2"], eps)
            if layer_outputs is not None:
                layer_outputs.append(x)
        return rms_norm(x, self.w["final.norm"], eps) @ self.w["head"].T
