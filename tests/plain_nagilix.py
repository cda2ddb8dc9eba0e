"""A plain, slow Nagilix for the tests: whole sequences, no cache, one function a mechanism.

It shares no code with ``nanoinfer_b200``: it takes a configuration (the dictionary of config.json) and a dictionary
of tensors by their checkpoint names, and computes in float64 torch.  Linear weights are [out, in] and applied as
W x.

Notation: h is a sublayer's input [n, width]; positions count from 0; rms(x) = x / sqrt(mean(x^2) + eps).
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch

Tensors = Dict[str, torch.Tensor]


# --------------------------------------------------------------------------- small pieces
def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def short_conv(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal convolution over time per channel: x [n, channels], w [channels, taps]; the last tap is the current
    token's and what lies before the sequence is zero."""
    n, taps = x.shape[0], w.shape[1]
    xx = torch.cat([torch.zeros(taps - 1, x.shape[1], dtype=x.dtype), x], 0)
    out = torch.zeros_like(x)
    for j in range(taps):
        out += w[:, j] * xx[j:j + n]
    if bias is not None:
        out = out + bias
    return out


def rotate_halves(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [n, heads, dim]: of every head the first ``dims`` values turn, value i paired with value i + dims/2, by the
    angle position * base^(-2i/dims); the other values pass."""
    if dims == 0:
        return x
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    ang = positions.to(torch.float64)[:, None] * base ** (-2.0 * i / dims)       # [n, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


# --------------------------------------------------------------------------- mixers
def chunked_sink_attention(h: torch.Tensor, w: Tensors, p: str, m: dict, eps: float) -> torch.Tensor:
    """Attention inside chunks of ``mask.size`` positions with a learned sink in the denominator, a temperature per
    head, a short convolution and a norm over the whole projection on queries and keys, and the keys (as they leave
    the convolution) as values."""
    n, H, G, d = h.shape[0], m["heads"], m.get("kv_heads") or m["heads"], m["dim"]
    pos = torch.arange(n)
    q, k = h @ w[p + "q"].T, h @ w[p + "k"].T
    if m.get("conv"):
        q, k = short_conv(q, w[p + "q.conv"]), short_conv(k, w[p + "k.conv"])
    v = k.view(n, G, d)
    q = rms(q, eps) * w[p + "q.norm"]
    k = rms(k, eps) * w[p + "k.norm"]
    rot = m.get("rot") or {}
    q = rotate_halves(q.view(n, H, d), pos, rot.get("dims", 0), rot.get("base", 1.0))
    k = rotate_halves(k.view(n, G, d), pos, rot.get("dims", 0), rot.get("base", 1.0))
    size = (m.get("mask") or {}).get("size") or 0
    i, j = pos[:, None], pos[None, :]
    seen = j <= i
    if size:
        seen = seen & (i // size == j // size)
    out = torch.zeros(n, H, d, dtype=torch.float64)
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * m["scale"] * w[p + "temp"][a]
        s = s.masked_fill(~seen, -math.inf)
        top = torch.maximum(s.max(dim=1, keepdim=True).values, w[p + "sink"][a])
        e = torch.exp(s - top)
        out[:, a] = (e @ v[:, g]) / (e.sum(dim=1, keepdim=True) + torch.exp(w[p + "sink"][a] - top))
    return out.reshape(n, H * d) @ w[p + "o"].T


def retention(h: torch.Tensor, w: Tensors, p: str, m: dict, eps: float) -> torch.Tensor:
    """Linear attention with one fixed decay per head: S <- decay S + k v^T, o = S^T q; no softmax."""
    n, H, d, dv = h.shape[0], m["heads"], m["dim"], m.get("vdim") or m["dim"]
    pos = torch.arange(n)
    rot = m.get("rot") or {}
    q = rotate_halves((h @ w[p + "q"].T).view(n, H, d), pos, rot.get("dims", 0), rot.get("base", 1.0))
    k = rotate_halves((h @ w[p + "k"].T).view(n, H, d), pos, rot.get("dims", 0), rot.get("base", 1.0)) * d ** -0.5
    v = (h @ w[p + "v"].T).view(n, H, dv)
    decay = torch.tensor(m["decay"], dtype=torch.float64)
    S = torch.zeros(H, d, dv, dtype=torch.float64)
    o = torch.zeros(n, H, dv, dtype=torch.float64)
    for t in range(n):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms(o, eps).reshape(n, H * dv) * silu(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def side_by_side(h: torch.Tensor, w: Tensors, p: str, m: dict, eps: float) -> torch.Tensor:
    left = chunked_sink_attention(h, w, p + "left.", m["left"], eps)
    right = retention(h, w, p + "right.", m["right"], eps)
    return 0.5 * (rms(left, eps) * w[p + "left.out"] + rms(right, eps) * w[p + "right.out"])


def selective_scan(h: torch.Tensor, w: Tensors, p: str, m: dict) -> torch.Tensor:
    """Mamba: a state [inner, state] per sequence whose decay, input and read-out depend on the token."""
    n, inner, N, R = h.shape[0], m["inner"], m["state"], m["dt_rank"]
    xz = h @ w[p + "in"].T
    x, z = xz[:, :inner], xz[:, inner:]
    x = silu(short_conv(x, w[p + "conv"], w[p + "conv.b"]))
    dbc = x @ w[p + "x"].T
    dt, B, C = dbc[:, :R], dbc[:, R:R + N], dbc[:, R + N:R + 2 * N]
    dt = softplus(dt @ w[p + "dt"].T + w[p + "dt.b"])
    A = -torch.exp(w[p + "A_log"])
    S = torch.zeros(inner, N, dtype=torch.float64)
    y = torch.zeros(n, inner, dtype=torch.float64)
    for t in range(n):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + w[p + "D"] * x[t]
    return (y * silu(z)) @ w[p + "o"].T


# --------------------------------------------------------------------------- feed-forward
def clamped_expert(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def routed(h: torch.Tensor, w: Tensors, p: str, m: dict, chosen: Optional[list] = None) -> torch.Tensor:
    """Experts chosen by softmax scores plus a correction; weighted by the scores themselves; the last
    ``router.identity`` outputs of the router stand for experts that hand their input on."""
    E, I, top = m["router"]["experts"], m["router"].get("identity", 0), m["router"]["top"]
    s = torch.softmax(h @ w[p + "router"].T, dim=-1)
    pick = torch.topk(s + w[p + "correction"], top, dim=-1).indices
    if chosen is not None:
        chosen.append(pick)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in pick[t].tolist():
            if e >= E:
                out[t] += s[t, e] * h[t]
            else:
                q = f"{p}e{e}."
                out[t] += s[t, e] * clamped_expert(h[t:t + 1], w[q + "gate"], w[q + "up"], w[q + "down"],
                                                   m["expert"]["limit"])[0]
    return out


# --------------------------------------------------------------------------- the model
def forward(cfg: dict, w: Tensors, tokens: Sequence[int], layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits [n, vocab] of a whole sequence.  ``layers_out`` receives the sum of the streams after every layer."""
    w = {k: v.to(torch.float64) for k, v in w.items()}
    eps, S = cfg["norm"]["eps"], cfg.get("streams", 1)
    tok = torch.tensor(list(tokens), dtype=torch.long)
    x0 = w["embed"][tok] + w["pos"][:len(tok)]
    X = [x0.clone() for _ in range(S)]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        for q, sub in ((1, "mixer"), (2, "mlp")):
            if layer.get(sub) is None:
                continue
            hc = f"{p}hc{q}."
            u = sum(w[hc + "in"][s] * X[s] for s in range(S))
            hN = rms(u, eps) * w[f"{p}norm{q}"]
            if sub == "mlp":
                y = routed(hN, w, p + "mlp.", layer["mlp"])
            elif layer["type"] == "mamba1":
                y = selective_scan(hN, w, p + "mix.", layer["mixer"])
            else:
                y = side_by_side(hN, w, p + "mix.", layer["mixer"], eps)
            y = y * torch.sigmoid(hN @ w[f"{p}rg{q}"].T + w[f"{p}rg{q}.b"])
            X = [sum(w[hc + "mix"][s, t] * X[s] for s in range(S)) + w[hc + "out"][t] * y for t in range(S)]
        if layers_out is not None:
            layers_out.append(sum(X))
    x = rms(sum(X), eps) * w["final.norm"]
    return (x @ w["head"].T) * cfg.get("logit_scale", 1.0)


def load_folder(model_dir: str):
    """(config, tensors) of a model folder, read with the ``safetensors`` package."""
    from safetensors import safe_open

    with open(os.path.join(model_dir, "config.json")) as fh:
        cfg = json.load(fh)
    w = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            w[name] = f.get_tensor(name)
    return cfg, w


class PlainNagilix:
    """The plain model of a folder: ``logits(tokens)`` float64 [n, vocab] of a whole sequence."""

    def __init__(self, model_dir: str):
        self.cfg, self.w = load_folder(model_dir)

    def logits(self, tokens: Sequence[int], layers_out: Optional[list] = None) -> torch.Tensor:
        return forward(self.cfg, self.w, tokens, layers_out)

    def greedy(self, prompt: Sequence[int], n: int) -> List[int]:
        """The ``n`` tokens that greedy decoding appends to ``prompt`` (ties to the lower index)."""
        seq, out = list(prompt), []
        for _ in range(n):
            out.append(int(torch.argmax(self.logits(seq)[-1])))
            seq.append(out[-1])
        return out
