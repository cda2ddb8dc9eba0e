"""A plain, slow Kemuzen for the tests: whole sequences, no cache, one function a mechanism.

It shares no code with ``nanoinfer_b200``: it reads the model folder with the ``safetensors`` package
and ``json`` and computes in float64 torch.  Linear weights are [out, in] and applied as W x.

Notation: h is a sublayer's input [n, width]; positions count from 0; rms(x) = x / sqrt(mean(x^2) + eps).
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch


# --------------------------------------------------------------------------- small pieces
def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def capped(z: torch.Tensor, cap: float) -> torch.Tensor:
    return cap * torch.tanh(z / cap)


def sinusoid(positions: torch.Tensor, width: int) -> torch.Tensor:
    """[n, width]: entry 2i is sin(p * 10000^(-2i/width)), entry 2i + 1 the cosine of the same angle."""
    out = torch.zeros(len(positions), width, dtype=torch.float64)
    for c in range(width):
        i = c // 2
        ang = positions.to(torch.float64) * 10000.0 ** (-2.0 * i / width)
        out[:, c] = torch.sin(ang) if c % 2 == 0 else torch.cos(ang)
    return out


def short_conv(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
               before: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal convolution over time per channel: x [n, channels], w [channels, taps], the last tap is the current
    token's; ``before`` holds the taps - 1 inputs ahead of x (zeros at the start of a sequence)."""
    n, taps = x.shape[0], w.shape[1]
    pad = torch.zeros(taps - 1, x.shape[1], dtype=x.dtype) if before is None else before
    xx = torch.cat([pad, x], 0)
    out = torch.zeros_like(x)
    for t in range(n):
        for j in range(taps):
            out[t] += w[:, j] * xx[t + j]
    if bias is not None:
        out = out + bias
    return out


def heads_rms(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x [n, heads, d]: every head over its root mean square, times one weight [d] shared by the heads."""
    return rms(x, eps) * weight


def visible(n: int, size: Optional[int], keep_first: int) -> torch.Tensor:
    """[n, n] booleans: row i sees column j if j <= i and (i - j < size or j < keep_first)."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    near = (i - j < size) if size else torch.ones(n, n, dtype=torch.bool)
    return (j <= i) & (near | (j < keep_first))


# --------------------------------------------------------------------------- mixers
def capped_attention_kv(h, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float):
    """Keys (after their norm) and values of a capped-attention layer: what its cache holds."""
    n, G, d, dv = h.shape[0], (m.get("kv_heads") or m["heads"]), m["dim"], m["vdim"]
    k = (h @ W[p + "k"].T + W[p + "k.b"]).view(n, G, d)
    v = (h @ W[p + "v"].T + W[p + "v.b"]).view(n, G, dv)
    return heads_rms(k, W[p + "k.norm"], eps), v


def capped_attention(h, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float, kv=None) -> torch.Tensor:
    """Attention with biases, query/key norm per head, no rotation, scores (q . k) scale squashed by
    cap tanh(s / cap), a sliding window that also keeps the first tokens, ordinary softmax.  ``kv``: another
    layer's (keys, values) to read instead of this layer's own."""
    n, H, G, d, dv = h.shape[0], m["heads"], (m.get("kv_heads") or m["heads"]), m["dim"], m["vdim"]
    q = heads_rms((h @ W[p + "q"].T + W[p + "q.b"]).view(n, H, d), W[p + "q.norm"], eps)
    k, v = kv if kv is not None else capped_attention_kv(h, W, p, m, eps)
    mask = m.get("mask") or {}
    see = visible(n, mask.get("size"), int(mask.get("keep_first", 0)))
    out = torch.zeros(n, H, dv, dtype=h.dtype)
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * m["scale"]
        if m.get("softcap"):
            s = capped(s, float(m["softcap"]))
        s = s.masked_fill(~see, -math.inf)
        out[:, a] = torch.softmax(s, dim=-1) @ v[:, g]
    return out.reshape(n, H * dv) @ W[p + "o"].T + W[p + "o.b"]


def distance_attention(h, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """Attention without biases, query/key norm per head, scores (q . k) scale - slope_a (i - j) with
    slope_a = 2^(-8 (a + 1) / H), a plain sliding window, softmax, every head's output times the sigmoid of
    one number of its own."""
    n, H, G, d, dv = h.shape[0], m["heads"], (m.get("kv_heads") or m["heads"]), m["dim"], m["vdim"]
    q = heads_rms((h @ W[p + "q"].T).view(n, H, d), W[p + "q.norm"], eps)
    k = heads_rms((h @ W[p + "k"].T).view(n, G, d), W[p + "k.norm"], eps)
    v = (h @ W[p + "v"].T).view(n, G, dv)
    see = visible(n, (m.get("mask") or {}).get("size"), 0)
    dist = (torch.arange(n)[:, None] - torch.arange(n)[None, :]).to(torch.float64)
    gate = torch.sigmoid(h @ W[p + "g"].T)
    out = torch.zeros(n, H, dv, dtype=h.dtype)
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * m["scale"] - 2.0 ** (-8.0 * (a + 1) / H) * dist
        s = s.masked_fill(~see, -math.inf)
        out[:, a] = (torch.softmax(s, dim=-1) @ v[:, g]) * gate[:, a:a + 1]
    return out.reshape(n, H * dv) @ W[p + "o"].T


def gated_delta(h, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """The gated delta rule, token by token.  Per head, with unit q (times dim^-1/2) and k:
        S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q."""
    n, H, G, d, dv = h.shape[0], m["heads"], (m.get("kv_heads") or m["heads"]), m["dim"], m["vdim"]
    q = silu(short_conv(h @ W[p + "q"].T, W[p + "q.conv"])).view(n, G, d)
    k = silu(short_conv(h @ W[p + "k"].T, W[p + "k.conv"])).view(n, G, d)
    v = silu(short_conv(h @ W[p + "v"].T, W[p + "v.conv"])).view(n, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ W[p + "b"].T)
    decay = torch.exp(-torch.exp(W[p + "A_log"]) * softplus(h @ W[p + "a"].T + W[p + "dt_bias"]))
    gate = silu(h @ W[p + "g"].T).view(n, H, dv)
    out = torch.zeros(n, H, dv, dtype=h.dtype)
    for a in range(H):
        c = a // (H // G)
        S = torch.zeros(d, dv, dtype=h.dtype)
        for t in range(n):
            S = decay[t, a] * S
            u = beta[t, a] * (v[t, a] - S.T @ k[t, c])
            S = S + torch.outer(k[t, c], u)
            out[t, a] = S.T @ q[t, c]
    out = rms(out, eps) * W[p + "norm"] * gate
    return out.reshape(n, H * dv) @ W[p + "o"].T


def state_space(h, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """Mamba-2, token by token.  W_in h = [z | x | B | C | dt]; x, B, C through the short convolution (with a
    bias) and silu; dt = softplus(dt + dt_bias); per head S <- exp(-exp(A_log) dt) S + dt B x^T (S is
    state x vdim), y = S^T C + D x; then y silu(z), RMS norm in groups, the weight, W_o."""
    n, H, dv, N, G = h.shape[0], m["heads"], m["vdim"], m["state"], (m.get("groups") or 1)
    inner = H * dv
    u = h @ W[p + "in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    xbc = silu(short_conv(xbc, W[p + "conv"], W[p + "conv.b"]))
    x = xbc[:, :inner].view(n, H, dv)
    B = xbc[:, inner:inner + G * N].view(n, G, N)
    C = xbc[:, inner + G * N:].view(n, G, N)
    dt = softplus(dt + W[p + "dt_bias"])
    y = torch.zeros(n, H, dv, dtype=h.dtype)
    for a in range(H):
        g = a // (H // G)
        S = torch.zeros(N, dv, dtype=h.dtype)
        for t in range(n):
            S = torch.exp(-torch.exp(W[p + "A_log"][a]) * dt[t, a]) * S + dt[t, a] * torch.outer(B[t, g], x[t, a])
            y[t, a] = S.T @ C[t, g] + W[p + "D"][a] * x[t, a]
    y = y.reshape(n, inner) * silu(z)
    parts = m.get("norm_groups") or 1
    y = rms(y.view(n, parts, inner // parts), eps).reshape(n, inner) * W[p + "norm"]
    return y @ W[p + "o"].T


def side_by_side(h, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    return (m.get("left_scale", 1.0) * distance_attention(h, W, p + "left.", m["left"], eps)
            + m.get("right_scale", 1.0) * state_space(h, W, p + "right.", m["right"], eps))


# --------------------------------------------------------------------------- feed-forward, token input
def gated_mlp(h, W: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return (silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def token_input(x, tokens, W: Dict[str, torch.Tensor], p: str, i: int, dim: int, eps: float) -> torch.Tensor:
    """What the layer's own piece of a second embedding adds: y = W_proj (gelu(W_gate x) * e), x + rms(y) w."""
    e = W["side.embed"][tokens][:, i * dim:(i + 1) * dim]
    y = (gelu_tanh(x @ W[p + "gate"].T) * e) @ W[p + "proj"].T
    return x + rms(y, eps) * W[p + "norm"]


# --------------------------------------------------------------------------- the model
class PlainKemuzen:
    def __init__(self, model_dir: str):
        from safetensors import safe_open

        with open(os.path.join(model_dir, "config.json")) as fh:
            self.cfg = json.load(fh)
        self.W: Dict[str, torch.Tensor] = {}
        with safe_open(os.path.join(model_dir, "model.safetensors"), "pt") as f:
            for name in f.keys():
                t = f.get_tensor(name)
                self.W[name] = t if t.dtype in (torch.int32, torch.int64) else t.to(torch.float64)
        self.eps = float(self.cfg["norm"]["eps"])

    def mixer(self, i: int, h: torch.Tensor, shared: dict) -> torch.Tensor:
        layer, W, p, eps = self.cfg["layers"][i], self.W, f"l{i}.mix.", self.eps
        m = layer["mixer"]
        if layer["type"] == "attention":
            if m.get("kv_from") is not None:
                return capped_attention(h, W, p, m, eps, kv=shared[int(m["kv_from"])])
            shared[i] = capped_attention_kv(h, W, p, m, eps)
            return capped_attention(h, W, p, m, eps, kv=shared[i])
        if layer["type"] == "delta":
            return gated_delta(h, W, p, m, eps)
        if layer["type"] == "parallel":
            return side_by_side(h, W, p, m, eps)
        raise ValueError(layer["type"])

    def forward(self, tokens: Sequence[int], return_layers: bool = False):
        """Logits [n, vocab] of a whole sequence from position 0 (and the stream after every layer)."""
        cfg, W, eps = self.cfg, self.W, self.eps
        tok = torch.tensor(list(tokens), dtype=torch.long)
        n, width = len(tok), cfg["width"]
        x = W["embed"][tok] * cfg["embedding"]["scale"] + sinusoid(torch.arange(n), width)
        side = cfg.get("token_side")
        shared: dict = {}
        layers: List[torch.Tensor] = []
        for i, layer in enumerate(cfg["layers"]):
            p = f"l{i}."
            x = x + rms(self.mixer(i, x, shared), eps) * (1.0 + W[p + "norm1"])
            if layer.get("mlp") is not None:
                x = x + rms(gated_mlp(x, W, p + "mlp."), eps) * (1.0 + W[p + "norm2"])
            if side is not None:
                x = token_input(x, tok, W, p + "side.", i, int(side["dim"]), eps)
            layers.append(x)
        logits = (rms(x, eps) * (1.0 + W["final.norm"])) @ W["embed"].T
        if cfg.get("logit_softcap"):
            logits = capped(logits, float(cfg["logit_softcap"]))
        return (logits, torch.stack(layers)) if return_layers else logits

    def logits(self, tokens: Sequence[int]) -> torch.Tensor:
        return self.forward(tokens)

    def greedy(self, prompt: Sequence[int], n_new: int) -> List[int]:
        """The prompt's greedy continuation, the whole sequence run again for every new token."""
        seq, out = list(prompt), []
        for _ in range(n_new):
            nxt = int(self.forward(seq)[-1].argmax())
            out.append(nxt)
            seq.append(nxt)
        return out
