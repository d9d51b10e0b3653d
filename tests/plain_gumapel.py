"""Plain, slow Gumapel: one function per mechanism, whole sequences, no cache.

Written from the design's equations in this file's own notation; shares no code with the package.
Everything runs on the CPU in one floating-point type (float64 by default), with loops where a
loop is the clearest form.  ``forward`` takes the parsed config.json and a dict of tensors by
checkpoint name and returns the logits of every position (and, if asked, the stream after
every layer).

Notation: T tokens, D width, H query heads, G key/value heads, dk and dv the per-head sizes of
keys and values, W the window, S the number of first tokens a window keeps.
"""

from __future__ import annotations

import math

import torch


# ------------------------------------------------------------------ pointwise
def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return rms_unit(x, eps) * weight


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gated_feed_forward(h, w_gate, w_up, w_down):
    """down . (gelu_tanh(gate . h) * (up . h)) for h [T, D]."""
    return (gelu_tanh(h @ w_gate.T) * (h @ w_up.T)) @ w_down.T


# ------------------------------------------------------------------- rotation
def rotate_interleaved(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, heads, d]: the pairs (2i, 2i + 1), i < dims / 2, of every head turn by
    position * base^(-2i / dims); dimensions from ``dims`` on stay."""
    out = x.clone()
    for i in range(dims // 2):
        frequency = base ** (-2.0 * i / dims)
        angle = positions.to(x.dtype) * frequency                    # [T]
        c, s = torch.cos(angle)[:, None], torch.sin(angle)[:, None]
        u, v = x[:, :, 2 * i], x[:, :, 2 * i + 1]
        out[:, :, 2 * i] = u * c - v * s
        out[:, :, 2 * i + 1] = v * c + u * s
    return out


# ----------------------------------------------------------------------- mask
def visible(i: int, j: int, window: int | None, keep_first: int) -> bool:
    """Whether the query at position i sees the key at position j."""
    if j > i:
        return False
    if window is None or i - j < window:
        return True
    return j < keep_first


def masked_attention(q, k, v, scale: float, window: int | None, keep_first: int = 0, first_position: int = 0):
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] of one sequence -> [T, H, dv]; softmax over the
    visible keys of each query, query head h with key/value head h // (H / G)."""
    tokens, heads, _ = q.shape
    group = heads // k.shape[1]
    out = torch.zeros(tokens, heads, v.shape[2], dtype=q.dtype)
    for h in range(heads):
        g = h // group
        for i in range(tokens):
            seen = [j for j in range(i + 1) if visible(first_position + i, first_position + j, window, keep_first)]
            scores = (k[seen, g] * q[i, h]).sum(dim=-1) * scale
            weights = torch.softmax(scores, dim=0)
            out[i, h] = (weights[:, None] * v[seen, g]).sum(dim=0)
    return out


def mix_values(v, v_first, lam):
    """(1 - lam) v + lam v_first"""
    return (1.0 - lam) * v + lam * v_first


# --------------------------------------------------------------------- mixers
def attention_mixer(kind: str, sizes: dict, tensors: dict, prefix: str, h, positions, eps: float,
                    v_first):
    """One mixer of kind 'attention' (unit-norm q and k, plain window, output gate) or
    'attention_2' (rotated q and k, window that keeps first tokens).  Returns (output [T, D],
    the values it would hand on as v_first or None)."""
    heads, kv_heads, dk, dv = sizes["heads"], sizes["kv_heads"], sizes["dim"], sizes["vdim"]
    tokens = h.shape[0]
    q = (h @ tensors[prefix + "q"].T).view(tokens, heads, dk)
    k = (h @ tensors[prefix + "k"].T).view(tokens, kv_heads, dk)
    v = (h @ tensors[prefix + "v"].T).view(tokens, kv_heads, dv)
    mask = sizes.get("mask") or {}
    window, keep = mask.get("size"), 0
    if kind == "attention":
        q, k = rms_unit(q, eps), rms_unit(k, eps)
    elif kind == "attention_2":
        rot = sizes["rot"]
        q = rotate_interleaved(q, positions, rot["dims"], rot["base"])
        k = rotate_interleaved(k, positions, rot["dims"], rot["base"])
        keep = mask.get("keep_first", 0)
    else:
        raise ValueError(kind)
    handed_on = None
    if sizes.get("v_mix"):
        if v_first is None:
            handed_on = v
        else:
            v = mix_values(v, v_first, tensors[prefix + "vmix"])
    mixed = masked_attention(q, k, v, sizes["scale"], window, keep).reshape(tokens, heads * dv)
    if kind == "attention":
        mixed = mixed * torch.sigmoid(h @ tensors[prefix + "g"].T)
    return mixed @ tensors[prefix + "o"].T, handed_on


# ---------------------------------------------------------------------- model
def forward(config: dict, tensors: dict, token_ids, *, dtype=torch.float64, layers_out: list | None = None):
    """Logits [T, vocab] of one sequence from position 0."""
    t = {name: (value.to(dtype) if value.is_floating_point() else value) for name, value in tensors.items()}
    eps = config["norm"]["eps"]
    ids = torch.as_tensor(token_ids, dtype=torch.long)
    positions = torch.arange(ids.shape[0])
    x = t["embed"][ids]
    v_first = None
    for index, layer in enumerate(config["layers"]):
        prefix = f"l{index}."
        h = rms_norm(x, t[prefix + "norm1"], eps)
        mixed, handed_on = attention_mixer(layer["type"], layer["mixer"], t, prefix + "mix.", h, positions, eps,
                                           v_first)
        if handed_on is not None:
            v_first = handed_on
        update = mixed
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(layer["mlp"]["kind"])
            update = update + gated_feed_forward(h, t[prefix + "mlp.gate"], t[prefix + "mlp.up"],
                                                 t[prefix + "mlp.down"])
        x = x + update
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, t["final.norm"], eps) @ t["head"].T
