"""Kelasun in plain loops and small matrix products: the oracle of the tests.

One function per mechanism, float64 on the CPU, nothing shared with the package.  ``config`` is
the parsed config.json (a dict), ``weights`` a dict of float64 tensors by checkpoint name.

A layer is post-norm: x <- LN1(a x + mixer(x)), then x <- LN2(a x + ff(x)) where the layer has a
feed-forward; a = ``postln_alpha``.  LN is a layer norm with a weight and no bias.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


# ------------------------------------------------------------------ norms
def layer_norm(x, weight, eps):
    mean = x.mean(-1, keepdim=True)
    centred = x - mean
    variance = (centred * centred).mean(-1, keepdim=True)
    return centred / torch.sqrt(variance + eps) * weight


def rms_norm(x, weight, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


# ------------------------------------------------------------------ rotation
def rotary_frequencies(rot):
    """(frequency of every pair, factor on cosine and sine) of a ``rot`` entry."""
    dims, base = rot["dims"], float(rot["base"])
    freqs = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    scaling = rot.get("scaling")
    if not scaling:
        return freqs, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def dim_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(dim_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(scaling["slow"]))), dims - 1)
    out = []
    for i, f in enumerate(freqs):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate_pairs(x, positions, freqs, magnitude):
    """x [tokens, ..., dims]: the pair (2i, 2i+1) turns by position * freqs[i]; cosine and sine are
    multiplied by ``magnitude``."""
    out = x.clone()
    for t, p in enumerate(positions):
        for i, f in enumerate(freqs):
            a = p * f
            c, s = math.cos(a) * magnitude, math.sin(a) * magnitude
            u, v = x[t, ..., 2 * i], x[t, ..., 2 * i + 1]
            out[t, ..., 2 * i] = u * c - v * s
            out[t, ..., 2 * i + 1] = v * c + u * s
    return out


# ------------------------------------------------------------------ mixers
def causal_softmax_rows(scores, sink=None):
    """scores [tokens, tokens] -> weights with key j <= query i; ``sink`` adds exp(sink) to every
    denominator."""
    n = scores.shape[0]
    weights = torch.zeros_like(scores)
    for i in range(n):
        row = scores[i, :i + 1]
        top = row.max() if sink is None else max(row.max().item(), float(sink))
        e = torch.exp(row - top)
        denominator = e.sum() + (math.exp(float(sink) - top) if sink is not None else 0.0)
        weights[i, :i + 1] = e / denominator
    return weights


def biased_sink_attention(h, w, prefix, mixer, eps):
    """The 'attention' mixer: q/k norm over the whole projection, query temperature, distance bias,
    sink, one gate a head."""
    heads, groups, dim, vdim = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    n = h.shape[0]
    q = rms_norm(h @ w[f"{prefix}.q"].T, w[f"{prefix}.q.norm"], eps)
    k = rms_norm(h @ w[f"{prefix}.k"].T, w[f"{prefix}.k.norm"], eps)
    v = h @ w[f"{prefix}.v"].T
    temp = mixer.get("q_temp")
    if temp:
        for p in range(n):
            q[p] = q[p] * (1.0 + temp["coef"] * math.log(math.floor((p + 1) / temp["every"]) + 1))
    gate = torch.sigmoid(h @ w[f"{prefix}.g"].T)                  # [n, heads]
    q, k, v = q.view(n, heads, dim), k.view(n, groups, dim), v.view(n, groups, vdim)
    distance = torch.arange(n, dtype=F64)[:, None] - torch.arange(n, dtype=F64)[None, :]
    out = torch.zeros(n, heads, vdim, dtype=F64)
    for head in range(heads):
        g = head // (heads // groups)
        slope = 2.0 ** (-8.0 * (head + 1) / heads)
        scores = (q[:, head] @ k[:, g].T) * mixer["scale"] - slope * distance
        weights = causal_softmax_rows(scores, sink=w[f"{prefix}.sink"][head])
        out[:, head] = (weights @ v[:, g]) * gate[:, head:head + 1]
    return out.reshape(n, heads * vdim) @ w[f"{prefix}.o"].T


def latent_attention(h, w, prefix, mixer, eps):
    """The 'latent_attention' mixer: queries and keys/values through latents, one rotated key part
    for all heads, a gate on the concatenated heads."""
    heads, dim, rot_dim, vdim, rank = (mixer["heads"], mixer["dim"], mixer["rot_dim"], mixer["vdim"],
                                       mixer["kv_rank"])
    n = h.shape[0]
    positions = list(range(n))
    freqs, magnitude = rotary_frequencies(mixer["rot"]) if rot_dim else ([], 1.0)
    c_q = rms_norm(h @ w[f"{prefix}.dq"].T, w[f"{prefix}.dq.norm"], eps)
    q = (c_q @ w[f"{prefix}.uq"].T).view(n, heads, dim + rot_dim)
    down = h @ w[f"{prefix}.dkv"].T
    c = rms_norm(down[:, :rank], w[f"{prefix}.dkv.norm"], eps)
    k_rot = rotate_pairs(down[:, rank:], positions, freqs, magnitude)          # [n, rot_dim]
    q_rot = rotate_pairs(q[:, :, dim:], positions, freqs, magnitude)
    k_plain = (c @ w[f"{prefix}.uk"].T).view(n, heads, dim)
    v = (c @ w[f"{prefix}.uv"].T).view(n, heads, vdim)
    out = torch.zeros(n, heads, vdim, dtype=F64)
    for head in range(heads):
        scores = (q[:, head, :dim] @ k_plain[:, head].T + q_rot[:, head] @ k_rot.T) * mixer["scale"]
        out[:, head] = causal_softmax_rows(scores) @ v[:, head]
    gated = out.reshape(n, heads * vdim) * torch.sigmoid(h @ w[f"{prefix}.g"].T)
    return gated @ w[f"{prefix}.o"].T


# ------------------------------------------------------------------ feed-forward
def expert(h, up, down):
    z = torch.relu(h @ up.T)
    return (z * z) @ down.T


def routed_experts(h, w, prefix, mlp):
    """Top experts by router logit, weighted by the softmax over the chosen logits, plus the shared
    expert."""
    top = mlp["router"]["top"]
    logits = h @ w[f"{prefix}.router"].T
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen = torch.topk(logits[t], top).indices
        share = torch.softmax(logits[t][chosen], 0)
        for e, s in zip(chosen.tolist(), share):
            out[t] += s * expert(h[t:t + 1], w[f"{prefix}.e{e}.up"], w[f"{prefix}.e{e}.down"])[0]
    if mlp.get("shared"):
        out = out + expert(h, w[f"{prefix}.shared.up"], w[f"{prefix}.shared.down"])
    return out


# ------------------------------------------------------------------ the model
def forward(config, weights, tokens, *, streams=None):
    """Logits [tokens, vocab] of one sequence from position 0; ``streams`` (a list) receives the
    residual stream after every layer."""
    w = {name: tensor.to(F64) for name, tensor in weights.items()}
    eps, alpha = config["norm"]["eps"], config["postln_alpha"]
    x = w["embed"][torch.as_tensor(tokens)]
    for index, layer in enumerate(config["layers"]):
        mix = biased_sink_attention if layer["type"] == "attention" else latent_attention
        x = layer_norm(alpha * x + mix(x, w, f"l{index}.mix", layer["mixer"], eps), w[f"l{index}.norm1"], eps)
        if layer.get("mlp") is not None:
            x = layer_norm(alpha * x + routed_experts(x, w, f"l{index}.mlp", layer["mlp"]),
                           w[f"l{index}.norm2"], eps)
        elif f"l{index}.norm2" in w:          # a second norm without a feed-forward: nothing is added
            x = layer_norm(alpha * x, w[f"l{index}.norm2"], eps)
        if streams is not None:
            streams.append(x.clone())
    x = layer_norm(x, w["final.norm"], eps)
    return (x @ w["head"].T) * config["logit_scale"]


def greedy(config, weights, prompt, new_tokens):
    tokens = list(prompt)
    for _ in range(new_tokens):
        tokens.append(int(forward(config, weights, tokens)[-1].argmax()))
    return tokens[len(prompt):]
