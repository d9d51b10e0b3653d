"""Small Gumapel configurations for the tests, their weights and their oracle.

The configurations differ in everything config.json can say: width, vocabulary, number and order
of layers, heads and groups (1, 2, 3 and 4 query heads a kv head), key and value sizes (equal or
not, multiples of 16 or not, one odd), rotated dimensions (all or part of a head), windows (shorter than a
page, longer than a chunk of 256 keys, none), kept first tokens (none, fewer than a page, more
than a page), layers without a feed-forward, layers that take no part in value blending, and a
first blending layer that is not the first layer.  Weights are drawn with a spread of
1 / sqrt(fan-in) and larger q and k, so that scores spread over several units and a key that is
wrongly seen or missed moves the logits.
"""

import json
import math
import random

import torch

import plain_gumapel as plain
from tinyvllm_b200.models import GumapelConfig
from tinyvllm_b200.models.gumapel import GumapelLayer


def _a(heads, kv, dim, vdim, window, *, v_mix=True, ff=None, scale=None):
    return GumapelLayer(type="attention", heads=heads, kv_heads=kv, dim=dim, vdim=vdim,
                        scale=scale or 1.3 / math.sqrt(dim), window=window, v_mix=v_mix, ff=ff)


def _b(heads, kv, dim, vdim, window, keep, rot, base, *, v_mix=True, ff=None, scale=None):
    return GumapelLayer(type="attention_2", heads=heads, kv_heads=kv, dim=dim, vdim=vdim,
                        scale=scale or 1.0 / math.sqrt(dim), window=window, keep_first=keep, rot_dims=rot,
                        rot_base=base, v_mix=v_mix, ff=ff)


GUMAPEL_CONFIGS = {
    # sizes the tensor-core kernels take; a window longer than a chunk of keys; kept tokens past one page
    "p": GumapelConfig(vocab=211, width=64, norm_eps=1e-5, layers=(
        _b(4, 2, 32, 16, 24, 3, 32, 10000.0, ff=96),
        _a(4, 2, 16, 16, 300, ff=96),
        _b(4, 2, 32, 16, 24, 3, 32, 10000.0, ff=None),
        _b(4, 1, 16, 32, 70, 20, 8, 500.0, v_mix=False, ff=128))),
    # sizes they do not take (key size 24, value size 40): the row kernel in both number formats; three
    # query heads a kv head; the first blending layer is the second layer; a layer without a window
    "q": GumapelConfig(vocab=97, width=48, norm_eps=1e-6, layers=(
        _a(3, 1, 24, 40, 9, v_mix=False, ff=64),
        _b(6, 2, 24, 40, 33, 5, 12, 1000000.0, ff=80),
        _a(6, 2, 9, 40, None, ff=None),
        _b(6, 2, 24, 40, 33, 5, 12, 1000000.0, ff=80))),
    # one head a group, equal key and value size 64, a window of one page exactly, nothing kept
    "r": GumapelConfig(vocab=130, width=128, norm_eps=1e-6, layers=(
        _b(2, 2, 64, 64, 16, 0, 64, 50000.0, ff=64),
        _a(2, 2, 64, 64, 16, ff=64))),
}
GUMAPEL_SEEDS = {"p": 11, "q": 12, "r": 13}
GUMAPEL_PAGES = {"p": 16, "q": 8, "r": 16}


def tensors_of(config: GumapelConfig, seed: int) -> dict:
    """Checkpoint tensors (float32) of ``config``, drawn from ``seed``."""
    g = torch.Generator().manual_seed(seed)

    def matrix(rows, cols, gain=1.0):
        return torch.randn(rows, cols, generator=g) * gain / math.sqrt(cols)

    def around_one(n):
        return 1.0 + 0.2 * (torch.rand(n, generator=g) - 0.5)

    d = config.width
    t = {"embed": torch.randn(config.vocab, d, generator=g), "final.norm": around_one(d),
         "head": matrix(config.vocab, d, 2.0)}
    for i, layer in enumerate(config.layers):
        p = f"l{i}."
        t[p + "norm1"] = around_one(d)
        t[p + "mix.q"] = matrix(layer.heads * layer.dim, d, 2.0)
        t[p + "mix.k"] = matrix(layer.kv_heads * layer.dim, d, 2.0)
        t[p + "mix.v"] = matrix(layer.kv_heads * layer.vdim, d)
        t[p + "mix.o"] = matrix(d, layer.heads * layer.vdim)
        if layer.type == "attention":
            t[p + "mix.g"] = matrix(layer.heads * layer.vdim, d, 2.0)
        if layer.v_mix:
            t[p + "mix.vmix"] = torch.rand((), generator=g) * 0.6 + 0.2
        if layer.ff is not None:
            t[p + "mlp.gate"] = matrix(layer.ff, d, 1.5)
            t[p + "mlp.up"] = matrix(layer.ff, d)
            t[p + "mlp.down"] = matrix(d, layer.ff)
    return t


def write_folder(folder, config: GumapelConfig, seed: int, dtype=torch.float32):
    """config.json and model.safetensors of ``config`` in ``folder``.  The values are rounded to
    bfloat16 whatever ``dtype`` stores them as, so that both number formats run the same model."""
    from safetensors.torch import save_file

    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config.to_json(), indent=1), encoding="utf-8")
    tensors = {name: value.to(torch.bfloat16).to(dtype).contiguous() for name, value in tensors_of(config, seed).items()}
    save_file(tensors, str(folder / "model.safetensors"))
    return folder


def read_folder(folder):
    from safetensors import safe_open

    config = json.loads((folder / "config.json").read_text(encoding="utf-8"))
    tensors = {}
    with safe_open(str(folder / "model.safetensors"), framework="pt", device="cpu") as f:
        for name in f.keys():
            tensors[name] = f.get_tensor(name)
    return config, tensors


_oracle: dict = {}


def oracle_logits(folder, requests: dict) -> dict:
    """{request: float64 logits [T, V]} of the plain implementation, remembered per folder and tokens."""
    config, tensors = read_folder(folder)
    out = {}
    for rid, tokens in requests.items():
        key = (str(folder), tuple(tokens))
        if key not in _oracle:
            _oracle[key] = plain.forward(config, tensors, tokens).to(torch.float32)
        out[rid] = _oracle[key]
    return out


def greedy_oracle(folder, prompt, new_tokens: int) -> list[int]:
    config, tensors = read_folder(folder)
    sequence = list(prompt)
    for _ in range(new_tokens):
        sequence.append(int(plain.forward(config, tensors, sequence)[-1].argmax()))
    return sequence[len(prompt):]


def tokens_of(vocab: int, count: int, seed: int) -> list[int]:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(count)]
