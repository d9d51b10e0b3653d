"""Small Kelasun configurations for the tests, their weights and their oracle.

The configurations differ in everything config.json can say: width, vocabulary, number and order of
layers, the residual factor and the logit scale, heads and groups (1, 2 and 3 query heads a kv
head), key and value sizes (equal or not, multiples of 8 or not, one odd), query temperatures (a
period shorter than a page, one longer than the prompts, none), latent sizes (a cached row shorter
than a page's worth of lanes and one wider than 256 elements), rotated parts (with and without
stretched frequencies), experts (one of five, all of three, four of sixteen), shared experts (none,
smaller and larger than an expert) and layers without a feed-forward.  Weights are drawn with a
spread of 1 / sqrt(fan-in), larger for routers and for what makes scores, so that scores spread over
several units, sinks and distance biases matter, and the chosen experts are chosen clearly.
"""

import json
import math
import random

import torch

import plain_kelasun as plain
from tinyvllm_b200.models import KelasunConfig
from tinyvllm_b200.models.kelasun import KelasunExperts, KelasunLayer


def _a(heads, kv, dim, vdim, q_temp, mlp, scale=None):
    return KelasunLayer(type="attention", heads=heads, kv_heads=kv, dim=dim, vdim=vdim,
                        scale=scale or 2.0 / math.sqrt(dim), q_temp=q_temp, mlp=mlp)


def _l(heads, dim, rot_dim, vdim, q_rank, kv_rank, base, scaling, mlp, scale=None):
    return KelasunLayer(type="latent_attention", heads=heads, dim=dim, vdim=vdim,
                        scale=scale or 2.5 / math.sqrt(dim + rot_dim), q_rank=q_rank, kv_rank=kv_rank,
                        rot_dim=rot_dim, rot_base=base if rot_dim else None, rot_scaling=scaling, mlp=mlp)


KELASUN_CONFIGS = {
    # two layers of each kind; a temperature period shorter than a page; stretched frequencies whose ramp
    # lies inside the pairs; a layer without a feed-forward
    "a": KelasunConfig(vocab=150, width=64, norm_eps=1e-5, postln_alpha=1.7, logit_scale=0.5, layers=(
        _a(4, 2, 16, 32, (0.3, 10), KelasunExperts(4, 2, 32, 48)),
        _l(4, 16, 8, 24, 40, 32, 10000.0, (8.0, 64.0, 16.0, 2.0), KelasunExperts(4, 2, 32, 48)),
        _a(4, 2, 16, 32, (0.3, 10), None),
        _l(4, 16, 8, 24, 40, 32, 10000.0, (8.0, 64.0, 16.0, 2.0), KelasunExperts(4, 2, 32, 16)))),
    # sizes no vector access fits (key 9, value 20, latent 20 + 4): three query heads on one kv head, a
    # head a group, no temperature, plain frequencies, two and one expert of five, all experts of three, no shared one
    "b": KelasunConfig(vocab=97, width=48, norm_eps=1e-6, postln_alpha=1.0, logit_scale=3.0, layers=(
        _l(6, 12, 4, 10, 24, 20, 500.0, None, KelasunExperts(5, 2, 24, 0)),
        _a(3, 1, 9, 20, None, KelasunExperts(3, 3, 24, 0)),
        _a(3, 3, 9, 20, (1.5, 300), KelasunExperts(5, 1, 24, 8)))),
    # a cached row wider than 256 elements (the wide form of the row kernel), no rotated part in one
    # layer, four of sixteen experts
    "c": KelasunConfig(vocab=130, width=128, norm_eps=1e-6, postln_alpha=3.0, logit_scale=1.0, layers=(
        _l(2, 32, 64, 32, 64, 256, 200000.0, (3.0, 128.0, 16.0, 1.0), KelasunExperts(16, 4, 16, 16)),
        _a(8, 8, 32, 16, (0.7, 64), KelasunExperts(16, 4, 16, 16)),
        _l(2, 32, 0, 32, 64, 96, None, None, None))),
    # sizes that fit no vector access at all: a width and a vocabulary that are no multiples of four, odd head
    # sizes, a single head, two experts of which one is used, a shared expert of three columns
    "d": KelasunConfig(vocab=101, width=50, norm_eps=1e-5, postln_alpha=2.0, logit_scale=1.5, layers=(
        _a(2, 1, 7, 10, (0.2, 3), KelasunExperts(2, 1, 5, 3)),
        _l(1, 5, 2, 7, 9, 11, 100.0, (2.0, 16.0, 4.0, 1.0), KelasunExperts(2, 2, 6, 0)),
        _l(3, 5, 6, 3, 9, 11, 100.0, None, None),
        _a(1, 1, 7, 10, None, None))),
}
KELASUN_SEEDS = {"a": 21, "b": 22, "c": 23, "d": 24}
KELASUN_PAGES = {"a": 16, "b": 8, "c": 16, "d": 4}


def tensors_of(config: KelasunConfig, seed: int, second_norms: bool = False) -> dict:
    """Checkpoint tensors (float32) of ``config``, drawn from ``seed``.  ``second_norms``: layers without a
    feed-forward hold a second norm all the same."""
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
        hv = layer.heads * layer.vdim
        if layer.type == "attention":
            t[p + "mix.q"] = matrix(layer.heads * layer.dim, d, 2.0)
            t[p + "mix.k"] = matrix(layer.kv_heads * layer.dim, d, 2.0)
            t[p + "mix.v"] = matrix(layer.kv_heads * layer.vdim, d)
            t[p + "mix.q.norm"] = around_one(layer.heads * layer.dim)
            t[p + "mix.k.norm"] = around_one(layer.kv_heads * layer.dim)
            t[p + "mix.sink"] = torch.randn(layer.heads, generator=g) * 1.5
            t[p + "mix.g"] = matrix(layer.heads, d, 2.0)
        else:
            t[p + "mix.dq"] = matrix(layer.q_rank, d)
            t[p + "mix.dq.norm"] = around_one(layer.q_rank)
            t[p + "mix.uq"] = matrix(layer.heads * (layer.dim + layer.rot_dim), layer.q_rank, 1.5)
            t[p + "mix.dkv"] = matrix(layer.kv_rank + layer.rot_dim, d, 1.5)
            t[p + "mix.dkv.norm"] = around_one(layer.kv_rank)
            t[p + "mix.uk"] = matrix(layer.heads * layer.dim, layer.kv_rank, 1.5)
            t[p + "mix.uv"] = matrix(hv, layer.kv_rank)
            t[p + "mix.g"] = matrix(hv, d, 2.0)
        t[p + "mix.o"] = matrix(d, hv)
        if layer.mlp is not None:
            m = layer.mlp
            t[p + "norm2"] = around_one(d)
            t[p + "mlp.router"] = matrix(m.experts, d, 6.0)
            for e in range(m.experts):
                t[p + f"mlp.e{e}.up"] = matrix(m.ff, d, 1.5)
                t[p + f"mlp.e{e}.down"] = matrix(d, m.ff)
            if m.shared_ff:
                t[p + "mlp.shared.up"] = matrix(m.shared_ff, d, 1.5)
                t[p + "mlp.shared.down"] = matrix(d, m.shared_ff)
        elif second_norms:
            t[p + "norm2"] = around_one(d)
    return t


def write_folder(folder, config: KelasunConfig, seed: int, dtype=torch.float32, second_norms: bool = False):
    """config.json and model.safetensors of ``config`` in ``folder``.  The values are rounded to
    bfloat16 whatever ``dtype`` stores them as, so that both number formats run the same model."""
    from safetensors.torch import save_file

    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config.to_json(), indent=1), encoding="utf-8")
    tensors = {name: value.to(torch.bfloat16).to(dtype).contiguous()
               for name, value in tensors_of(config, seed, second_norms).items()}
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
    """{request: float32 logits [T, V]} of the plain implementation, remembered per folder and tokens."""
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
    return plain.greedy(config, tensors, prompt, new_tokens)


def tokens_of(vocab: int, count: int, seed: int) -> list[int]:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(count)]
