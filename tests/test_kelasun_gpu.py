"""Kelasun on the GPU against the plain implementation: each mechanism alone, then whole models
through the step function, the trace program and the generation entry point."""

import json
import math
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import plain_kelasun as plain
import replay_helpers as rh
from kelasun_configs import (KELASUN_CONFIGS, KELASUN_PAGES, KELASUN_SEEDS, greedy_oracle, oracle_logits,
                             tokens_of, write_folder)

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]
IDS = ["f32", "bf16"]
CUDA = "cuda:0"
F64 = torch.float64
# angles are float32 products of position and frequency: at position 1,500 they are off by up to 1e-4
# of a radian against the plain implementation's float64 angles
ANGLE_LIMIT = 1.5e-4


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: write_folder(tmp_path_factory.mktemp(f"kelasun_{name}"), config, KELASUN_SEEDS[name])
            for name, config in KELASUN_CONFIGS.items()}


def close(got, want, dtype, scale=None, limit=None):
    scale = scale if scale is not None else max(want.abs().max().item(), 1e-6)
    limit = limit or (4e-6 if dtype == torch.float32 else 1.2e-2)
    worst = (got.double().cpu() - want.double().cpu()).abs().max().item() / scale
    assert worst <= limit, f"largest difference {worst:.3g} of the scale, allowed {limit:.3g}"


def rounded(t, dtype):
    """Values of ``t`` as ``dtype`` stores them, in float64."""
    return t.to(dtype).double()


# ------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("width", [40, 384, 1030])
def test_layer_norm_behind_the_residual_sum(width, dtype):
    from tinyvllm_b200.ops import kernels

    g = torch.Generator().manual_seed(width)
    x = torch.randn(9, width, generator=g) * 3 + 0.7
    y = torch.randn(9, width, generator=g).to(dtype)
    w = (1 + 0.3 * torch.randn(width, generator=g)).to(dtype)
    want = plain.layer_norm(2.5 * x.double() + y.double(), w.double(), 1e-5)
    out, stream = kernels.post_layer_norm(x.to(CUDA), w.to(CUDA), 1e-5, alpha=2.5, add=y.to(CUDA), out_dtype=dtype)
    assert stream.dtype == torch.float32 and out.dtype == dtype
    close(stream, want, torch.float32)
    close(out, want, dtype)
    # a stream that starts in the storage type (the embedding), no addend, chosen rows only
    start = x.to(dtype)
    rows = torch.tensor([7, 0, 3], dtype=torch.int32, device=CUDA)
    some, nothing = kernels.post_layer_norm(start.to(CUDA), w.to(CUDA), 1e-5, rows=rows, out_dtype=dtype)
    close(some, plain.layer_norm(start.double(), w.double(), 1e-5)[[7, 0, 3]], dtype)
    # a row does not depend on the rows beside it
    alone, _ = kernels.post_layer_norm(x[4:5].to(CUDA), w.to(CUDA), 1e-5, alpha=2.5, add=y[4:5].to(CUDA), out_dtype=dtype)
    assert torch.equal(alone[0], out[4])


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("q_cols,k_cols,extra,kd,vd", [(44, 18, 7, 9, 3), (64, 32, 24, 16, 8), (1024, 256, 64, 128, 32)])
def test_norm_over_whole_projections_and_query_temperature(q_cols, k_cols, extra, kd, vd, dtype):
    """Sizes that fit no 16-byte access, and sizes that do (the kernel then moves eight values at a time)."""
    from tinyvllm_b200.ops import kernels

    g = torch.Generator().manual_seed(5)
    proj = (torch.randn(6, q_cols + k_cols + extra, generator=g) * 2).to(dtype)
    qw = (1 + 0.3 * torch.randn(q_cols, generator=g)).to(dtype)
    kw = (1 + 0.3 * torch.randn(k_cols, generator=g)).to(dtype)
    positions = [0, 8, 9, 10, 29, 4000]
    coef, every = 0.4, 10
    want = proj.double().clone()
    q = plain.rms_norm(want[:, :q_cols], qw.double(), 1e-5)
    for t, p in enumerate(positions):
        q[t] *= 1.0 + coef * math.log(math.floor((p + 1) / every) + 1)
    want[:, :q_cols] = q
    want[:, q_cols:q_cols + k_cols] = plain.rms_norm(want[:, q_cols:q_cols + k_cols], kw.double(), 1e-5)
    dev = proj.to(CUDA)
    kernels.projection_norm(dev, [(0, q_cols, qw.to(CUDA), True), (q_cols, k_cols, kw.to(CUDA), False)],
                            torch.tensor(positions, dtype=torch.int32, device=CUDA), 1e-5, temperature=(coef, every))
    close(dev, want, dtype)
    assert torch.equal(dev[:, q_cols + k_cols:].cpu(), proj[:, q_cols + k_cols:])          # the rest is untouched
    # the same launch may store: the second segment as 2 kv heads of keys, and 2 heads of values from the rest
    page, pages = 4, 4
    key_cache = torch.full((pages, 2, page, kd), float("nan"), dtype=dtype, device=CUDA)
    value_cache = torch.full((pages, 2, page, vd), float("nan"), dtype=dtype, device=CUDA)
    slots = [5, 0, 15, 9, -1, 2]
    again = proj.to(CUDA)
    kernels.projection_norm(again, [(0, q_cols, qw.to(CUDA), True), (q_cols, k_cols, kw.to(CUDA), False)],
                            torch.tensor(positions, dtype=torch.int32, device=CUDA), 1e-5, temperature=(coef, every),
                            store=dict(slots=torch.tensor(slots, dtype=torch.int32, device=CUDA), key_cache=key_cache,
                                       value_cache=value_cache, v_at=q_cols + k_cols))
    assert torch.equal(again, dev)
    for t, slot in enumerate(slots):
        if slot < 0:
            continue
        for head in range(2):
            assert torch.equal(key_cache[slot // page, head, slot % page], dev[t, q_cols + kd * head:q_cols + kd * head + kd])
            assert torch.equal(value_cache[slot // page, head, slot % page],
                               proj[t, q_cols + k_cols + vd * head:q_cols + k_cols + vd * head + vd].to(CUDA))
    assert torch.isnan(key_cache.float()).sum().item() == (pages * page - 5) * 2 * kd      # no other row was touched
    if dtype == torch.bfloat16:
        # norm weights that a checkpoint stores in 32-bit stay so: the same values give the same result
        wide = proj.to(CUDA)
        kernels.projection_norm(wide, [(0, q_cols, qw.float().to(CUDA), True), (q_cols, k_cols, kw.float().to(CUDA), False)],
                                torch.tensor(positions, dtype=torch.int32, device=CUDA), 1e-5, temperature=(coef, every))
        assert torch.equal(wide, dev)
    # positions 8 and 9 lie on the two sides of a period's edge: (p + 1) / every is 0 and then 1
    ratio = (dev[2, :q_cols].double() / want[2, :q_cols].cuda()).mean().item()
    assert ratio == pytest.approx(1.0, abs=2e-2)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("q_rank,kv_rank,rot_dim", [(24, 20, 4), (40, 32, 8), (64, 256, 64), (16, 48, 0)])
def test_latents_norms_rotation_and_cache_rows(q_rank, kv_rank, rot_dim, dtype):
    from tinyvllm_b200.ops import kernels

    g = torch.Generator().manual_seed(q_rank)
    tokens, page, pages = 7, 4, 5
    proj = (torch.randn(tokens, 3 + q_rank + kv_rank + rot_dim + 5, generator=g) * 2).to(dtype)
    qw = (1 + 0.3 * torch.randn(q_rank, generator=g)).to(dtype)
    kw = (1 + 0.3 * torch.randn(kv_rank, generator=g)).to(dtype)
    rot = {"dims": rot_dim, "base": 300.0, "scaling": {"factor": 4.0, "original": 32.0, "fast": 8.0, "slow": 1.0}}
    freqs, magnitude = plain.rotary_frequencies(rot) if rot_dim else ([], 1.0)
    positions = [0, 1, 2, 77, 1500, 31, 32]
    slots = [9, 0, 17, 3, 12, 5, 19]
    cache = torch.full((pages, 1, page, kv_rank + rot_dim), float("nan"), dtype=dtype, device=CUDA)
    inv_freq = torch.tensor(freqs, dtype=torch.float32, device=CUDA) if rot_dim else None
    q_latent = kernels.latent_prepare(
        proj.to(CUDA), dq_at=3, q_rank=q_rank, q_weight=qw.to(CUDA), dkv_at=3 + q_rank, kv_rank=kv_rank,
        kv_weight=kw.to(CUDA), rot_dim=rot_dim, inv_freq=inv_freq, magnitude=magnitude,
        positions=torch.tensor(positions, dtype=torch.int32, device=CUDA),
        slots=torch.tensor(slots, dtype=torch.int32, device=CUDA), key_cache=cache, eps=1e-5)
    p64 = proj.double()
    close(q_latent, plain.rms_norm(p64[:, 3:3 + q_rank], qw.double(), 1e-5), dtype)
    latent = plain.rms_norm(p64[:, 3 + q_rank:3 + q_rank + kv_rank], kw.double(), 1e-5)
    rows = cache.view(-1, kv_rank + rot_dim)[torch.tensor(slots, device=CUDA)]
    close(rows[:, :kv_rank], latent, dtype)
    if rot_dim:
        turned = plain.rotate_pairs(p64[:, 3 + q_rank + kv_rank:3 + q_rank + kv_rank + rot_dim], positions, freqs, magnitude)
        close(rows[:, kv_rank:], turned, dtype, limit=ANGLE_LIMIT if dtype == torch.float32 else None)
    written = torch.zeros(pages * page, dtype=torch.bool)
    written[slots] = True
    assert torch.isnan(cache.view(-1, kv_rank + rot_dim)[~written.to(CUDA)].float()).all()    # no other slot touched
    if rot_dim:
        # the query side: heads with strides of their own
        heads = 3
        src = (torch.randn(tokens, heads, 10 + rot_dim, generator=g)).to(dtype)
        dst = torch.zeros(tokens, heads, kv_rank + rot_dim, dtype=dtype, device=CUDA)
        kernels.rotate_heads(src.to(CUDA)[:, :, 10:], dst[:, :, kv_rank:], inv_freq, magnitude,
                             torch.tensor(positions, dtype=torch.int32, device=CUDA))
        close(dst[:, :, kv_rank:], plain.rotate_pairs(src.double()[:, :, 10:], positions, freqs, magnitude), dtype,
              limit=ANGLE_LIMIT if dtype == torch.float32 else None)
        assert (dst[:, :, :kv_rank] == 0).all()


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("tokens,heads,n,k", [(1, 3, 10, 20), (13, 6, 24, 9), (70, 2, 256, 32), (9, 4, 16, 512)])
def test_a_product_a_head_with_a_gate(tokens, heads, n, k, dtype):
    from tinyvllm_b200.ops import kernels

    g = torch.Generator().manual_seed(n + k)
    x = torch.randn(tokens, heads, k + 5, generator=g).to(dtype)
    w = (torch.randn(heads, n, k, generator=g) / math.sqrt(k)).to(dtype)
    gate = torch.randn(tokens, heads * n + 3, generator=g).to(dtype)
    want = torch.einsum("thk,hnk->thn", x.double()[:, :, 2:2 + k], w.double())
    out = torch.zeros(tokens, heads, n + 4, dtype=dtype, device=CUDA)
    kernels.head_product(x.to(CUDA)[:, :, 2:2 + k], w.to(CUDA), out[:, :, 1:1 + n])
    close(out[:, :, 1:1 + n], want, dtype)
    assert (out[:, :, 0] == 0).all() and (out[:, :, 1 + n:] == 0).all()
    kernels.head_product(x.to(CUDA)[:, :, 2:2 + k], w.to(CUDA), out[:, :, 1:1 + n], gate=gate.to(CUDA)[:, :heads * n])
    close(out[:, :, 1:1 + n], want * torch.sigmoid(gate.double()[:, :heads * n]).view(tokens, heads, n), dtype)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("experts,top,ff,shared", [(5, 1, 24, 0), (3, 3, 8, 16), (16, 4, 16, 16), (40, 6, 7, 3)])
def test_routing_weights_and_activation(experts, top, ff, shared, dtype):
    from tinyvllm_b200.ops import kernels

    g = torch.Generator().manual_seed(experts)
    tokens = 11
    logits = torch.randn(tokens, experts, generator=g) * 3
    up = torch.randn(tokens, experts * ff + shared, generator=g).to(dtype)
    weights = torch.empty(tokens, experts, dtype=torch.float32, device=CUDA)
    out = kernels.route_act(logits.to(CUDA), up.to(CUDA), experts=experts, top=top, ff=ff, shared_ff=shared,
                            weights_out=weights)
    want_w = torch.zeros(tokens, experts, dtype=F64)
    for t in range(tokens):
        chosen = torch.topk(logits[t].double(), top).indices
        want_w[t, chosen] = torch.softmax(logits[t].double()[chosen], 0)
    close(weights, want_w, torch.float32)
    assert ((weights > 0).sum(1) == top).all()
    act = torch.relu(up.double()) ** 2
    want = act.clone()
    want[:, :experts * ff] = (act[:, :experts * ff].view(tokens, experts, ff) * want_w[:, :, None]).view(tokens, -1)
    close(out, want, dtype)
    assert (out[:, :experts * ff].view(tokens, experts, ff)[weights == 0] == 0).all()     # exact zeros


def _paged(keys, values, page, dtype, seed, fill=float("nan")):
    """Keys [n, kv, dk] and values [n, kv, dv] of one request spread over shuffled pages."""
    n, kv, dk = keys.shape
    count = -(-n // page)
    order = list(range(count + 3))
    import random
    random.Random(seed).shuffle(order)
    table = order[:count]
    key_cache = torch.full((count + 3, kv, page, dk), fill, dtype=dtype)
    value_cache = None if values is None else torch.full((count + 3, kv, page, values.shape[2]), fill, dtype=dtype)
    for j in range(n):
        key_cache[table[j // page], :, j % page] = keys[j].to(dtype)
        if values is not None:
            value_cache[table[j // page], :, j % page] = values[j].to(dtype)
    return key_cache, value_cache, torch.tensor([table], dtype=torch.int32)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("kind", ["rows", "split", "tiles", "singles"])
@pytest.mark.parametrize("heads,kv,dk,dv", [(4, 2, 16, 32), (3, 1, 9, 20), (8, 8, 32, 16), (40, 2, 16, 16)])
def test_attention_with_distance_bias_sink_and_head_gate(heads, kv, dk, dv, kind, dtype):
    """Random scores plus one key per checked query that is made to stand out: far back (position 3 from
    position 700), at both sides of a page border and of a chunk border of 256 keys, the query's own.
    The distance bias takes slope * distance off it, the sink shares the denominator, the gate is one
    number a head."""
    from tinyvllm_b200.ops import kernels

    if kind in ("tiles", "singles") and (dtype != torch.bfloat16 or dk % 16 or dv % 16):
        pytest.skip("the tensor-core kernels take bfloat16 and sizes in steps of 16")
    n, page, scale = 701, 8, 0.4
    g = torch.Generator().manual_seed(heads * 100 + dk)
    q = torch.randn(n, heads, dk, generator=g)
    k = torch.randn(n, kv, dk, generator=g)
    v = torch.randn(n, kv, dv, generator=g)
    checked = {700: 3, 699: 255, 698: 256, 697: 8 * 31, 696: 8 * 31 - 1, 695: 695, 0: 0, 1: 0, 300: 299}
    slope_0 = 2.0 ** (-8.0 / heads)
    axis = {key: i for i, key in enumerate(sorted(set(checked.values())))}
    for key, i in axis.items():
        k[key, 0] = 0.0
        k[key, 0, i] = 62.5           # a long key along an axis of its own
    for query, key in checked.items():
        # this query's first head looks along that axis: a score of 100 after the distance bias, where the
        # other keys stay within a few units
        q[query, 0] = 0.0
        q[query, 0, axis[key]] = 4.0 * (100.0 + slope_0 * (query - key)) / 100.0
    q, k, v = rounded(q, dtype), rounded(k, dtype), rounded(v, dtype)
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)], dtype=F64)
    sinks = torch.randn(heads, generator=g).double() * 2
    sinks[0] = 100.0                  # as strong as the key that stands out for the first head
    gate = rounded(torch.randn(n, heads, generator=g), dtype)
    rows = sorted(checked)
    want = torch.zeros(len(rows), heads, dv, dtype=F64)
    for h in range(heads):
        group = h // (heads // kv)
        distance = torch.arange(n, dtype=F64)[:, None] - torch.arange(n, dtype=F64)[None, :]
        scores = (q[:, h] @ k[:, group].T) * scale - slopes[h] * distance
        weights = plain.causal_softmax_rows(scores, sink=sinks[h])
        want[:, h] = (weights @ v[:, group])[rows] * torch.sigmoid(gate[rows, h:h + 1])
    key_cache, value_cache, table = _paged(k, v, page, dtype, 3, fill=float("nan") if kind in ("rows", "split") else 1e30)
    extras = dict(gate_per_head=True, slopes=slopes.float().to(CUDA), sinks=sinks.float().to(CUDA))
    if kind in ("rows", "split"):
        positions = torch.tensor(rows, dtype=torch.int32, device=CUDA)
        chunks = 3 if kind == "split" else 0
        scratch = torch.empty(kernels.attention_rows_scratch_floats(len(rows), heads, dv, 3), dtype=torch.float32,
                              device=CUDA) if chunks else None
        got = kernels.attention_rows(
            q[rows].to(dtype).reshape(len(rows), heads * dk).to(CUDA), heads * dk, key_cache.to(CUDA), value_cache.to(CUDA),
            table.to(CUDA), torch.zeros(len(rows), dtype=torch.int32, device=CUDA), positions, num_q=heads, num_kv=kv,
            head_dim=dk, value_dim=dv, window=None, scale=scale, gate=gate[rows].to(dtype).to(CUDA), **extras,
            scratch=scratch, max_chunks=chunks)
    elif kind == "tiles":
        # the whole prompt in tiles of up to 64 tokens, cut at odd places
        firsts = [0, 1, 3, 50] + list(range(114, n, 64))
        counts = [b - a for a, b in zip(firsts, firsts[1:] + [n])]
        ints = lambda values: torch.tensor(values, dtype=torch.int32, device=CUDA)
        out = torch.empty(n, heads * dv, dtype=dtype, device=CUDA)
        kernels.attention_tiles(
            q.to(dtype).reshape(n, heads * dk).to(CUDA), key_cache.to(CUDA), value_cache.to(CUDA), table.to(CUDA),
            ints(list(range(n))), ints([0] * len(firsts)), ints(firsts), ints(counts), num_q=heads, num_kv=kv, key_dim=dk,
            value_dim=dv, window=None, keep_first=0, scale=scale, out=out, gate=gate.to(dtype).to(CUDA), **extras)
        got = out[rows]
    else:
        out = torch.empty(len(rows), heads * dv, dtype=dtype, device=CUDA)
        need = kernels.attention_tiles_singles_floats(len(rows), heads, dv, None, 0, 704)
        kernels.attention_tiles_singles(
            q[rows].to(dtype).reshape(len(rows), heads * dk).to(CUDA), key_cache.to(CUDA), value_cache.to(CUDA),
            table.to(CUDA), torch.tensor(rows, dtype=torch.int32, device=CUDA),
            torch.zeros(len(rows), dtype=torch.int32, device=CUDA), num_q=heads, num_kv=kv, key_dim=dk, value_dim=dv,
            window=None, keep_first=0, scale=scale, max_context=704,
            scratch=torch.empty(need, dtype=torch.float32, device=CUDA), out=out, gate=gate[rows].to(dtype).to(CUDA),
            **extras)
        got = out
    # scores of a hundred and more carry float32 rounding of 1e-5 into their exponentials
    close(got.view(len(rows), heads, dv), want, dtype, scale=want.abs().max().item(),
          limit=3e-5 if dtype == torch.float32 else None)
    # the far key carries weight: it and the sink share the first head's denominator at position 700 (in
    # bfloat16 the rounding of q moves the score by up to half a unit, and the shares with it)
    far = rows.index(700)
    alone = torch.sigmoid(gate[700, 0]) * v[3, 0]
    share = (want[far, 0] @ alone / (alone @ alone)).item()
    assert 0.1 < share < 0.9
    assert (want[far, 0] - share * alone).abs().max() < 0.05 * alone.abs().max()


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("rank,rot", [(20, 4), (32, 8), (48, 16), (256, 64)])
def test_attention_whose_values_lie_inside_the_key_rows(rank, rot, dtype):
    """One kv head whose rows are [latent | rotated part]: the values are the first ``rank`` elements of
    the same rows; a far key stands out."""
    from tinyvllm_b200.ops import kernels

    n, page, heads, scale = 530, 16, 3, 0.3
    g = torch.Generator().manual_seed(rank)
    q = torch.randn(n, heads, rank + rot, generator=g)
    rows_kv = torch.randn(n, 1, rank + rot, generator=g)
    q[529, 1] = rows_kv[2, 0] * (60.0 / scale / rows_kv[2, 0].pow(2).sum())
    q, rows_kv = rounded(q, dtype), rounded(rows_kv, dtype)
    checked = [0, 1, 255, 256, 257, 511, 512, 529]
    want = torch.zeros(len(checked), heads, rank, dtype=F64)
    for h in range(heads):
        weights = plain.causal_softmax_rows((q[:, h] @ rows_kv[:, 0].T) * scale)
        want[:, h] = (weights @ rows_kv[:, 0, :rank])[checked]
    key_cache, _, table = _paged(rows_kv, None, page, dtype, 4)
    ints = lambda values: torch.tensor(values, dtype=torch.int32, device=CUDA)
    for chunks in (0, 3):
        scratch = torch.empty(kernels.attention_rows_scratch_floats(len(checked), heads, rank, 3), dtype=torch.float32,
                              device=CUDA) if chunks else None
        got = kernels.attention_rows(
            q[checked].to(dtype).reshape(len(checked), -1).to(CUDA), heads * (rank + rot), key_cache.to(CUDA), None,
            table.to(CUDA), torch.zeros(len(checked), dtype=torch.int32, device=CUDA), ints(checked), num_q=heads,
            num_kv=1, head_dim=rank + rot, value_dim=rank, value_offset=0, window=None, scale=scale, scratch=scratch,
            max_chunks=chunks)
        close(got.view(len(checked), heads, rank), want, dtype)
    if dtype == torch.bfloat16 and kernels.attention_tiles_supports(rank + rot, rank, heads, 1, value_in_key=True):
        key_cache, _, table = _paged(rows_kv, None, page, dtype, 4, fill=1e30)
        sizes = dict(num_q=heads, num_kv=1, key_dim=rank + rot, value_dim=rank, window=None, keep_first=0, scale=scale)
        firsts = [0, 2, 9] + list(range(73, n, 64))
        counts = [b - a for a, b in zip(firsts, firsts[1:] + [n])]
        out = torch.empty(n, heads * rank, dtype=dtype, device=CUDA)
        kernels.attention_tiles(q.to(dtype).reshape(n, -1).to(CUDA), key_cache.to(CUDA), None, table.to(CUDA),
                                ints(list(range(n))), ints([0] * len(firsts)), ints(firsts), ints(counts), **sizes, out=out)
        close(out[checked].view(len(checked), heads, rank), want, dtype)
        out = torch.empty(len(checked), heads * rank, dtype=dtype, device=CUDA)
        need = kernels.attention_tiles_singles_floats(len(checked), heads, rank, None, 0, 544)
        kernels.attention_tiles_singles(
            q[checked].to(dtype).reshape(len(checked), -1).to(CUDA), key_cache.to(CUDA), None, table.to(CUDA),
            ints(checked), ints([0] * len(checked)), **sizes, max_context=544,
            scratch=torch.empty(need, dtype=torch.float32, device=CUDA), out=out)
        close(out.view(len(checked), heads, rank), want, dtype)
    assert (want[-1, 1] - rows_kv[2, 0, :rank]).abs().max() < 0.05 * rows_kv[2, 0, :rank].abs().max()


# ---------------------------------------------------------------- whole models
def requests_of(name):
    vocab = KELASUN_CONFIGS[name].vocab
    return {f"{name}{n}": tokens_of(vocab, n, 500 + n) for n in (1, 2, 37, 150, 420)}


def make_runner(folder, dtype, page, pages, max_len=None):
    from tinyvllm_b200 import read_model_config
    from tinyvllm_b200.engine.model import Model
    from tinyvllm_b200.engine.step import StepRunner

    model = Model(read_model_config(folder).to_spec(), device=CUDA, dtype=dtype).load(folder)
    return StepRunner(model, page_size=page, num_pages=pages, max_requests=4, max_model_len=max_len or pages * page)


def compare(got: dict, folder, requests, dtype):
    """float32: every row within rounding of the plain logits.  bfloat16: 16-bit activations move a router
    logit by a hundredth of its size, and a token whose last chosen expert led the next one by less than
    that goes to another expert than in the plain implementation (with one expert a token, to a wholly
    different feed-forward); so the bfloat16 rows are judged as a whole: the median row and nine rows in
    ten within the rounding of 16-bit activations.  (Observed: medians 0.005 to 0.010, the ninth decile
    0.009 to 0.035; float32 rows 5e-6 at most.)"""
    expected = oracle_logits(folder, requests)
    assert got, "no logits came back"
    errors = []
    for (rid, position), row in got.items():
        want = expected[rid]
        assert torch.isfinite(row).all()
        errors.append((row.double() - want[position].double()).abs().max().item() / want.abs().max().item())
    errors.sort()
    if dtype == torch.float32:
        assert errors[-1] <= 3e-5, f"largest difference {errors[-1]:.3g} of the largest logit"
        return
    median, ninth = errors[len(errors) // 2], errors[len(errors) * 9 // 10]
    assert median <= 2e-2 and ninth <= 5e-2, f"median {median:.3g}, ninth decile {ninth:.3g} of the largest logit"


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", sorted(KELASUN_CONFIGS))
@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed"])
def test_every_way_of_cutting_gives_the_plain_logits(cut, name, dtype, folders):
    """Whole prompts; prompts whose last 40 tokens come one by one; portions of changing size down to two
    tokens; up to four live requests with portions beside single tokens, in a pool with room for little
    more than the live tokens, so that pages that finished requests gave back are taken again."""
    requests = requests_of(name)
    page = KELASUN_PAGES[name]
    steps = {"whole": lambda: rh.whole(requests), "tail": lambda: rh.tail_by_one(requests, 40),
             "portions": lambda: rh.portions(requests, 3, sizes=(2, 3, 5, 8, 13, 31, 64, 100, 200)),
             "mixed": lambda: rh.mixed(requests, 4, live=4, decode_tail=20, sizes=(2, 3, 7, 16, 40, 90))}[cut]()
    pages = -(-rh.live_token_need(steps, page) // page) if cut == "mixed" else max(64, -(-448 // page))
    runner = make_runner(folders[name], dtype, page, pages)
    with torch.inference_mode():
        got = rh.run_steps(runner, steps)
    compare(got, folders[name], requests, dtype)
    assert not runner.manager.open_requests()
    assert all(runner.manager.free_pages(g) == pages for g in range(len(runner.manager.groups)))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_a_request_is_not_moved_by_its_neighbours(dtype, folders):
    """The same request alone and beside three others, in other pages and slots: equal beyond rounding."""
    name = "a"
    requests = requests_of(name)
    page = KELASUN_PAGES[name]
    alone = {"x": requests["a150"]}
    with torch.inference_mode():
        first = rh.run_steps(make_runner(folders[name], dtype, page, 64), rh.portions(alone, 9, sizes=(7, 50)))
        crowd = dict(list(requests.items())[2:])
        crowd["x"] = requests["a150"]
        second = rh.run_steps(make_runner(folders[name], dtype, page, 96), rh.mixed(crowd, 1, live=4, decode_tail=5))
    scale = oracle_logits(folders[name], alone)["x"].abs().max().item()
    errors = sorted((first[key].double() - second[key].double()).abs().max().item() / scale for key in first)
    if dtype == torch.float32:
        assert errors[-1] <= 1e-5
    else:
        assert errors[len(errors) * 39 // 40 - 1] <= 2e-2


def test_a_second_norm_without_a_feed_forward(tmp_path):
    """A checkpoint that holds the second norm of a layer without a feed-forward: the layer then ends with
    x <- norm2(alpha x)."""
    name = "a"
    folder = write_folder(tmp_path / "with_norms", KELASUN_CONFIGS[name], KELASUN_SEEDS[name], second_norms=True)
    requests = {"n": tokens_of(KELASUN_CONFIGS[name].vocab, 90, 77)}
    runner = make_runner(folder, torch.float32, 16, 16)
    with torch.inference_mode():
        got = rh.run_steps(runner, rh.portions(requests, 5, sizes=(2, 9, 40)))
    compare(got, folder, requests, torch.float32)
    plain_logits = oracle_logits(write_folder(tmp_path / "without", KELASUN_CONFIGS[name], KELASUN_SEEDS[name]), requests)["n"]
    assert (plain_logits - oracle_logits(folder, requests)["n"]).abs().max() > 1e-3          # the norm matters


def test_long_decoding(folders):
    """A prompt of five tokens and 330 tokens decoded one by one, float32, past a chunk border of the
    keys and several periods of the query temperature."""
    name = "a"
    tokens = tokens_of(KELASUN_CONFIGS[name].vocab, 335, 9)
    requests = {"long": tokens}
    runner = make_runner(folders[name], torch.float32, 16, 22, max_len=352)
    with torch.inference_mode():
        got = rh.run_steps(runner, rh.tail_by_one(requests, 330))
    compare(got, folders[name], requests, torch.float32)


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
def test_trace_program(dtype_name, folders, tmp_path):
    name = "b"
    requests = requests_of(name)
    steps = rh.mixed(requests, 2, live=3)
    need = rh.live_token_need(steps)
    lines = "\n".join(json.dumps(step) for step in steps) + "\n"
    out = tmp_path / "out"
    root = Path(__file__).resolve().parent.parent
    done = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(folders[name]),
                           "--dtype", dtype_name, "--out", str(out), "--max-tokens", str(need)],
                          input=lines, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    assert [line for line in done.stdout.splitlines() if line.startswith("done ")] == [f"done {s['step']}" for s in steps]
    got = rh.read_trace_output(steps, out, KELASUN_CONFIGS[name].vocab)
    compare(got, folders[name], requests, getattr(torch, dtype_name))


@pytest.mark.parametrize("eager", [True, False], ids=["eager", "graphs"])
@pytest.mark.parametrize("name", sorted(KELASUN_CONFIGS))
def test_greedy_generation_through_the_engine(name, eager, folders):
    """LLM.generate (scheduler, chunked prefill, decode graphs and runs of decode steps) against
    greedy decoding with the plain implementation, float32."""
    from tinyvllm_b200 import LLM, EngineConfig, SamplingParams

    config = KELASUN_CONFIGS[name]
    prompts = [tokens_of(config.vocab, n, 700 + n) for n in (1, 9, 40, 77, 130)]
    engine_config = EngineConfig(
        model=folders[name], dtype="float32", max_model_len=512, max_num_seqs=4, max_num_batched_tokens=64,
        prefill_chunk_size=24, kv_block_size=KELASUN_PAGES[name], kv_cache_memory_bytes=16 * 1024 * 1024,
        prefill_reserve_tokens=0, prefill_reserve_requests=0, enforce_eager=eager)
    with LLM(engine_config) as llm:
        outputs = llm.generate(prompts, SamplingParams(max_new_tokens=40, ignore_eos=True))
        if not eager:
            assert llm.engine.graph_steps > 0
    for prompt, output in zip(prompts, outputs):
        assert list(output.output_token_ids) == greedy_oracle(folders[name], prompt, 40)


def test_bfloat16_generation_through_the_engine(folders):
    from tinyvllm_b200 import LLM, EngineConfig, SamplingParams

    name = "a"
    config = KELASUN_CONFIGS[name]
    prompts = [tokens_of(config.vocab, n, 800 + n) for n in (70, 3)]
    engine_config = EngineConfig(
        model=folders[name], dtype="bfloat16", max_model_len=256, max_num_seqs=4, max_num_batched_tokens=64,
        prefill_chunk_size=32, kv_block_size=16, kv_cache_memory_bytes=8 * 1024 * 1024,
        prefill_reserve_tokens=0, prefill_reserve_requests=0)
    with LLM(engine_config) as llm:
        outputs = llm.generate(prompts, SamplingParams(max_new_tokens=12, ignore_eos=True))
    assert all(len(output.output_token_ids) == 12 for output in outputs)
    for prompt, output in zip(prompts, outputs):
        logits = oracle_logits(folders[name], {"g": prompt})["g"][-1]
        top = logits.topk(2).values
        if (top[0] - top[1]).item() > 0.05 * logits.abs().max().item():
            assert output.output_token_ids[0] == int(logits.argmax())


def test_bfloat16_steps_run_on_the_tensor_core_kernels(folders, monkeypatch):
    """Sizes in steps of 16: prompt portions of both mixers go to the tile kernel, decoded tokens to the
    kernel for single tokens, none to the row kernel; the latent layers hand over no value cache."""
    from tinyvllm_b200.ops import kernels

    seen = {"attention_tiles": [], "attention_tiles_singles": [], "attention_rows": []}
    for fn in seen:
        original = getattr(kernels, fn)

        def watched(*args, _original=original, _fn=fn, **kwargs):
            seen[_fn].append(args[2] is None)          # the value cache
            return _original(*args, **kwargs)
        monkeypatch.setattr(kernels, fn, watched)
    name = "c"
    requests = {"t": tokens_of(KELASUN_CONFIGS[name].vocab, 90, 31)}
    runner = make_runner(folders[name], torch.bfloat16, 16, 16)
    with torch.inference_mode():
        rh.run_steps(runner, rh.tail_by_one(requests, 3))
    layers = [layer.type for layer in KELASUN_CONFIGS[name].layers]
    latent = [kind == "latent_attention" for kind in layers]
    assert seen["attention_tiles"] == latent                      # one prompt step
    assert seen["attention_tiles_singles"] == latent * 3          # three decoded tokens
    assert not seen["attention_rows"]


def test_command_line(folders, capsys):
    """python -m tinyvllm_b200 on a Kelasun folder: greedy tokens of the plain implementation, also
    streamed, and with weights drawn from a seed instead of the file."""
    from tinyvllm_b200.__main__ import main

    name = "b"
    prompts = [tokens_of(KELASUN_CONFIGS[name].vocab, n, 950 + n) for n in (3, 45)]
    want = [greedy_oracle(folders[name], prompt, 10) for prompt in prompts]
    common = ["--model", str(folders[name]), "--max-new-tokens", "10", "--ignore-eos", "--kv-cache-mib", "16",
              "--max-model-len", "256", "--kv-block-size", "8"]
    ids = [arg for prompt in prompts for arg in ("--prompt-ids", ",".join(map(str, prompt)))]
    main(common + ["--dtype", "float32", "--stream"] + ids)
    lines = [json.loads(line) for line in capsys.readouterr().out.strip().splitlines()]
    streamed = {0: [], 1: []}
    for line in lines[:-1]:
        streamed[line["prompt"]].append(line["token_id"])
    assert [streamed[0], streamed[1]] == want
    assert [record["output_token_ids"] for record in lines[-1]["outputs"]] == want
    main(common + ["--dtype", "bfloat16", "--random-weights", "7"] + ids)
    records = json.loads(capsys.readouterr().out.strip().splitlines()[-1])["outputs"]
    assert [len(record["output_token_ids"]) for record in records] == [10, 10]
