"""Gumapel on the GPU against the plain implementation: each mechanism alone, then whole models
through the step function, the trace program and the generation entry point."""

import json
import math
import subprocess
import sys

import pytest
import torch

import plain_gumapel as plain
import replay_helpers as rh
from gumapel_configs import (GUMAPEL_CONFIGS, GUMAPEL_PAGES, GUMAPEL_SEEDS, greedy_oracle, oracle_logits,
                             tokens_of, write_folder)

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]
IDS = ["f32", "bf16"]
CUDA = "cuda:0"


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: write_folder(tmp_path_factory.mktemp(f"gumapel_{name}"), config, GUMAPEL_SEEDS[name])
            for name, config in GUMAPEL_CONFIGS.items()}


def close(got, want, dtype, scale=None):
    scale = scale if scale is not None else max(want.abs().max().item(), 1e-6)
    limit = 3e-6 if dtype == torch.float32 else 1.2e-2
    worst = (got.double().cpu() - want.double().cpu()).abs().max().item() / scale
    assert worst <= limit, f"largest difference {worst:.3g} of the scale, allowed {limit:.3g}"


# ------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("width", [40, 384, 1024])
def test_stream_norm(width, dtype):
    from tinyvllm_b200.ops import kernels

    g = torch.Generator().manual_seed(width)
    stream = torch.randn(7, width, generator=g) * 3
    a, b = (torch.randn(7, width, generator=g).to(dtype) for _ in range(2))
    weight = (1 + 0.3 * torch.randn(width, generator=g)).to(dtype)
    on = lambda t: t.to(CUDA)
    y, new = kernels.stream_norm(on(stream.clone()), on(weight), 1e-5, add=on(a), add2=on(b), out_dtype=dtype)
    total = stream.double() + (a.double() + b.double())
    close(new, total, torch.float32)
    close(y, plain.rms_norm(total, weight.double(), 1e-5), dtype)
    # activations start a stream; chosen rows; no addend
    y, new = kernels.stream_norm(None, on(weight), 1e-5, add=on(a), out_dtype=dtype)
    assert new.dtype == torch.float32 and torch.equal(new.cpu(), a.float())
    close(y, plain.rms_norm(a.double(), weight.double(), 1e-5), dtype)
    rows = torch.tensor([5, 0, 5], dtype=torch.int32)
    y, none = kernels.stream_norm(on(stream.clone()), on(weight), 1e-5, add=on(a), rows=on(rows), out_dtype=dtype)
    assert none is None
    close(y, plain.rms_norm((stream.double() + a.double())[rows.long()], weight.double(), 1e-5), dtype)
    y, _ = kernels.stream_norm(on(stream.clone()), on(weight), 1e-5, out_dtype=dtype)
    close(y, plain.rms_norm(stream.double(), weight.double(), 1e-5), dtype)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_gated_activation(dtype):
    from tinyvllm_b200.ops import kernels

    g = torch.Generator().manual_seed(3)
    packed = (torch.randn(9, 5 + 2 * 37, generator=g) * 3).to(dtype)
    out = torch.zeros(9, 50, dtype=dtype, device=CUDA)
    kernels.gated_act(packed.to(CUDA), 5, 5 + 37, 37, "gelu_tanh", out=out[:, 4:41])
    want = plain.gelu_tanh(packed[:, 5:42].double()) * packed[:, 42:79].double()
    close(out[:, 4:41], want, dtype)
    assert out[:, :4].abs().sum() == 0 and out[:, 41:].abs().sum() == 0
    silu = kernels.gated_act(packed.to(CUDA), 5, 42, 37, "silu")
    x = packed[:, 5:42].double()
    close(silu, x / (1 + torch.exp(-x)) * packed[:, 42:79].double(), dtype)


def _caches(pages, kv, page, dk, dv, dtype):
    return (torch.full((pages, kv, page, dk), float("nan"), dtype=dtype, device=CUDA),
            torch.full((pages, kv, page, dv), float("nan"), dtype=dtype, device=CUDA))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("dk,dv", [(20, 24), (21, 7), (32, 24), (128, 64)])
@pytest.mark.parametrize("norm,rot,pairing", [("unit", 0, "interleaved"), (None, 12, "interleaved"),
                                              (None, 20, "interleaved"), ("weight", 8, "half_split"),
                                              ("weight", 16, "interleaved")])
def test_prepare_norm_rotation_blend_and_store(norm, rot, pairing, dk, dv, dtype):
    """Heads of 20 keys and 24 values (the general kernel) and of 32 and 128 keys (in bfloat16: the
    kernel of 16-byte words) at positions up to 100,000, blended values, scattered slots."""
    from tinyvllm_b200.ops import kernels

    g = torch.Generator().manual_seed(rot + 1)
    tokens, heads, kv, page = 6, 4, 2, 4
    at = 8
    cols = at + heads * dk + kv * dk + kv * dv + 3
    proj = torch.randn(tokens, cols, generator=g).to(dtype)
    positions = torch.tensor([0, 1, 17, 4095, 99999, 31], dtype=torch.int32)
    slots = torch.tensor([5, 0, 11, 2, -1, 7], dtype=torch.int32)          # token 4 writes nothing
    base = 500000.0
    inv_freq = None
    if rot:
        inv_freq = (base ** -(torch.arange(0, rot, 2, dtype=torch.float64) / rot)).float()
    v_first = torch.randn(tokens, kv * dv + 5, generator=g).to(dtype)[:, 2:2 + kv * dv]
    blend = torch.tensor([0.3], dtype=dtype)
    qw, kw = ((1 + 0.2 * torch.randn(dk, generator=g)).to(dtype) for _ in range(2))
    keys, values = _caches(3, kv, page, dk, dv, dtype)
    device = proj.to(CUDA)
    kernels.qkv_prepare(
        device, q_at=at, k_at=at + heads * dk, v_at=at + (heads + kv) * dk, num_q=heads, num_kv=kv, key_dim=dk,
        value_dim=dv, positions=positions.to(CUDA), norm=norm, q_weight=qw.to(CUDA) if norm == "weight" else None,
        k_weight=kw.to(CUDA) if norm == "weight" else None, eps=1e-6,
        inv_freq=None if inv_freq is None else inv_freq.to(CUDA), rot_dims=rot, pairing=pairing,
        slots=slots.to(CUDA), key_cache=keys, value_cache=values, v_first=v_first.to(CUDA), blend=blend.to(CUDA))

    def prepared(x, weight):
        x = x.double()
        if norm is not None:
            x = plain.rms_unit(x, 1e-6)
        if norm == "weight":
            x = x * weight.double()
        if rot and pairing == "interleaved":
            # the angle is a float32 product of position and frequency, as the design computes it
            out = x.clone()
            for i in range(rot // 2):
                angle = (positions.float() * inv_freq[i]).double()
                c, s = torch.cos(angle)[:, None], torch.sin(angle)[:, None]
                out[:, :, 2 * i] = x[:, :, 2 * i] * c - x[:, :, 2 * i + 1] * s
                out[:, :, 2 * i + 1] = x[:, :, 2 * i + 1] * c + x[:, :, 2 * i] * s
            x = out
        elif rot:
            out = x.clone()
            for i in range(rot // 2):
                angle = (positions.float() * inv_freq[i]).double()
                c, s = torch.cos(angle)[:, None], torch.sin(angle)[:, None]
                out[:, :, i] = x[:, :, i] * c - x[:, :, i + rot // 2] * s
                out[:, :, i + rot // 2] = x[:, :, i + rot // 2] * c + x[:, :, i] * s
            x = out
        return x

    q = prepared(proj[:, at:at + heads * dk].view(tokens, heads, dk), qw)
    k = prepared(proj[:, at + heads * dk:at + (heads + kv) * dk].view(tokens, kv, dk), kw)
    v = plain.mix_values(proj[:, at + (heads + kv) * dk:at + (heads + kv) * dk + kv * dv].double(),
                         v_first.double(), blend.double()).view(tokens, kv, dv)
    got = device.cpu()
    close(got[:, at:at + heads * dk].view(tokens, heads, dk), q, dtype)
    assert torch.equal(got[:, :at], proj[:, :at]) and torch.equal(got[:, -3:], proj[:, -3:])
    written = 0
    for token, slot in enumerate(slots.tolist()):
        if slot < 0:
            continue
        close(keys[slot // page, :, slot % page].cpu(), k[token], dtype)
        close(values[slot // page, :, slot % page].cpu(), v[token], dtype)
        written += 1
    assert torch.isnan(keys.float()).sum().item() == (3 * page - written) * kv * dk      # nothing else was touched
    # the oracle's own rotation (angles in double precision) agrees where positions are small
    if rot and pairing == "interleaved" and norm is None:
        mine = plain.rotate_interleaved(proj[:3, at:at + heads * dk].view(3, heads, dk).double(), positions[:3],
                                        rot, base)
        close(got[:3, at:at + heads * dk].view(3, heads, dk), mine, dtype, scale=10.0 if dtype == torch.float32 else None)


def _attend(kind, q, keys, values, table, positions, token_row, tiles, sizes, gate, dtype, max_context):
    """Run one of the three attention kernels on prepared queries."""
    from tinyvllm_b200.ops import kernels

    heads, kv, dk, dv, window, keep, scale = sizes
    tokens = q.shape[0]
    out = torch.zeros(tokens, heads * dv + 6, dtype=dtype, device=CUDA)[:, 2:2 + heads * dv]
    common = dict(num_q=heads, num_kv=kv, window=window, keep_first=keep, scale=scale, out=out, gate=gate)
    if kind == "rows" or kind == "rows_split":
        chunks = 0 if kind == "rows" else -(-max_context // kernels.attention_chunk_keys())
        scratch = torch.empty(max(1, kernels.attention_rows_scratch_floats(tokens, heads, dv, chunks)),
                              dtype=torch.float32, device=CUDA)
        kernels.attention_rows(q, q.stride(0), keys, values, table, token_row, positions, head_dim=dk, value_dim=dv,
                               scratch=scratch, max_chunks=chunks, **common)
    elif kind == "tiles":
        kernels.attention_tiles(q, keys, values, table, positions, *tiles, key_dim=dk, value_dim=dv, **common)
    else:
        scratch = torch.empty(kernels.attention_tiles_singles_floats(tokens, heads, dv, window, keep, max_context),
                              dtype=torch.float32, device=CUDA)
        kernels.attention_tiles_singles(q, keys, values, table, positions, token_row, key_dim=dk, value_dim=dv,
                                        max_context=max_context, scratch=scratch, **common)
    return out


def _paged(k, v, page, dtype, seed):
    """Keys [T, G, dk] and values of one sequence laid into shuffled pages; unused slots are NaN (row
    kernel) so that a key read from outside the sequence shows."""
    length, kv, dk = k.shape
    dv = v.shape[2]
    count = -(-length // page)
    order = list(range(count + 3))
    __import__("random").Random(seed).shuffle(order)
    keys = torch.full((count + 3, kv, page, dk), float("nan"), dtype=dtype)
    values = torch.full((count + 3, kv, page, dv), float("nan"), dtype=dtype)
    where = torch.tensor([order[p // page] for p in range(length)])
    inside = torch.arange(length) % page
    keys[where, :, inside] = k.to(dtype)
    values[where, :, inside] = v.to(dtype)
    keys, values = keys.to(CUDA), values.to(CUDA)
    table = torch.tensor([order[:count] + [-1] * 3], dtype=torch.int32, device=CUDA)
    return keys, values, table


ATTENTION_KINDS = [("rows", torch.float32), ("rows_split", torch.float32), ("rows", torch.bfloat16),
                   ("tiles", torch.bfloat16), ("singles", torch.bfloat16)]


@pytest.mark.parametrize("kind,dtype", ATTENTION_KINDS, ids=[f"{k}-{'f32' if d == torch.float32 else 'bf16'}"
                                                             for k, d in ATTENTION_KINDS])
@pytest.mark.parametrize("window,keep", [(40, 4), (300, 0), (16, 20), (None, 0), (1, 2)])
def test_attention_sees_exactly_its_window_and_the_kept_first_keys(kind, dtype, window, keep):
    """One key at a time is made to stand out (its dot product with every query is far above the
    others') and given a value no other key has: the outputs tell which queries saw it.  The marked
    keys lie at both edges of windows, at the edge of the kept first keys, at borders of pages,
    tiles and chunks, and far back."""
    heads, kv, dk, dv, page, length = 4, 2, 32, 48, 16, 700
    g = torch.Generator().manual_seed(5)
    scale = 0.25
    queries = list(range(length - 70, length)) + [0, 1, 2, 3, 15, 16, 17, 31, 32, 33, 255, 256, 257, 299, 300, 301, 339]
    queries = sorted(set(queries))
    marked_keys = {0, 1, 3, 4, 15, 16, 19, 20, 31, 32, 255, 256, length - 1, length - 2}
    for i in (length - 1, length - 33, 339, 300):
        if window is not None:
            marked_keys |= {i - window + 1, i - window, i - window - 1} & set(range(length))
    direction = torch.nn.functional.normalize(torch.randn(dk, generator=g), dim=0)
    for marked in sorted(marked_keys):
        k = torch.randn(length, kv, dk, generator=g) * 0.3
        k -= (k @ direction)[..., None] * direction            # no other key points along the direction
        v = torch.randn(length, kv, dv, generator=g) * 0.1
        k[marked] += 40.0 * direction
        v[marked] = 5.0
        q = torch.randn(length, heads, dk, generator=g) * 0.3 + 4.0 * direction
        q, k, v = (t.to(torch.bfloat16).double() for t in (q, k, v))
        keys, values, table = _paged(k, v, page, dtype, marked)
        rows = torch.tensor(queries)
        if kind == "tiles":
            # consecutive tokens: the last 64 + 6 queries are one tile of 64 and one of 6
            rows = torch.arange(length - 70, length)
            tiles = [torch.tensor(x, dtype=torch.int32, device=CUDA) for x in ([0, 0], [0, 64], [64, 6])]
        else:
            tiles = None
        qd = torch.zeros(len(rows), heads * dk + 8, dtype=dtype)[:, :heads * dk]
        qd[:] = q[rows].reshape(len(rows), -1).to(dtype)
        got = _attend(kind, qd.to(CUDA), keys, values, table, rows.to(torch.int32).to(CUDA),
                      torch.zeros(len(rows), dtype=torch.int32, device=CUDA), tiles,
                      (heads, kv, dk, dv, window, keep, scale), None, dtype, 1024).cpu().view(len(rows), heads, dv)
        for n, i in enumerate(rows.tolist()):
            sees = plain.visible(i, marked, window, keep if window is not None else 0)
            value = got[n].double().mean().item()
            assert (value > 4.5) == sees, f"query {i} and key {marked}: mean output {value:.3f}, sees = {sees}"


@pytest.mark.parametrize("kind,dtype", ATTENTION_KINDS, ids=[f"{k}-{'f32' if d == torch.float32 else 'bf16'}"
                                                             for k, d in ATTENTION_KINDS])
@pytest.mark.parametrize("group,dk,dv", [(1, 16, 64), (3, 48, 32), (8, 64, 16), (20, 16, 32)])
def test_attention_values_with_a_gate(kind, dtype, group, dk, dv):
    """Random queries of several requests in one launch against the plain attention, gated."""
    kv, page, window, keep, scale = 2, 8, 45, 6, 0.2
    heads = kv * group
    g = torch.Generator().manual_seed(group)
    lengths = [130, 47, 300]
    from tinyvllm_b200.ops import kernels  # noqa: F401

    pieces, tables, qs, positions, token_row, want, gates = [], [], [], [], [], [], []
    offset_pages = 0
    all_keys, all_values = [], []
    for r, length in enumerate(lengths):
        q = (torch.randn(length, heads, dk, generator=g)).to(torch.bfloat16).double()
        k = (torch.randn(length, kv, dk, generator=g)).to(torch.bfloat16).double()
        v = (torch.randn(length, kv, dv, generator=g)).to(torch.bfloat16).double()
        keys, values, table = _paged(k, v, page, dtype, r)
        all_keys.append(torch.nan_to_num(keys, nan=1e4))
        all_values.append(torch.nan_to_num(values, nan=1e4))
        tables.append(torch.where(table >= 0, table + offset_pages, table))
        offset_pages += keys.shape[0]
        full = plain.masked_attention(q, k, v, scale, window, keep)
        take = list(range(length - 20, length)) if kind != "singles" and kind != "rows_split" else [length - 1, length - 9]
        for i in take:
            qs.append(q[i].reshape(-1)), positions.append(i), token_row.append(r), want.append(full[i].reshape(-1))
        pieces.append((r, len(take)))
    width = max(t.shape[1] for t in tables)
    table = torch.cat([torch.nn.functional.pad(t, (0, width - t.shape[1]), value=-1) for t in tables])
    keys, values = torch.cat(all_keys), torch.cat(all_values)
    tokens = len(qs)
    gate = torch.randn(tokens, heads * dv, generator=g).to(dtype)
    tiles, first = [[], [], []], 0
    for r, count in pieces:
        tiles[0].append(r), tiles[1].append(first), tiles[2].append(count)
        first += count
    tiles = [torch.tensor(x, dtype=torch.int32, device=CUDA) for x in tiles]
    got = _attend(kind, torch.stack(qs).to(dtype).to(CUDA), keys, values, table,
                  torch.tensor(positions, dtype=torch.int32, device=CUDA),
                  torch.tensor(token_row, dtype=torch.int32, device=CUDA), tiles,
                  (heads, kv, dk, dv, window, keep, scale), gate.to(CUDA), dtype, 512)
    close(got, torch.stack(want) * torch.sigmoid(gate.double()), dtype)


# ---------------------------------------------------------------- whole models
def requests_of(name):
    vocab = GUMAPEL_CONFIGS[name].vocab
    return {f"{name}{n}": tokens_of(vocab, n, 500 + n) for n in (1, 2, 37, 150, 420)}


def make_runner(folder, dtype, page, pages, max_len=None):
    from tinyvllm_b200 import read_model_config
    from tinyvllm_b200.engine.model import Model
    from tinyvllm_b200.engine.step import StepRunner

    model = Model(read_model_config(folder).to_spec(), device=CUDA, dtype=dtype).load(folder)
    return StepRunner(model, page_size=page, num_pages=pages, max_requests=4, max_model_len=max_len or pages * page)


def compare(got: dict, folder, requests, dtype):
    expected = oracle_logits(folder, requests)
    assert got, "no logits came back"
    worst = 0.0
    for (rid, position), row in got.items():
        want = expected[rid]
        worst = max(worst, (row.double() - want[position].double()).abs().max().item() / want.abs().max().item())
    limit = 2e-5 if dtype == torch.float32 else rh.TOLERANCE[torch.bfloat16]
    assert worst <= limit, f"largest difference {worst:.3g} of the largest logit, allowed {limit:.3g}"


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", sorted(GUMAPEL_CONFIGS))
@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed"])
def test_every_way_of_cutting_gives_the_plain_logits(cut, name, dtype, folders):
    """Whole prompts; prompts whose last 40 tokens come one by one (windows pass over decoded tokens);
    portions of changing size down to two tokens; up to four live requests with portions beside single
    tokens, in a pool with room for little more than the live tokens, so that pages that were given
    back, by windows and by finished requests, are taken again."""
    requests = requests_of(name)
    page = GUMAPEL_PAGES[name]
    steps = {"whole": lambda: rh.whole(requests), "tail": lambda: rh.tail_by_one(requests, 40),
             "portions": lambda: rh.portions(requests, 3, sizes=(2, 3, 5, 8, 13, 31, 64, 100, 200)),
             "mixed": lambda: rh.mixed(requests, 4, live=4, decode_tail=20, sizes=(2, 3, 7, 16, 40, 90))}[cut]()
    pages = -(-rh.live_token_need(steps, page) // page) if cut == "mixed" else 64
    runner = make_runner(folders[name], dtype, page, pages)
    with torch.inference_mode():
        got = rh.run_steps(runner, steps)
    compare(got, folders[name], requests, dtype)
    assert not runner.manager.open_requests()
    assert all(runner.manager.free_pages(g) == pages for g in range(len(runner.manager.groups)))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_a_request_is_not_moved_by_its_neighbours(dtype, folders):
    """The same request alone and beside three others, in other pages: equal beyond rounding."""
    name = "p"
    requests = requests_of(name)
    page = GUMAPEL_PAGES[name]
    alone = {"x": requests["p150"]}
    with torch.inference_mode():
        first = rh.run_steps(make_runner(folders[name], dtype, page, 64), rh.portions(alone, 9, sizes=(7, 50)))
        crowd = dict(list(requests.items())[2:])
        crowd["x"] = requests["p150"]
        second = rh.run_steps(make_runner(folders[name], dtype, page, 96), rh.mixed(crowd, 1, live=4, decode_tail=5))
    scale = oracle_logits(folders[name], alone)["x"].abs().max().item()
    worst = max((first[key].double() - second[key].double()).abs().max().item() for key in first) / scale
    assert worst <= (1e-5 if dtype == torch.float32 else 2e-2)


def test_long_decoding_far_past_every_window(folders):
    """A prompt of five tokens and 400 tokens decoded one by one, float32: the windows and the kept
    first tokens are long behind, pages have been given back and taken again many times."""
    name = "p"
    tokens = tokens_of(GUMAPEL_CONFIGS[name].vocab, 405, 9)
    requests = {"long": tokens}
    steps = rh.tail_by_one(requests, 400)
    runner = make_runner(folders[name], torch.float32, 16, 24, max_len=512)   # room for 384 of 405 tokens: windows free pages
    with torch.inference_mode():
        got = rh.run_steps(runner, steps)
    compare(got, folders[name], requests, torch.float32)


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
def test_trace_program(dtype_name, folders, tmp_path):
    name = "p"
    requests = requests_of(name)
    steps = rh.mixed(requests, 2, live=3)
    need = rh.live_token_need(steps)
    lines = "\n".join(json.dumps(step) for step in steps) + "\n"
    out = tmp_path / "out"
    done = subprocess.run([sys.executable, str(rh_root() / "bin" / "trace_run"), "--model", str(folders[name]),
                           "--dtype", dtype_name, "--out", str(out), "--max-tokens", str(need)],
                          input=lines, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    assert [line for line in done.stdout.splitlines() if line.startswith("done ")] == [f"done {s['step']}" for s in steps]
    got = rh.read_trace_output(steps, out, GUMAPEL_CONFIGS[name].vocab)
    compare(got, folders[name], requests, getattr(torch, dtype_name))


def rh_root():
    from pathlib import Path
    return Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("eager", [True, False], ids=["eager", "graphs"])
@pytest.mark.parametrize("name", sorted(GUMAPEL_CONFIGS))
def test_greedy_generation_through_the_engine(name, eager, folders):
    """LLM.generate (scheduler, chunked prefill, decode graphs and runs of decode steps) against
    greedy decoding with the plain implementation, float32."""
    from tinyvllm_b200 import LLM, EngineConfig, SamplingParams

    config = GUMAPEL_CONFIGS[name]
    prompts = [tokens_of(config.vocab, n, 700 + n) for n in (1, 9, 40, 77, 130)]
    engine_config = EngineConfig(
        model=folders[name], dtype="float32", max_model_len=512, max_num_seqs=4, max_num_batched_tokens=64,
        prefill_chunk_size=24, kv_block_size=GUMAPEL_PAGES[name], kv_cache_memory_bytes=16 * 1024 * 1024,
        prefill_reserve_tokens=0, prefill_reserve_requests=0, enforce_eager=eager)
    with LLM(engine_config) as llm:
        outputs = llm.generate(prompts, SamplingParams(max_new_tokens=48, ignore_eos=True))
        if not eager:
            assert llm.engine.graph_steps > 0
    for prompt, output in zip(prompts, outputs):
        assert list(output.output_token_ids) == greedy_oracle(folders[name], prompt, 48)


def test_bfloat16_generation_runs_on_the_tensor_core_kernels(folders, monkeypatch):
    from tinyvllm_b200 import LLM, EngineConfig, SamplingParams
    from tinyvllm_b200.ops import kernels

    seen = {"tiles": 0, "singles": 0}
    for key, fn in (("tiles", "attention_tiles"), ("singles", "attention_tiles_singles")):
        original = getattr(kernels, fn)

        def watched(*args, _original=original, _key=key, **kwargs):
            seen[_key] += 1
            return _original(*args, **kwargs)
        monkeypatch.setattr(kernels, fn, watched)
    name = "p"
    config = GUMAPEL_CONFIGS[name]
    prompts = [tokens_of(config.vocab, n, 800 + n) for n in (70, 3)]
    engine_config = EngineConfig(
        model=folders[name], dtype="bfloat16", max_model_len=256, max_num_seqs=4, max_num_batched_tokens=64,
        prefill_chunk_size=32, kv_block_size=16, kv_cache_memory_bytes=8 * 1024 * 1024,
        prefill_reserve_tokens=0, prefill_reserve_requests=0, enforce_eager=True)
    with LLM(engine_config) as llm:
        outputs = llm.generate(prompts, SamplingParams(max_new_tokens=12, ignore_eos=True))
    assert all(len(output.output_token_ids) == 12 for output in outputs)
    assert seen["tiles"] > 0 and seen["singles"] > 0
    # the first new token is the plain implementation's where its lead over the runner-up is clear
    for prompt, output in zip(prompts, outputs):
        logits = oracle_logits(folders[name], {"g": prompt})["g"][-1]
        top = logits.topk(2).values
        if (top[0] - top[1]).item() > 0.05 * logits.abs().max().item():
            assert output.output_token_ids[0] == int(logits.argmax())
    assert math.isfinite(sum(sum(o.output_token_ids) for o in outputs))


def test_command_line(folders, capsys):
    """python -m tinyvllm_b200 on a Gumapel folder: greedy tokens of the plain implementation, also
    streamed, and with weights drawn from a seed instead of the file."""
    from tinyvllm_b200.__main__ import main

    name = "r"
    prompts = [tokens_of(GUMAPEL_CONFIGS[name].vocab, n, 950 + n) for n in (3, 45)]
    want = [greedy_oracle(folders[name], prompt, 10) for prompt in prompts]
    common = ["--model", str(folders[name]), "--max-new-tokens", "10", "--ignore-eos", "--kv-cache-mib", "16",
              "--max-model-len", "256", "--kv-block-size", "16"]
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
