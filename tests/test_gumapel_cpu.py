"""Gumapel without a GPU: configuration, description as parts, weights, cache bookkeeping, and the
plain implementation's own consistency."""

import json

import pytest
import torch

import plain_gumapel as plain
from gumapel_configs import GUMAPEL_CONFIGS, GUMAPEL_SEEDS, read_folder, tensors_of, tokens_of, write_folder
from tinyvllm_b200 import ConfigError, read_model_config
from tinyvllm_b200.cache.manager import CacheGroup, CacheManager
from tinyvllm_b200.cache.storage import bytes_per_page, group_runs
from tinyvllm_b200.config.registry import parse_model_config
from tinyvllm_b200.engine.model import Model
from tinyvllm_b200.models import GumapelConfig
from tinyvllm_b200.parts.base import KVNeed, ParamSpec
from tinyvllm_b200.weights.loader import WeightsError, bind_tensors


# --------------------------------------------------------------- configuration
@pytest.mark.parametrize("name", sorted(GUMAPEL_CONFIGS))
def test_config_round_trip(name, tmp_path):
    config = GUMAPEL_CONFIGS[name]
    folder = write_folder(tmp_path / name, config, GUMAPEL_SEEDS[name])
    again = read_model_config(folder)
    assert isinstance(again, GumapelConfig) and again == config
    assert json.loads((folder / "config.json").read_text())["architecture"] == "Gumapel"


def test_config_refusals():
    good = GUMAPEL_CONFIGS["p"].to_json()
    assert parse_model_config(good) == GUMAPEL_CONFIGS["p"]

    def broken(change):
        data = json.loads(json.dumps(good))
        change(data)
        with pytest.raises(ConfigError):
            parse_model_config(data)

    broken(lambda d: d.pop("vocab"))
    broken(lambda d: d["layers"][0].__setitem__("type", "attention_3"))
    broken(lambda d: d["layers"][0]["mixer"].pop("scale"))
    broken(lambda d: d["layers"][0]["mixer"].__setitem__("heads", 3))            # 3 heads over 2 kv heads
    broken(lambda d: d["layers"][0]["mixer"]["rot"].__setitem__("dims", 34))     # more than the head has
    broken(lambda d: d["layers"][0]["mlp"].__setitem__("kind", "routed"))
    broken(lambda d: d["layers"][1]["mixer"].__setitem__("vdim", 32))            # blends with values of another size
    broken(lambda d: d.__setitem__("architecture", "Nothing"))


def test_spec_names_the_mechanisms():
    spec = GUMAPEL_CONFIGS["q"].to_spec()
    kinds = [(layer.block.kind, layer.mixer.kind, layer.norm.kind) for layer in spec.layers]
    assert set(kinds) == {("parallel_residual", "windowed_attention", "rms_norm_stream32")}
    first, second, third, fourth = (layer.mixer.params for layer in spec.layers)
    assert first["qk_norm"] == "unit" and first["gate"] and "position" not in first and "value_mix" not in first
    assert second["value_mix"] == "first" and third["value_mix"] == "blend" and fourth["value_mix"] == "blend"
    assert second["position"].kind == "rope_interleaved" and second["position"].params["dims"] == 12
    assert second["keep_first"] == 5 and second["window"] == 33 and third["window"] is None
    assert spec.layers[2].feed_forward is None and spec.layers[0].feed_forward.params["activation"] == "gelu_tanh"


def test_tensor_names_and_shapes():
    config = GUMAPEL_CONFIGS["p"]
    model = Model(config.to_spec(), device=torch.device("meta"), dtype=torch.float32)
    from tinyvllm_b200.weights.loader import source_shape

    declared = {source.name: source_shape(spec, source) for _, spec in model.param_targets() for source in spec.sources}
    drawn = {name: tuple(t.shape) for name, t in tensors_of(config, 0).items()}
    assert declared == drawn
    assert declared["l1.mix.vmix"] == () and "l3.mix.vmix" not in declared and "l2.mlp.gate" not in declared


def test_weights_packed_by_rows_by_columns_and_scalars():
    class Holder:
        def bind(self, attr, tensor):
            setattr(self, attr, tensor)

    holder = Holder()
    specs = [ParamSpec.packed("rows", [("a", 2), ("b", 3)], 4),
             ParamSpec.side_by_side("cols", 3, [("c", 2), ("d", 5)]),
             ParamSpec.scalar("one", "s")]
    tensors = {"a": torch.ones(2, 4), "b": 2 * torch.ones(3, 4), "c": 3 * torch.ones(3, 2),
               "d": 4 * torch.ones(3, 5), "s": torch.tensor(0.25)}
    bind_tensors([(holder, spec) for spec in specs], tensors, dtype=torch.float32, device="cpu")
    assert holder.rows.shape == (5, 4) and holder.rows[:2].eq(1).all() and holder.rows[2:].eq(2).all()
    assert holder.cols.shape == (3, 7) and holder.cols[:, :2].eq(3).all() and holder.cols[:, 2:].eq(4).all()
    assert holder.one.shape == (1,) and holder.one.item() == 0.25
    tensors["d"] = torch.ones(3, 4)
    with pytest.raises(WeightsError) as failure:
        bind_tensors([(holder, spec) for spec in specs], tensors, dtype=torch.float32, device="cpu")
    assert failure.value.wrong_shape[0][:2] == ("d", (3, 5))


# ------------------------------------------------------------------------ cache
def test_groups_by_geometry():
    needs = [KVNeed(2, 48, 40, 64, 4), KVNeed(2, 48, 40, 64, 4), KVNeed(2, 64, 96, 64, 0), KVNeed(2, 48, 40, 64, 3),
             KVNeed(2, 48, None, 64, 9), KVNeed(2, 48, None, 64, 0)]
    groups, where = group_runs(needs, [None] * len(needs))
    assert [g.runs for g in groups] == [(0, 1), (2,), (3,), (4, 5)]        # kept tokens mean nothing without a window
    assert groups[0].value_size == 64 and groups[0].keep_first == 4 and where[1] == (0, 1)
    assert bytes_per_page(groups[0], 16, 2) == 2 * 16 * 2 * (48 + 64) * 2


def test_window_gives_pages_back_but_not_the_kept_first():
    page, window, keep = 4, 10, 6
    manager = CacheManager([CacheGroup((0,), 1, 8, window, None, keep), CacheGroup((1,), 1, 8, window)], page, [64, 64], 2)
    manager.open("r")
    length = 0
    for count in (5, 1, 30, 1, 1, 1, 2, 40):
        plan = manager.plan([("r", count)])
        manager.commit(plan)
        length += count
        first_in_window = max(0, length - window + 1)          # of the next query
        kept, plain_window = manager.block_table("r", 0), manager.block_table("r", 1)
        for index in range(len(kept)):
            last_of_page = index * page + page - 1
            needed = last_of_page >= first_in_window
            assert (plain_window[index] >= 0) == needed
            assert (kept[index] >= 0) == (needed or index * page < keep)
        manager.check()
    assert manager.kept_pages(0) == 2 and manager.kept_pages(1) == 0
    assert manager.peak_pages(0, 10_000, 16) == manager.peak_pages(1, 10_000, 16) + 2
    manager.close("r")
    assert manager.free_pages(0) == 64 and manager.free_pages(1) == 64


# ------------------------------------------------------- the plain implementation
def test_plain_mask():
    assert plain.visible(10, 10, 1, 0) and not plain.visible(10, 9, 1, 0) and not plain.visible(9, 10, None, 0)
    assert plain.visible(50, 11, 40, 0) and not plain.visible(50, 10, 40, 0)
    assert plain.visible(50, 3, 40, 4) and not plain.visible(50, 4, 40, 4)
    assert plain.visible(50, 0, None, 0)


def test_plain_rotation_is_a_rotation_of_pairs():
    x = torch.randn(5, 2, 12, dtype=torch.float64)
    positions = torch.tensor([0, 1, 7, 100, 1000])
    y = plain.rotate_interleaved(x, positions, 8, 10000.0)
    assert torch.equal(y[0], x[0]) and torch.equal(y[..., 8:], x[..., 8:])
    pairs_before = (x[..., 0:8:2] ** 2 + x[..., 1:8:2] ** 2)
    pairs_after = (y[..., 0:8:2] ** 2 + y[..., 1:8:2] ** 2)
    assert torch.allclose(pairs_before, pairs_after)
    # the dot product of a rotated q and k depends on the distance only
    q, k = torch.randn(1, 1, 8, dtype=torch.float64), torch.randn(1, 1, 8, dtype=torch.float64)
    def dot(i, j):
        return (plain.rotate_interleaved(q, torch.tensor([i]), 8, 100.0) *
                plain.rotate_interleaved(k, torch.tensor([j]), 8, 100.0)).sum()
    assert torch.allclose(dot(13, 4), dot(109, 100))


@pytest.mark.parametrize("name", sorted(GUMAPEL_CONFIGS))
def test_plain_logits_do_not_depend_on_later_tokens(name, tmp_path):
    config = GUMAPEL_CONFIGS[name]
    folder = write_folder(tmp_path / name, config, GUMAPEL_SEEDS[name])
    parsed, tensors = read_folder(folder)
    tokens = tokens_of(config.vocab, 90, 1)
    whole = plain.forward(parsed, tensors, tokens)
    part = plain.forward(parsed, tensors, tokens[:61])
    assert torch.allclose(whole[:61], part, atol=1e-9)
    # a token far behind every window and not among the kept first ones is not seen at all
    if all(layer.window is not None for layer in config.layers):
        far = max(layer.keep_first for layer in config.layers) + 1
        reach = sum(layer.window - 1 for layer in config.layers)
        if far + reach < 89:
            changed = list(tokens)
            changed[far] = (changed[far] + 1) % config.vocab
            assert torch.allclose(plain.forward(parsed, tensors, changed)[-1], whole[-1], atol=1e-9)
