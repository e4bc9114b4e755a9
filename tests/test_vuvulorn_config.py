"""Host-side parts of the Vuvulorn design: its configuration class, the names of its tensors, cache needs of several
parts, and which pages a window with kept first tokens gives back."""

from __future__ import annotations

import copy
import json

import pytest
import torch

from lalamo_b200.cache.manager import CacheManager, flatten_needs
from lalamo_b200.config import (
    AttentionSpec, ConfigError, GatedDeltaSpec, GatedMLPSpec, OutputNormBlockSpec, ParallelMixerSpec, RoutedMLPSpec, VuvulornConfig, config_from_dict, load_config,
)
from lalamo_b200.parts.base import CompositeNeed, PagedKVNeed, SlotStateNeed
from lalamo_b200.parts.model import plan_tensor_decls
from lalamo_b200.weights.loader import WeightsError, load_weights
from tiny_vuvulorn import CONFIG_P, CONFIG_Q, tensor_shapes, write_model


def test_every_size_and_constant_comes_from_the_configuration():
    config = config_from_dict(CONFIG_P)
    assert isinstance(config, VuvulornConfig)
    plan = config.to_plan()
    assert plan.vocab_size == 160 and plan.model_dim == 64 and not plan.tie_embeddings and plan.final_norm.eps == 1e-5
    first, second, third = plan.layers
    assert all(isinstance(layer, OutputNormBlockSpec) and isinstance(layer.mixer, ParallelMixerSpec) for layer in plan.layers)
    (left_name, left, left_scale), (right_name, right, right_scale) = first.mixer.branches
    assert (left_name, right_name, left_scale, right_scale) == ("left", "right", 0.7, 1.1)
    assert isinstance(left, AttentionSpec) and (left.num_heads, left.num_groups, left.head_dim, left.value_dim) == (4, 2, 16, 32)
    assert (left.window, left.keep_first, left.scale, left.has_bias) == (8, 3, 0.25, True)
    assert left.position.rotary_dim == 8 and left.position.theta == 10000.0 and left.qk_norm.dim == 16 and left.qk_norm.eps == 1e-5
    assert isinstance(right, GatedDeltaSpec) and (right.num_heads, right.num_groups, right.key_dim, right.value_dim, right.conv_taps) == (2, 1, 16, 32, 3)
    assert (right.decay_rank, right.gate_rank, right.norm_eps) == (6, 5, 1e-5)
    assert isinstance(first.ffn, RoutedMLPSpec) and (first.ffn.num_experts, first.ffn.top, first.ffn.group_count, first.ffn.group_keep, first.ffn.hidden_dim) == (6, 2, 3, 2, 32)
    assert first.ffn.score == "sigmoid" and not first.ffn.renormalize
    assert second.ffn is None and second.ffn_norm is None
    assert isinstance(third.ffn, GatedMLPSpec) and third.ffn.hidden_dim == 96
    no_rotation = config_from_dict(CONFIG_Q).to_plan().layers[0].mixer.branches[0][1]
    assert no_rotation.position is None and no_rotation.keep_first == 0 and no_rotation.window == 1


@pytest.mark.parametrize("path,value,key", [
    (("layers", 0, "type"), "serial", "layers[0].type"),
    (("layers", 1, "mixer", "left", "kv_heads"), 3, "layers[1].mixer.left.kv_heads"),
    (("layers", 0, "mixer", "left", "rot", "dims"), 18, "layers[0].mixer.left.rot.dims"),
    (("layers", 0, "mlp", "router", "groups", "count"), 4, "layers[0].mlp.router.groups.count"),
    (("layers", 0, "mlp", "router", "top"), 5, "layers[0].mlp.router.top"),
    (("layers", 2, "mlp", "kind"), "sparse", "layers[2].mlp.kind"),
    (("layers", 2, "mixer", "right", "conv"), 0, "layers[2].mixer.right.conv"),
    (("width",), None, "config.width"),
])
def test_errors_name_the_key(path, value, key):
    raw = copy.deepcopy(CONFIG_P)
    node = raw
    for step in path[:-1]:
        node = node[step]
    node[path[-1]] = value
    with pytest.raises(ConfigError) as error:
        config_from_dict(raw)
    assert error.value.key == key


def test_tensor_names_and_ranks_from_the_checkpoint(tmp_path):
    folder, _ = write_model(tmp_path / "p", CONFIG_P, 3)   # its config.json does not say the bottleneck ranks
    assert "decay_rank" not in json.loads((folder / "config.json").read_text())["layers"][0]["mixer"]["right"]
    config = load_config(folder)
    right = config.to_plan().layers[0].mixer.branches[1][1]
    assert (right.decay_rank, right.gate_rank) == (6, 5)
    tensors = load_weights(folder, config)
    named = {config.checkpoint_names(*key)[0]: tuple(tensor.shape) for key, tensor in tensors.items()}
    assert named == tensor_shapes(CONFIG_P)
    assert set(plan_tensor_decls(config.to_plan())) == set(tensors)
    # a tensor too many and one of the wrong shape are both reported
    from lalamo_b200.weights.safetensors_io import open_checkpoint, write_safetensors

    checkpoint = open_checkpoint(folder)
    changed = {name: checkpoint.read(name).clone() for name in checkpoint}
    changed["l1.mlp.gate"] = torch.zeros(4, 4)
    changed["l0.mix.left.o.b"] = torch.zeros(65)
    other = tmp_path / "changed"   # the first folder's file is still mapped into memory
    other.mkdir()
    (other / "config.json").write_text((folder / "config.json").read_text())
    write_safetensors(other / "model.safetensors", changed)
    with pytest.raises(WeightsError) as error:
        load_weights(other, load_config(other))
    assert error.value.unexpected == ["l1.mlp.gate"] and [name for name, _, _ in error.value.wrong_shape] == ["l0.mix.left.o.b"]


def test_random_weights_round_trip(tmp_path):
    from lalamo_b200.weights import write_random_model

    folder = write_random_model(tmp_path / "random", CONFIG_Q, seed=5)
    config = load_config(folder)
    tensors = load_weights(folder, config)
    assert {config.checkpoint_names(*key)[0] for key in tensors} == set(tensor_shapes(CONFIG_Q))
    again = config_from_dict(config.to_json_dict())
    assert again.to_plan() == config.to_plan()


def test_needs_of_several_parts_become_cells():
    window = PagedKVNeed(2, 16, window=8, value_dim=32, keep_first=3)
    other_window = PagedKVNeed(2, 16, window=8, keep_first=0)
    matrix, conv = SlotStateNeed((2, 16, 32), torch.float32), SlotStateNeed((2, 96))
    needs = [CompositeNeed((window, CompositeNeed((matrix, conv)))), None, CompositeNeed((other_window, CompositeNeed((matrix, conv)))), window]
    cells, cache_from, shapes = flatten_needs(needs, [None, None, None, None])
    assert cells == [window, matrix, conv, None, other_window, matrix, conv, window]
    assert shapes == [[0, [1, 2]], 3, [4, [5, 6]], 7] and cache_from == [None] * 8
    manager = CacheManager(needs, [None, None, None, None], None, page_size=16, num_pages=8, num_slots=2)
    # the same window with other kept tokens is another group: its pages live differently
    assert manager.layout.group_windows == [8, 8] and manager.layout.group_keep_first == [3, 0]
    assert manager.layout.group_entries == [[0, 7], [4]] and manager.layout.slot_entries == [1, 2, 5, 6]
    with pytest.raises(ValueError):
        flatten_needs([CompositeNeed((window, matrix)), window], [None, 0])


@pytest.mark.parametrize("keep_first,kept_blocks", [(0, 0), (1, 1), (16, 1), (17, 2), (40, 3)])
def test_a_window_frees_pages_but_not_those_of_the_kept_tokens(keep_first, kept_blocks):
    need = PagedKVNeed(1, 16, window=20, keep_first=keep_first)
    manager = CacheManager([need], [None], None, page_size=16, num_pages=12, num_slots=2)
    manager.admit("a")
    length = 0
    for count in (5, 30, 1, 1, 64, 3, 1, 50):
        manager.reserve("a", length + count)
        length += count
        manager.commit("a", length)
        manager.check()
        blocks = manager.requests["a"].blocks[0]
        first_needed = (length - 20 + 1) // 16 if length >= 20 else 0   # the block of the oldest key a later query sees
        for index, page in enumerate(blocks):
            assert (page >= 0) == (index < kept_blocks or index >= first_needed), (length, index)
    manager.release("a")
    assert manager.free_pages() == 12
