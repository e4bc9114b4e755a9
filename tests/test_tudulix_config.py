"""Host-side parts of the Tudulix design: its configuration class, the order in which layers run, the names of its
tensors, the cache a latent layer asks for, and the plain implementation's own rotation and routing on hand-made cases."""

from __future__ import annotations

import copy

import numpy as np
import pytest
import torch

import plain_tudulix as plain
from lalamo_b200.cache.manager import CacheManager
from lalamo_b200.config import (
    AttentionSpec, ConfigError, GatedMLPSpec, LatentAttentionSpec, RoutedMLPSpec, SandwichBlockSpec, TudulixConfig, config_from_dict, load_config,
)
from lalamo_b200.parts.base import PagedKVNeed
from lalamo_b200.parts.model import plan_tensor_decls
from lalamo_b200.weights.loader import WeightsError, load_weights
from tiny_tudulix import CONFIG_A, CONFIG_B, CONFIG_E, CONFIGS, tensor_shapes, write_model


def test_every_size_and_constant_comes_from_the_configuration():
    config = config_from_dict(CONFIG_A)
    assert isinstance(config, TudulixConfig)
    plan = config.to_plan()
    assert plan.vocab_size == 160 and plan.model_dim == 64 and plan.embedding.scale == 4.0 and plan.head.scale == 0.25 and not plan.head.tied
    assert plan.final_norm.eps == 1e-5 and plan.final_norm.scale_offset == 1.0 and plan.final_norm.exact
    assert all(isinstance(layer, SandwichBlockSpec) for layer in plan.layers)
    first, second, third, fourth = plan.layers
    assert isinstance(first.mixer, LatentAttentionSpec)
    assert (first.mixer.num_heads, first.mixer.head_dim, first.mixer.rope_dim, first.mixer.value_dim, first.mixer.latent_dim) == (4, 16, 8, 24, 32)
    assert (first.mixer.window, first.mixer.scale, first.mixer.gated) == (11, 0.2, True)
    assert first.mixer.position.pairing == "half" and first.mixer.position.theta == 500.0 and first.mixer.position.rotary_dim == 8
    assert first.mixer.latent_norm.dim == 32 and first.mixer.latent_norm.scale_offset == 0.0 and first.mixer.latent_norm.eps == 1e-5
    assert isinstance(second.mixer, AttentionSpec)
    assert (second.mixer.num_heads, second.mixer.num_groups, second.mixer.head_dim, second.mixer.value_dim, second.mixer.window) == (4, 2, 16, 32, 8)
    assert second.mixer.position.pairing == "interleaved" and second.mixer.position.rotary_dim == 8 and not second.mixer.has_bias and second.mixer.qk_norm is None
    assert third.ffn is None and third.ffn_norm is None and third.ffn_out_norm is None and third.mixer.position.theta == 77.0
    ffn = second.ffn
    assert isinstance(ffn, RoutedMLPSpec) and (ffn.num_experts, ffn.top, ffn.hidden_dim, ffn.limit) == (5, 3, 24, 2.5)
    assert ffn.score == "logits" and ffn.chosen_softmax and ffn.router_bias and ffn.activation == "sigmoid_limit"
    assert isinstance(ffn.shared, GatedMLPSpec) and (ffn.shared.hidden_dim, ffn.shared.limit, ffn.shared.activation) == (16, 1.0, "sigmoid_limit")
    plain_b = config_from_dict(CONFIG_B).to_plan()
    assert plain_b.layers[0].mixer.position is None and plain_b.layers[0].ffn.shared is None and plain_b.embedding.scale == 1.0


def test_the_order_in_which_layers_run():
    for name, config in CONFIGS.items():
        schedule = config_from_dict(config).to_plan().schedule
        assert [(entry.layer, entry.add_embedding) for entry in schedule] == plain.layer_runs(config), name
        assert all(entry.cache_from is None for entry in schedule)   # every run has a cache of its own
    runs = [(entry.layer, entry.add_embedding) for entry in config_from_dict(CONFIG_A).to_plan().schedule]
    assert runs == [(0, False), (1, False), (2, False), (1, True), (2, False), (1, True), (2, False), (3, False)]
    edge = copy.deepcopy(CONFIG_A)
    edge["loop"] = {"start": 2, "stop": 2, "times": 5}   # an empty stretch: every layer once
    assert [entry.layer for entry in config_from_dict(edge).to_plan().schedule] == [0, 1, 2, 3]


@pytest.mark.parametrize("path,value,key", [
    (("layers", 0, "type"), "recurrent", "layers[0].type"),
    (("layers", 1, "mixer", "kv_heads"), 3, "layers[1].mixer.kv_heads"),
    (("layers", 1, "mixer", "rot", "dims"), 18, "layers[1].mixer.rot.dims"),
    (("layers", 0, "mixer", "rot_dim"), 7, "layers[0].mixer.rot_dim"),
    (("layers", 0, "mixer", "kv_rank"), None, "layers[0].mixer.kv_rank"),
    (("layers", 0, "mlp", "router", "top"), 7, "layers[0].mlp.router.top"),
    (("layers", 1, "mlp", "kind"), "dense", "layers[1].mlp.kind"),
    (("layers", 1, "mlp", "expert", "limit"), None, "layers[1].mlp.expert.limit"),
    (("loop", "stop"), 9, "loop"),
    (("width",), None, "config.width"),
])
def test_errors_name_the_key(path, value, key):
    raw = copy.deepcopy(CONFIG_A)
    node = raw
    for step in path[:-1]:
        node = node[step]
    node[path[-1]] = value
    with pytest.raises(ConfigError) as error:
        config_from_dict(raw)
    assert key in str(error.value)


def test_tensor_names_and_shapes_and_loading(tmp_path):
    for name in ("A", "B"):
        config = CONFIGS[name]
        folder, _ = write_model(tmp_path / name, config, 3)
        typed = load_config(folder)
        plan = typed.to_plan()
        declared = {typed.checkpoint_names(*key)[0]: tuple(decl.shape) for key, decl in plan_tensor_decls(plan).items()}
        assert declared == tensor_shapes(config)
        tensors = load_weights(folder, typed, plan)
        assert len(tensors) == len(declared)
    missing = copy.deepcopy(CONFIG_A)
    missing["layers"][0]["mixer"]["kv_rank"] = 40   # the checkpoint's tensors do not fit
    (tmp_path / "A" / "config.json").write_text(__import__("json").dumps(missing))
    with pytest.raises(WeightsError):
        load_weights(tmp_path / "A", load_config(tmp_path / "A"))


def test_random_weights_round_trip(tmp_path):
    from lalamo_b200.weights.random_init import write_random_model

    folder = write_random_model(tmp_path / "random", CONFIG_A, seed=5)
    typed = load_config(folder)
    assert typed.to_json_dict()["loop"] == CONFIG_A["loop"]
    tensors = load_weights(folder, typed)
    norm = tensors[(("layers", 0, "mixer_norm"), "scale")]
    assert norm.abs().max() < 0.5   # used as 1 + w: made around zero
    assert (tensors[(("layers", 0, "mixer"), "latent_norm")] - 1).abs().max() < 0.5


def test_a_latent_layer_caches_one_row_per_token():
    from lalamo_b200.parts.latent_attention import LatentAttention

    spec = config_from_dict(CONFIG_E).to_plan().layers[0].mixer
    need = LatentAttention.cache_need(type("Holder", (), {"spec": spec})())
    assert need == PagedKVNeed(num_groups=1, head_dim=52, window=13, value_dim=40, values_in_keys=True)
    manager = CacheManager([need, need], [None, None], None, page_size=4, num_pages=8, num_slots=2)
    manager.admit("a")
    manager.reserve("a", 30)
    manager.commit("a", 30)
    # positions 18 .. 29 stay visible to the next query: blocks 0 .. 3 are given back
    assert manager.requests["a"].blocks[0][:4] == [-1] * 4 and all(page >= 0 for page in manager.requests["a"].blocks[0][4:])
    manager.release("a")
    manager.check()


def test_plain_rotations_agree_on_reordered_channels():
    """Pairs (2i, 2i + 1) are pairs (i, i + dims / 2) of the channels taken evens first, odds second."""
    generator = np.random.default_rng(0)
    x = generator.standard_normal((5, 3, 12))
    positions = np.array([0, 1, 7, 100, 4000])
    order = np.concatenate([np.arange(0, 8, 2), np.arange(1, 8, 2), np.arange(8, 12)])
    pairs = plain.rotate_pairs(x, positions, 8, 50.0)
    halves = plain.rotate_half(x[..., order], positions, 8, 50.0)
    assert np.allclose(pairs[..., order], halves)
    assert np.allclose(pairs[..., 8:], x[..., 8:]) and np.allclose(pairs[0], x[0])   # the rest passes; position 0 turns nothing
    assert np.allclose(np.linalg.norm(pairs, axis=-1), np.linalg.norm(x, axis=-1))


def test_plain_routing_by_hand():
    w = {"r.router": np.array([[1.0, 0.0], [0.0, 1.0], [1.0, 1.0]]), "r.router.b": np.array([0.0, 0.5, -3.0])}
    chosen, weights = plain.route(np.array([[2.0, 1.0], [0.0, 0.0]]), w, "r.", 2)
    assert chosen.tolist() == [[0, 1], [1, 0]]   # logits (2, 1.5, 0) and (0, 0.5, -3)
    assert np.allclose(weights[0], np.exp([2.0, 1.5]) / np.exp([2.0, 1.5]).sum()) and np.allclose(weights.sum(-1), 1.0)
    hidden = plain.expert(np.array([[1.0]]), {"e.gate": np.array([[5.0]]), "e.up": np.array([[-7.0]]), "e.down": np.array([[1.0]])}, "e.", 2.0)
    assert np.allclose(hidden, 2.0 / (1.0 + np.exp(-1.702 * 2.0)) * (-2.0 + 1.0))
