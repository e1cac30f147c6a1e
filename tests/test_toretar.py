"""Toretar without a GPU: the configuration reader, the plan, the checkpoint layout, the cache
need of a latent attention layer, and the plain implementation's mechanisms against hand-worked
numbers."""
import copy

import numpy as np
import pytest

import plain_toretar as plain
from tiny_configs import TORETAR_A, TORETAR_B


def test_config_selects_the_architecture_and_reads_back():
    from gemmars_b200.config.registry import resolve_architecture
    arch = resolve_architecture(TORETAR_A)
    assert arch.name == "Toretar"
    cfg = arch.config_class.from_dict(TORETAR_A)
    assert cfg.vocab == 301 and cfg.width == 72 and len(cfg.layers) == 3
    assert arch.config_class.from_dict(cfg.to_dict()) == cfg


def test_config_reports_every_problem_at_once():
    from gemmars_b200.config.base import ConfigError
    from gemmars_b200.models.toretar import ToretarConfig
    bad = copy.deepcopy(TORETAR_A)
    bad["vocab"] = "many"
    bad["layers"][0]["mixer"]["heads"] = 0
    bad["layers"][0]["mlp"]["router"]["top"] = 9
    bad["layers"][1]["type"] = "convolution"
    bad["layers"][2]["mixer"]["rot"]["dims"] = 3
    with pytest.raises(ConfigError) as e:
        ToretarConfig.from_dict(bad)
    msg = str(e.value)
    for piece in ("config.vocab", "layers[0].mixer.heads", "layers[0].mlp.router.top", "layers[1].type", "layers[2].mixer.rot.dims"):
        assert piece in msg, piece


@pytest.mark.parametrize("raw", [TORETAR_A, TORETAR_B], ids=["A", "B"])
def test_plan_wants_exactly_the_checkpoint_layout(raw):
    from gemmars_b200.engine.model import DecoderModel
    from gemmars_b200.models.toretar import ToretarConfig, build_plan, checkpoint_layout
    cfg = ToretarConfig.from_dict(raw)
    model = DecoderModel(build_plan(cfg), "float32", "cpu")
    want = model.expected_tensors()
    layout = {n: tuple(s) for n, (s, _) in checkpoint_layout(cfg).items()}
    assert want == layout
    # a layer without a feed-forward has two parts, the others three; every layer keeps one cache
    assert [len(b.parts()) for b in model.blocks] == [3 if layer["mlp"] else 2 for layer in raw["layers"]]
    needs = model.cache_needs()
    assert len(needs) == len(raw["layers"])
    for (_, (need,)), layer in zip(needs, raw["layers"]):
        m = layer["mixer"]
        assert (need.num_kv_heads, need.head_dim, need.value_dim, need.window) == (1, m["kv_rank"] + m["rot_dim"], 0, None)


def test_a_need_without_values_keeps_no_value_storage():
    import torch
    from gemmars_b200.cache.pool import KVNeed, SequenceCache
    cache = SequenceCache([(0, KVNeed(1, 40, None, value_dim=0)), (1, KVNeed(2, 16))], 256, 4, 0, 64, torch.float32, "cpu")
    g, k, v = cache.kv(0)
    assert k.shape[1:] == (1, 64, 40) and v.numel() == 0
    g2, k2, v2 = cache.kv(1)
    assert v2.shape[1:] == (2, 16, 64)
    s = cache.open()
    cache.extend(s, 70)
    assert g.pages.held_count == 2 and g2.pages.held_count == 2
    cache.close(s)
    assert cache.pages_held() == 0


def test_rotation_pairs_neighbours_and_leaves_the_rest():
    v = np.array([[[1.0, 0.0, 0.0, 2.0, 5.0, 7.0]]])         # one token, one head, 6 dims, 4 rotate
    out = plain.rotate_pairs(v, [3], 4, 100.0)
    a0, a1 = 3.0, 3.0 * 100.0 ** -0.5
    want = [np.cos(a0), np.sin(a0), -2 * np.sin(a1), 2 * np.cos(a1), 5.0, 7.0]
    assert np.allclose(out[0, 0], want, atol=1e-12)
    assert np.allclose(plain.rotate_pairs(v, [0], 4, 100.0), v)     # position 0 turns nothing


def test_router_softmax_is_over_the_chosen_only():
    h = np.eye(3)[:1]
    router = np.array([[1.0, 0, 0], [3.0, 0, 0], [2.0, 0, 0], [-1.0, 0, 0]])
    idx, wt = plain.route(h, router, np.array([0.0, 0.0, 0.5, 0.0]), 2)
    assert idx.tolist() == [[1, 2]]
    e = np.exp([3.0, 2.5])
    assert np.allclose(wt[0], e / e.sum())


def test_expert_clamps_before_the_activation():
    h = np.array([[1.0]])
    one = lambda g, u, lim: plain.expert(h, np.array([[g]]), np.array([[u]]), np.array([[1.0]]), lim)[0, 0]
    sig = lambda z: 1 / (1 + np.exp(-z))
    assert np.isclose(one(5.0, 0.2, 1.0), 1.0 * sig(1.702) * 1.2)          # gate clamped from above only
    assert np.isclose(one(-5.0, 0.2, 1.0), -5.0 * sig(-5 * 1.702) * 1.2)
    assert np.isclose(one(0.5, -9.0, 2.0), 0.5 * sig(0.851) * (-2.0 + 1))  # up clamped on both sides
    assert np.isclose(one(0.5, 9.0, 2.0), 0.5 * sig(0.851) * 3.0)


def test_plain_attention_is_causal_and_gated(tmp_path):
    from gemmars_b200.weights import write_random_model
    folder = write_random_model(str(tmp_path / "m"), TORETAR_A, 5)
    cfg, w = plain.load_folder(folder)
    rng = np.random.default_rng(0)
    toks = rng.integers(0, cfg["vocab"], 12).tolist()
    full = plain.forward(cfg, w, toks)
    assert np.allclose(plain.forward(cfg, w, toks[:7]), full[:7], atol=1e-12)
    # a layer without feed-forward adds the mixer's output and nothing else; with zero gate weights
    # every head passes at sigmoid(0) = 1/2, so the mixer is half of what it is with the gates open
    w2 = dict(w)
    w2["l1.mix.g"] = np.zeros_like(w["l1.mix.g"])
    res = []
    plain.forward(cfg, w2, toks, res)
    h = plain.rms_norm(res[0], w2["l1.norm1"], cfg["norm"]["eps"])
    halved = plain.latent_attention(h, w2, "l1.mix.", cfg["layers"][1]["mixer"], cfg["norm"]["eps"])
    assert np.allclose(res[1], res[0] + halved, atol=1e-9) and np.abs(halved).max() > 0
    w3 = dict(w2)
    w3["l1.mix.o"] = 2.0 * w2["l1.mix.o"]
    assert np.allclose(plain.latent_attention(h, w3, "l1.mix.", cfg["layers"][1]["mixer"], cfg["norm"]["eps"]), 2.0 * halved)
