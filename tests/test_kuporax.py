"""Kuporax without a GPU: the configuration, the plan against the checkpoint layout, what the
layers ask of the cache, and the plain implementation's mechanisms against hand-worked numbers."""
import copy

import numpy as np
import pytest

import plain_kuporax as plain
from tiny_configs import KUPORAX_A, KUPORAX_B, KUPORAX_C


def test_configuration_reports_every_problem_at_once():
    from gemmars_b200.config.base import ConfigError
    from gemmars_b200.models.kuporax import KuporaxConfig
    cfg = KuporaxConfig.from_dict(KUPORAX_A)
    assert cfg.vocab == 211 and cfg.logit_scale == 1.7 and len(cfg.layers) == 4
    assert KuporaxConfig.from_dict(cfg.to_dict()) == cfg
    bad = copy.deepcopy(KUPORAX_A)
    bad["layers"][0]["mixer"]["left"]["rot"]["dims"] = 26          # more than dim
    bad["layers"][1]["mixer"]["heads"] = 5                          # not a multiple of kv_heads
    bad["layers"][2]["type"] = "conv"
    del bad["logit_scale"]
    bad["layers"][3]["mlp"]["kind"] = "moe"
    with pytest.raises(ConfigError) as e:
        KuporaxConfig.from_dict(bad)
    text = str(e.value)
    for piece in ("rot.dims", "5 heads", "unknown mixer 'conv'", "logit_scale", "unknown feed-forward 'moe'"):
        assert piece in text


@pytest.mark.parametrize("raw", [KUPORAX_A, KUPORAX_B, KUPORAX_C], ids="ABC")
def test_plan_wants_exactly_the_checkpoint(raw):
    from gemmars_b200.config.registry import resolve_architecture
    from gemmars_b200.engine.model import DecoderModel
    arch = resolve_architecture(raw)
    cfg = arch.config_class.from_dict(raw)
    model = DecoderModel(arch.build_plan(cfg, None), "float32", "cpu")
    layout = {name: tuple(shape) for name, (shape, _) in arch.checkpoint_layout(cfg).items()}
    assert model.expected_tensors() == layout
    assert model.plan.max_positions == raw["max_positions"]


def test_what_the_layers_keep_per_sequence():
    import torch
    from gemmars_b200.cache.pool import KVNeed, SequenceCache, StateNeed
    from gemmars_b200.engine.model import build_model
    from gemmars_b200.weights import random_weights
    model = build_model(raw_config=KUPORAX_A, tensors=random_weights(KUPORAX_A, 1), dtype="float32", device="cpu",
                        compile_kernels=False)
    needs = dict(model.cache_needs())
    # (a recurrent state's dims are padded to 32 a lane: 32 * lanes * vdim floats a head)
    # side by side: keys of 24 with values of 40 in a window of 50 and one tap of memory, then the
    # state-space branch's filter memory and state
    assert needs[0] == [KVNeed(2, 24, 50, 40), StateNeed((1, 6 * 24 + 2 * 40)), StateNeed((2, 48 + 24)), StateNeed((3, 32 * 16))]
    assert needs[1] == [StateNeed((2, 2 * 64 + 96)), StateNeed((4, 32 * 24))]
    # a filter of one tap remembers nothing
    assert needs[2] == [KVNeed(3, 32, 9, 16), StateNeed((1, 32 + 2 * 4 * 20)), StateNeed((4, 32 * 8))]
    cache = SequenceCache(model.cache_needs(), 512, 4, 600, 64, torch.float32, "cpu")
    slot = cache.open()
    cache.extend(slot, 300)
    windows = sorted(g.need.window for g in cache.kv_groups)
    assert windows == [9, 50]
    assert all(g.table_width < 5 for g in cache.kv_groups)         # rings, not 300 tokens' worth of pages
    state = cache.state_groups[0].data
    state[:, slot] = 1.0
    cache.close(slot)
    assert cache.pages_held() == 0
    assert cache.open() == slot and not cache.state_groups[0].data[:, slot].any()      # a slot taken again starts from zero


def test_short_filter_by_hand():
    u = np.array([[1.0, 10.0], [2.0, 20.0], [3.0, 30.0], [4.0, 40.0]])
    taps = np.array([[0.5, 0.25, 1.0], [0.0, 1.0, -1.0]])         # last column: the current token
    y = plain.short_conv(u, taps)
    assert np.allclose(y[:, 0], [1.0, 2.0 + 0.25, 3.0 + 0.5 + 0.5, 4.0 + 0.75 + 1.0])
    assert np.allclose(y[:, 1], [-10.0, -10.0, -10.0, -10.0])
    assert np.allclose(plain.short_conv(u, taps, np.array([1.0, 2.0])), y + [1.0, 2.0])


def test_rotation_of_halves_by_hand():
    x = np.zeros((2, 1, 6))
    x[:, 0] = [1.0, 2.0, 3.0, 4.0, 5.0, 6.0]
    out = plain.rotate_half(x, np.array([0, 3]), 100.0, 4)
    assert np.allclose(out[0], x[0])                                # position 0 turns nothing
    a0, a1 = 3.0, 3.0 * 100.0 ** -0.5
    assert np.allclose(out[1, 0, [0, 2]], [np.cos(a0) - 3 * np.sin(a0), 3 * np.cos(a0) + np.sin(a0)])
    assert np.allclose(out[1, 0, [1, 3]], [2 * np.cos(a1) - 4 * np.sin(a1), 4 * np.cos(a1) + 2 * np.sin(a1)])
    assert np.allclose(out[1, 0, 4:], [5.0, 6.0])                   # beyond the rotated dims


def test_delta_rule_by_hand():
    # one head, keys along the axes: the first token writes v0 under e0; the second, with the same
    # key, replaces a share beta of what is read there; the read-out sees the write of its own token
    e0 = np.array([1.0, 0.0])
    q = np.stack([e0, e0, e0]).reshape(3, 1, 2)
    k = q.copy()
    v = np.array([[2.0, 4.0], [10.0, 20.0], [0.0, 0.0]]).reshape(3, 1, 2)
    beta = np.array([[1.0], [0.5], [0.0]])
    decay = np.array([[1.0], [0.5], [1.0]])
    out, S = plain.delta_scan(q, k, v, beta, decay)
    assert np.allclose(out[0, 0], [2.0, 4.0])
    # S decays to [1, 2]; u = 0.5 ([10, 20] - [1, 2]) = [4.5, 9]; S = [5.5, 11]
    assert np.allclose(out[1, 0], [5.5, 11.0])
    assert np.allclose(out[2, 0], [5.5, 11.0])                      # beta 0 writes nothing, decay 1 keeps all
    assert np.allclose(S[0], [[5.5, 11.0], [0.0, 0.0]])


def test_state_space_by_hand():
    x = np.array([[[2.0]], [[3.0]]])                                # one head, one value dim
    B = np.array([[[1.0, 0.0]], [[0.0, 1.0]]])
    C = np.array([[[1.0, 1.0]], [[1.0, 2.0]]])
    dt = np.array([[0.5], [2.0]])
    y, S = plain.ssd_scan(x, B, C, dt, np.array([1.0]), np.array([10.0]))
    assert np.allclose(y[0, 0], 0.5 * 2.0 + 10.0 * 2.0)
    d = np.exp(-2.0)
    assert np.allclose(S[0, :, 0], [d * 1.0, 6.0])
    assert np.allclose(y[1, 0], d * 1.0 + 2 * 6.0 + 30.0)


def test_window_and_cap_by_hand():
    k = np.zeros((4, 1, 2))
    k[:, 0, 0] = [1.0, 2.0, 3.0, 4.0]
    v = np.arange(4.0).reshape(4, 1, 1)
    q = np.ones((1, 1, 2))
    # the query at position 3 with a window of 2 sees positions 2 and 3 only
    out = plain.capped_attention(q, k, v, [3], [0, 1, 2, 3], 1.0, None, 2)
    w = np.exp([3.0, 4.0]) / np.exp([3.0, 4.0]).sum()
    assert np.allclose(out[0, 0, 0], w @ [2.0, 3.0])
    out = plain.capped_attention(q, k, v, [3], [0, 1, 2, 3], 1.0, 2.0, None)
    s = 2.0 * np.tanh(np.array([1.0, 2.0, 3.0, 4.0]) / 2.0)
    assert np.allclose(out[0, 0, 0], (np.exp(s) / np.exp(s).sum()) @ [0.0, 1.0, 2.0, 3.0])


def test_the_first_tokens_see_nothing_before_them():
    from gemmars_b200.weights import random_weights
    w = {k: v.double().numpy() for k, v in random_weights(KUPORAX_C, 4).items()}
    toks = [3, 50, 7, 7, 90, 11]
    whole = plain.forward(KUPORAX_C, w, toks)
    for n in (1, 2, 3):
        assert np.allclose(plain.forward(KUPORAX_C, w, toks[:n]), whole[:n], atol=1e-12)     # causal throughout
    other = plain.forward(KUPORAX_C, w, [4] + toks[1:])
    assert not np.allclose(other[-1], whole[-1])                    # the recurrent layers remember the first token
