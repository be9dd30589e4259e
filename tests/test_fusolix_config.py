"""The Fusolix configuration on the CPU: registry, the model's description and tensor names, refused configurations,
cache groups and state, and the plain implementation's own consistency (a retention in portions and in closed form,
the convolution with a history, which blocks a query sees, the choice of experts within groups)."""
import copy

import pytest
import torch

import fusolix_cases as cases
import plain_fusolix as plain
from torchlet_b200.config import FusolixConfig, config_from_dict, known_architectures
from torchlet_b200.parts import LayeredModel, expected_tensors


def test_registered_and_chosen_by_name():
    assert "Fusolix" in known_architectures()
    for name in ("P", "Q", "R", "S", "T"):
        config = config_from_dict(cases.CASES[name])
        assert isinstance(config, FusolixConfig)
        assert FusolixConfig.from_dict(config.to_dict()) == config


def test_description_and_tensor_names():
    spec = cases.config_for("P").model_spec()
    assert [layer.block for layer in spec.layers] == ["hyper_connected"] * 4 and spec.streams == 3
    assert [layer.mixer.kind for layer in spec.layers] == ["parallel_mixers"] * 4
    assert [b["mixer"].kind for b in spec.layers[0].mixer.params["branches"]] == ["pooled_window_attention", "retention"]
    assert [layer.feed_forward.kind if layer.feed_forward else None for layer in spec.layers] == \
        ["clamped_glu", "routed_clamped_glu", None, "routed_clamped_glu"]
    assert spec.layers[2].feed_forward is None and len(spec.layers[2].norms) == 1
    names = {t.name: t.shape for t in expected_tensors(spec)}
    for name, shape in {"embed": (101, 96), "head": (101, 96), "final.norm": (96,), "final.norm.b": (96,),
                        "l0.norm1": (96,), "l0.norm1.b": (96,), "l0.norm2.b": (96,), "l0.canon1": (96, 4), "l0.canon2": (96, 4),
                        "l0.hc1.in": (3,), "l0.hc1.out": (3,), "l0.hc2.mix": (3, 3),
                        "l0.mix.left.q": (96, 96), "l0.mix.left.q.b": (96,), "l0.mix.left.k": (48, 96), "l0.mix.left.v": (32, 96),
                        "l0.mix.left.v.b": (32,), "l0.mix.left.o": (96, 64), "l0.mix.left.o.b": (96,),
                        "l0.mix.right.q": (36, 96), "l0.mix.right.k": (36, 96), "l0.mix.right.v": (60, 96),
                        "l0.mix.right.g": (60, 96), "l0.mix.right.o": (96, 60),
                        "l0.mlp.gate": (40, 96), "l0.mlp.up": (40, 96), "l0.mlp.down": (96, 40),
                        "l1.mlp.router": (6, 96), "l1.mlp.e5.gate": (24, 96), "l1.mlp.e0.down": (96, 24),
                        "l2.mix.left.v": (40, 96), "l2.hc1.mix": (3, 3)}.items():
        assert names[name] == shape, name
    for absent in ("l2.norm2", "l2.hc2.in", "l2.canon2", "l2.mlp.gate", "l0.mix.right.q.b", "l1.mlp.gate"):
        assert absent not in names
    assert not spec.tie_word_embeddings and spec.embedding_scale == 1.7
    routed = spec.layers[1].feed_forward.params
    assert (routed["groups"], routed["keep"], routed["score"], routed["renormalize"], routed["limit"]) == (3, 2, "softmax", True, None)
    plain_names = {t.name for t in expected_tensors(cases.config_for("T").model_spec())}
    assert not any("canon" in name for name in plain_names)


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="conv"), "unknown type"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["right"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(decay=[0.5]), "decays for"),
    (lambda c: c["layers"][0]["mixer"]["left"].pop("mask"), "lacks mask"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=5), "exceeds"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=4), "equal groups"),
    (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), "unknown mlp kind"),
    (lambda c: c["canon"].update(taps=9), "taps"),
    (lambda c: c.update(streams=0), "positive"),
    (lambda c: c.pop("width"), "lacks required keys"),
])
def test_refused_configurations(change, message):
    raw = copy.deepcopy(cases.CASES["P"])
    change(raw)
    with pytest.raises(ValueError, match=message):
        FusolixConfig.from_dict(raw)


def test_cache_groups_and_state():
    model = LayeredModel(cases.config_for("P").model_spec())
    needs = model.cache_needs()
    # one row [key | value] a token; held while the token is in the window or its block is open
    assert [(n.kv.num_kv_heads, n.kv.head_dim, n.kv.window) for n in needs] == [(2, 40, 13), (2, 40, 37), (1, 52, 16), (3, 16, 20)]
    for need, (pool, shape, state) in zip(needs, [(5, (2, 40), (3, 12, 20)), (3, (2, 40), (2, 24, 8)), (16, (1, 52), (3, 12, 20)),
                                                  (4, (3, 16), (1, 40, 8))]):
        assert need.state["left."].per_tokens == pool and tuple(need.state["left."].shape) == shape
        assert need.state["left."].slot_shape(100) == (-(-100 // pool), *shape)
        assert tuple(need.state["right."].shape) == state and need.state["right."].dtype == "float32"
    assert [sorted(n.block_state) for n in needs] == [["feed_forward", "mixer"]] * 2 + [["mixer"]] + [["feed_forward", "mixer"]]
    assert tuple(needs[0].block_state["mixer"].shape) == (3, 96)
    for name in ("S", "T"):  # one tap and no convolution keep nothing
        assert all(n.block_state is None for n in LayeredModel(cases.config_for(name).model_spec()).cache_needs())


def test_plain_retention_in_portions_and_in_closed_form():
    g = torch.Generator().manual_seed(3)
    q, k = (torch.rand(30, 6, generator=g, dtype=torch.float64) for _ in range(2))
    v = torch.rand(30, 4, generator=g, dtype=torch.float64)
    whole, _ = plain.retention(q, k, v, 0.9)
    first, state = plain.retention(q[:11], k[:11], v[:11], 0.9)
    rest, _ = plain.retention(q[11:], k[11:], v[11:], 0.9, state)
    assert torch.allclose(torch.cat([first, rest]), whole, rtol=1e-12)
    t = 7
    want = sum(0.9 ** (t - s) * (k[s] @ q[t]) * v[s] for s in range(t + 1))  # o_t = sum_s a^(t - s) (k_s . q_t) v_s
    assert torch.allclose(whole[t], want, rtol=1e-12)


def test_plain_convolution_with_a_history():
    g = torch.Generator().manual_seed(4)
    h = torch.rand(12, 5, generator=g, dtype=torch.float64)
    w = torch.rand(5, 3, generator=g, dtype=torch.float64)
    whole = plain.causal_conv(h, w)
    assert torch.allclose(whole[0], w[:, 2] * h[0]) and torch.allclose(whole[1], w[:, 1] * h[0] + w[:, 2] * h[1])
    assert torch.allclose(whole[5], w[:, 0] * h[3] + w[:, 1] * h[4] + w[:, 2] * h[5])
    rest = plain.causal_conv(h[7:], w, history=h[5:7])
    assert torch.allclose(rest, whole[7:], rtol=1e-12)
    assert torch.allclose(plain.causal_conv(h, w[:, :1]), w[:, :1].T * h)  # one tap: a factor on the token itself


def test_which_blocks_a_query_sees():
    # a window of 5, blocks of 3: block 0 (positions 0..2) is seen from position 7 on (2 <= 7 - 5), block 1 from 10 on
    assert [plain.visible_blocks(i, 5, 3) for i in range(12)] == [0, 0, 0, 0, 0, 0, 0, 1, 1, 1, 2, 2]
    assert [plain.visible_blocks(i, 1, 1) for i in range(4)] == [0, 1, 2, 3]
    T = 12
    v = torch.eye(T, dtype=torch.float64)
    out = plain.pooled_window_attention(torch.zeros(T, 2, dtype=torch.float64), torch.zeros(T, 2, dtype=torch.float64), v, 1.0, 5, 3)
    # position 8: the window holds 4..8, block 0 is seen as one key whose value is the mean of rows 0..2; token 3 is
    # out of the window and its block not yet seen: six keys of equal score
    want = torch.tensor([1 / 18] * 3 + [0] + [1 / 6] * 5 + [0] * 3, dtype=torch.float64)
    assert torch.allclose(out[8], want)
    assert torch.allclose(out[3], torch.tensor([0.25] * 4 + [0] * 8, dtype=torch.float64))


def test_choice_of_experts_within_groups():
    s = torch.tensor([0.05, 0.30, 0.20, 0.02, 0.25, 0.03, 0.05, 0.10], dtype=torch.float64)
    assert plain.choose_experts(s, 2, 1, 1) == [1, 4]
    assert plain.choose_experts(s, 3, 4, 2) == [1, 4, 0]   # groups 0 (0.30) and 2 (0.25) are kept: expert 2 is out
    assert plain.choose_experts(s, 2, 4, 1) == [1, 0]
    assert plain.choose_experts(torch.full((6,), 1 / 6, dtype=torch.float64), 3, 3, 2) == [0, 1, 2]  # the lower index wins
