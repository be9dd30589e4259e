"""The Kilatar configuration on the CPU: registry, the model's description and tensor names, the order in which looped
layers run, refused configurations, cache groups and state, and the plain implementation's own consistency (the
recurrences in closed form, the convolution, which keys a chunk shows, the frequency table, the router)."""
import copy
import math

import pytest
import torch

import kilatar_cases as cases
import plain_kilatar as plain
from torchlet_b200.config import KilatarConfig, config_from_dict, known_architectures
from torchlet_b200.parts import LayeredModel, expected_tensors


def test_registered_and_chosen_by_name():
    assert "Kilatar" in known_architectures()
    for name in ("P", "Q", "R"):
        config = config_from_dict(cases.CASES[name])
        assert isinstance(config, KilatarConfig)
        assert KilatarConfig.from_dict(config.to_dict()) == config


def test_description_and_tensor_names():
    spec = cases.config_for("P").model_spec()
    assert [layer.block for layer in spec.layers] == ["parallel_scaled"] * 5
    assert [layer.mixer.kind for layer in spec.layers] == ["parallel_mixers", "mamba2", "latent_attention", "parallel_mixers", "mamba2"]
    branches = spec.layers[0].mixer.params["branches"]
    assert [b["mixer"].kind for b in branches] == ["gated_attention", "retention"]
    assert [b["scale"] for b in branches] == [0.5, 0.5] and all(b["norm"].kind == "rms_norm" for b in branches)
    assert branches[0]["mixer"].params["chunk"] == 13 and branches[0]["mixer"].params["positions"].params["pairing"] == "interleaved"
    assert [layer.feed_forward.kind if layer.feed_forward else None for layer in spec.layers] == \
        ["routed_clamped_glu", "gated_mlp", "routed_clamped_glu", None, None]
    assert spec.embedding_norm is not None and spec.embedding_norm_prefix == "embed.norm"
    names = {t.name: t.shape for t in expected_tensors(spec)}
    for name, shape in {"embed": (101, 96), "embed.norm": (96,), "head": (101, 96), "final.norm": (96,), "l0.norm1": (96,),
                        "l0.mix.left.q": (96, 96), "l0.mix.left.k": (48, 96), "l0.mix.left.v": (32, 96), "l0.mix.left.o": (96, 64),
                        "l0.mix.left.out": (96,), "l0.mix.right.out": (96,), "l0.mix.right.q": (36, 96), "l0.mix.right.v": (60, 96),
                        "l0.mix.right.g": (60, 96), "l0.mix.right.norm": (60,), "l0.mix.right.o": (96, 60),
                        "l0.mlp.router": (8, 96), "l0.mlp.correction": (8,), "l0.mlp.e5.gate": (24, 96), "l0.mlp.shared.up": (40, 96),
                        "l0.mlp.shared.sg": (1, 96), "l1.mix.in": (2 * 48 + 2 * 40 + 4, 96), "l1.mix.conv": (48 + 80, 4),
                        "l1.mix.conv.b": (128,), "l1.mix.dt_bias": (4,), "l1.mix.A_log": (4,), "l1.mix.D": (4,), "l1.mix.norm": (48,),
                        "l1.mix.o": (96, 48), "l1.mlp.gate": (40, 96), "l1.mlp.gate.b": (40,), "l1.mlp.down.b": (96,),
                        "l2.mix.q": (96, 96), "l2.mix.dkv": (52, 96), "l2.mix.dkv.norm": (40,), "l2.mix.uk": (60, 40),
                        "l2.mix.uv": (84, 40), "l2.mix.g": (84, 96), "l2.mix.o": (96, 84), "l2.mlp.router": (5, 96)}.items():
        assert names[name] == shape, name
    for absent in ("l0.mlp.e6.gate", "l2.mlp.shared.gate", "l3.mlp.gate", "l4.mlp.router", "l2.mix.dq", "l0.norm2"):
        assert absent not in names
    routed = spec.layers[0].feed_forward.params
    assert (routed["identity"], routed["weight_scale"], routed["score"], routed["renormalize"], routed["correction"]) == \
        (2, 1.7, "softmax", True, True)


def test_the_order_in_which_looped_layers_run():
    runs = lambda name: [(e.layer, e.add_embedding) for e in cases.config_for(name).model_spec().schedule]
    assert runs("P") == [(0, False), (1, False), (2, False), (1, True), (2, False), (1, True), (2, False), (3, False), (4, False)]
    assert runs("Q") == [(0, False), (1, False), (0, True), (1, False), (2, False)]
    assert runs("R") == [(i, False) for i in range(4)]
    assert plain.layer_runs(cases.CASES["P"]) == runs("P") and plain.layer_runs(cases.CASES["Q"]) == runs("Q")
    once = copy.deepcopy(cases.CASES["P"])
    once["loop"]["times"] = 1
    assert [(e.layer, e.add_embedding) for e in KilatarConfig.from_dict(once).model_spec().schedule] == [(i, False) for i in range(5)]


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="conv"), "unknown type"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(decay=[0.5]), "decays for"),
    (lambda c: c["layers"][0]["mixer"]["left"].pop("mask"), "lacks mask"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "do not fit"),
    (lambda c: c["layers"][1]["mlp"].update(kind="sparse"), "unknown mlp kind"),
    (lambda c: c["layers"][1]["mixer"].update(groups=3), "do not split"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=14), "at most"),
    (lambda c: c["loop"].update(stop=9), "do not lie within"),
    (lambda c: c.pop("width"), "lacks required keys"),
])
def test_refused_configurations(change, message):
    raw = copy.deepcopy(cases.CASES["P"])
    change(raw)
    with pytest.raises(ValueError, match=message):
        KilatarConfig.from_dict(raw)


def test_cache_groups_and_state():
    model = LayeredModel(cases.config_for("P").model_spec())
    needs = model.cache_needs()
    assert len(needs) == 9 and [n.owner for n in needs] == list(range(9))  # every run of a looped layer keeps its own
    first = needs[0]  # heads of 24 x 16 are laid out in rows of 24; pages are given back a chunk behind
    assert (first.kv.num_kv_heads, first.kv.head_dim, first.kv.window, first.kv.planes) == (2, 24, 13, 2)
    assert tuple(first.state["right."].shape) == (3, 12, 20) and "left." not in first.state
    mamba = needs[1]
    assert mamba.kv is None and tuple(mamba.state["ssm"].shape) == (4, 20, 12) and tuple(mamba.state["conv"].shape) == (3, 128)
    latent = needs[2]
    assert (latent.kv.num_kv_heads, latent.kv.head_dim, latent.kv.window, latent.kv.planes) == (1, 52, None, 1)
    assert needs[7].kv.head_dim == 16 and needs[7].kv.window == 5  # 8 x 12 heads: rows of 16
    one_tap = LayeredModel(cases.config_for("Q").model_spec()).cache_needs()[4]
    assert sorted(one_tap.state) == ["ssm"]  # one tap reads the token itself: nothing to keep


def test_plain_recurrences_in_closed_form():
    g = torch.Generator().manual_seed(3)
    width, T = 10, 9
    h = torch.rand(T, width, generator=g, dtype=torch.float64)
    m = {"heads": 1, "dim": 3, "vdim": 2, "decay": [0.8]}
    w = {"r.q": torch.rand(3, width, generator=g, dtype=torch.float64), "r.k": torch.rand(3, width, generator=g, dtype=torch.float64),
         "r.v": torch.rand(2, width, generator=g, dtype=torch.float64), "r.g": torch.zeros(2, width, dtype=torch.float64),
         "r.o": torch.eye(2, dtype=torch.float64), "r.norm": torch.ones(2, dtype=torch.float64)}
    got = plain.lightning_attention(m, w, "r.", h, 1e-9)
    q, k, v = (plain.silu(h @ w[n].T) for n in ("r.q", "r.k", "r.v"))
    t = 6
    o = sum(0.8 ** (t - s) * (k[s] @ q[t]) * v[s] for s in range(t + 1))  # o_t = sum_s a^(t - s) (k_s . q_t) v_s
    assert torch.allclose(got[t], 0.5 * plain.rms(o, 1e-9), rtol=1e-9)  # sigmoid(0) = 1/2
    # the state-space recurrence: y_t = sum_s prod_(s < r <= t) a_r dt_s (B_s . C_t) x_s + D x_t
    m = {"heads": 1, "vdim": 2, "state": 3, "groups": 1, "conv": 1, "norm_groups": 1}
    inner, n = 2, 3
    w = {"m.in": torch.rand(2 * inner + 2 * n + 1, width, generator=g, dtype=torch.float64) - 0.5,
         "m.conv": torch.ones(inner + 2 * n, 1, dtype=torch.float64), "m.conv.b": torch.zeros(inner + 2 * n, dtype=torch.float64),
         "m.dt_bias": torch.tensor([0.3], dtype=torch.float64), "m.A_log": torch.tensor([-0.5], dtype=torch.float64),
         "m.D": torch.tensor([1.5], dtype=torch.float64), "m.norm": torch.ones(inner, dtype=torch.float64),
         "m.o": torch.eye(inner, dtype=torch.float64)}
    got = plain.mamba2(m, w, "m.", h, 1e-12)
    proj = h @ w["m.in"].T
    z, x, B, C = proj[:, :2], plain.silu(proj[:, 2:4]), plain.silu(proj[:, 4:7]), plain.silu(proj[:, 7:10])
    dt = torch.log1p(torch.exp(proj[:, 10] + 0.3))
    a = torch.exp(-math.exp(-0.5) * dt)
    y = 1.5 * x[t] + sum(torch.prod(a[s + 1:t + 1]) * dt[s] * (B[s] @ C[t]) * x[s] for s in range(t + 1))
    assert torch.allclose(got[t], plain.rms(y * plain.silu(z[t]), 1e-12), rtol=1e-9)


def test_plain_convolution_and_chunks():
    g = torch.Generator().manual_seed(4)
    x = torch.rand(12, 5, generator=g, dtype=torch.float64)
    w = torch.rand(5, 3, generator=g, dtype=torch.float64)
    b = torch.rand(5, generator=g, dtype=torch.float64)
    out = plain.causal_conv(x, w, b)
    assert torch.allclose(out[0], b + w[:, 2] * x[0]) and torch.allclose(out[1], b + w[:, 1] * x[0] + w[:, 2] * x[1])
    assert torch.allclose(out[5], b + w[:, 0] * x[3] + w[:, 1] * x[4] + w[:, 2] * x[5])
    # chunks of 4: position 9 sees 8 and 9 only; equal scores give their mean
    T = 12
    v = torch.eye(T, dtype=torch.float64).view(T, 1, T)
    zero = torch.zeros(T, 1, 2, dtype=torch.float64)
    out = plain.softmax_attention(zero, zero, v, 1.0, lambda i, j: i // 4 == j // 4)[:, 0]
    want = torch.zeros(T, dtype=torch.float64)
    want[8:10] = 0.5
    assert torch.allclose(out[9], want)
    assert torch.allclose(out[8], torch.eye(T, dtype=torch.float64)[8]) and torch.allclose(out[7, 4:8], torch.full((4,), 0.25, dtype=torch.float64))


def test_plain_frequencies_and_router():
    f = plain.frequencies({"base": 100.0, "dims": 4, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 16}})
    # wavelengths 2 pi and 20 pi: the first lies between 16 / 4 and 16 / 1 and is blended; the second is longer than
    # 16 / 1 and slowed down by the factor
    s = (16 / (2 * math.pi) - 1.0) / 3.0
    assert math.isclose(float(f[0]), (1 - s) / 4.0 + s) and math.isclose(float(f[1]), 0.1 / 4.0)
    mlp = {"router": {"experts": 2, "top": 2, "identity": 1, "scale": 3.0}}
    w = {"m.router": torch.tensor([[1.0], [0.0], [2.0]], dtype=torch.float64),
         "m.correction": torch.tensor([0.0, 0.7, 0.0], dtype=torch.float64)}
    chosen, weight = plain.route(mlp, w, "m.", torch.ones(1, 1, dtype=torch.float64))
    s = torch.softmax(torch.tensor([1.0, 0.0, 2.0], dtype=torch.float64), 0)
    assert chosen.tolist() == [[1, 2]]  # expert 1 by its correction, then the identity expert
    assert torch.allclose(weight[0], 3.0 * s[[1, 2]] / (s[1] + s[2]))
