"""Rotepel on the CPU: the configuration reader, the run order, the tensor manifest, and the plain
implementation checked against closed forms of its own recurrences."""
import math

import pytest
import torch

from tests.plain import rotepel_plain as plain
from vllm_oxide_b200 import models  # noqa: F401  (registers the architectures)
from vllm_oxide_b200.config import RotepelConfig, architecture_for
from vllm_oxide_b200.errors import ConfigError, WeightsError
from vllm_oxide_b200.models.rotepel import rotepel_manifest
from vllm_oxide_b200.weights import random_tensors, weights_from_tensors


def _dict():
    return {"architecture": "Rotepel", "vocab": 40, "width": 24, "streams": 3, "norm": {"eps": 1e-5, "groups": 3},
            "loop": {"start": 1, "stop": 3, "times": 3},
            "layers": [
                {"type": "general_delta", "mixer": {"heads": 2, "dim": 8, "decay_rank": 3}, "mlp": {"kind": "dense", "ff": 20}},
                {"type": "retention", "mixer": {"heads": 2, "dim": 8, "vdim": 4, "decay": [0.9, 0.99], "rot": {"dims": 4, "base": 100.0}}, "mlp": None},
                {"type": "latent_attention", "mixer": {"heads": 2, "dim": 8, "rot_dim": 4, "vdim": 6, "kv_rank": 10, "scale": 0.25,
                                                       "rot": {"dims": 4, "base": 50.0}}, "mlp": {"kind": "dense", "ff": 16}},
                {"type": "general_delta", "mixer": {"heads": 1, "dim": 12}, "mlp": None}]}


def test_config_round_trip_run_order_and_registry():
    d = _dict()
    arch = architecture_for(d)
    assert arch.name == "Rotepel"
    cfg = arch.config_cls.from_dict(d)
    assert cfg.run_order() == (0, 1, 2, 1, 2, 1, 2, 3)
    assert RotepelConfig.from_dict(cfg.to_dict()) == cfg
    assert cfg.layers[1].ff == 0 and cfg.layers[0].decay_rank == 3 and cfg.layers[3].decay_rank is None
    d2 = _dict()
    del d2["loop"], d2["streams"]
    cfg2 = RotepelConfig.from_dict(d2)
    assert cfg2.run_order() == (0, 1, 2, 3) and cfg2.streams is None
    assert plain.run_order(d) == list(cfg.run_order()) and plain.run_order(d2) == [0, 1, 2, 3]


@pytest.mark.parametrize("change,msg", [
    (lambda d: d["layers"][0].update(type="conv"), "type"),
    (lambda d: d["layers"][1]["mixer"].update(decay=[0.9]), "decay"),
    (lambda d: d["layers"][2]["mixer"].update(rot_dim=6), "rot_dim"),
    (lambda d: d["norm"].update(groups=5), "groups"),
    (lambda d: d["loop"].update(stop=9), "loop"),
    (lambda d: d["layers"][2]["mlp"].update(kind="routed"), "kind"),
    (lambda d: d.pop("width"), "width"),
])
def test_config_refuses_what_does_not_fit(change, msg):
    d = _dict()
    change(d)
    with pytest.raises(ConfigError, match=msg):
        RotepelConfig.from_dict(d)


def test_manifest_names_shapes_and_a_dimension_left_to_the_file():
    cfg = RotepelConfig.from_dict(_dict())
    m = rotepel_manifest(cfg)
    assert m["l0.mix.w1"].shape == (3, 24) and m["l0.mix.w2"].shape == (16, 3) and m["l0.mix.a.b"].shape == (16,)
    assert m["l1.mix.q"].shape == (16, 24) and m["l1.mix.v"].shape == (8, 24) and "l1.norm2" not in m and "l1.hc2.in" not in m
    assert m["l2.mix.q"].shape == (24, 24) and m["l2.mix.dkv"].shape == (14, 24) and m["l2.mix.uk"].shape == (16, 10)
    assert m["l2.hc2.mix"].shape == (3, 3) and m["head"].shape == (40, 24)
    assert m["l3.mix.w1"].shape == (-1, 24)
    # the free dimension takes whatever the stored tensor has, as long as both tensors agree with their own shapes
    with pytest.raises(ValueError, match="left to the stored tensor"):
        random_tensors(m, 1)
    fixed = dict(m)
    for n in ("l3.mix.w1", "l3.mix.w2"):
        fixed[n] = type(m[n])(tuple(5 if x == -1 else x for x in m[n].shape))
    t = random_tensors(fixed, 1, dtype=torch.float32)
    weights_from_tensors(t, m)
    t["l3.mix.w1"] = torch.zeros(5, 23)
    with pytest.raises(WeightsError):
        weights_from_tensors(t, m)
    no_streams = dict(_dict())
    del no_streams["streams"]
    assert not any(".hc" in n for n in rotepel_manifest(RotepelConfig.from_dict(no_streams)))


def test_plain_retention_equals_its_closed_form():
    """o_t = sum_{j <= t} decay^(t - j) (q_t . k_j) v_j."""
    torch.manual_seed(0)
    T, W, H, D, V = 9, 12, 2, 4, 3
    t = {"q": torch.randn(H * D, W), "k": torch.randn(H * D, W), "v": torch.randn(H * V, W), "g": torch.randn(H * V, W),
         "o": torch.eye(H * V)}
    t = {k: v.double() for k, v in t.items()}
    h = torch.randn(T, W, dtype=torch.float64)
    decay = [0.8, 0.95]
    pos = torch.arange(T)
    got = plain.retention(h, t, "", pos, H, D, V, decay, 2, 100.0, 1e-5)
    q = plain.rotate((h @ t["q"].T).reshape(T, H, D), pos, 2, 100.0)
    k = plain.rotate((h @ t["k"].T).reshape(T, H, D), pos, 2, 100.0) / math.sqrt(D)
    v = (h @ t["v"].T).reshape(T, H, V)
    o = torch.zeros(T, H, V, dtype=torch.float64)
    for i in range(T):
        for j in range(i + 1):
            for n in range(H):
                o[i, n] += decay[n] ** (i - j) * (q[i, n] @ k[j, n]) * v[j, n]
    g = h @ t["g"].T
    want = plain.rms(o, 1e-5).reshape(T, H * V) * (g * torch.sigmoid(g))
    assert torch.allclose(got, want, atol=1e-10)


def test_plain_rotation_pairs_and_leaves_the_rest():
    z = torch.arange(12, dtype=torch.float64).reshape(1, 1, 12) + 1
    out = plain.rotate(z, torch.tensor([3]), 4, 10.0)
    assert torch.equal(out[..., 4:], z[..., 4:])
    a0, a1 = 3 * 1.0, 3 * 10.0 ** -0.5
    assert torch.allclose(out[0, 0, :4], torch.tensor([1 * math.cos(a0) - 3 * math.sin(a0), 2 * math.cos(a1) - 4 * math.sin(a1),
                                                        3 * math.cos(a0) + 1 * math.sin(a0), 4 * math.cos(a1) + 2 * math.sin(a1)], dtype=torch.float64))
    assert torch.equal(plain.rotate(z, torch.tensor([0]), 4, 10.0), z)


def test_plain_delta_rule_without_removal_or_decay_is_linear_attention():
    """With a = 0 and w = 1 the state is the plain sum of k v^T; with a = 1 and w = 1 a repeated unit key
    has its old value replaced. Both are forced through the biases."""
    torch.manual_seed(1)
    T, W, H, D = 6, 10, 1, 4
    t = {n: torch.randn(H * D, W, dtype=torch.float64) for n in ("r", "k", "v", "g", "a")}
    t.update({"w1": torch.zeros(2, W, dtype=torch.float64), "w2": torch.zeros(H * D, 2, dtype=torch.float64),
              "w0": torch.full((H * D,), -60.0, dtype=torch.float64), "a.b": torch.full((H * D,), -60.0, dtype=torch.float64),
              "norm": torch.ones(H * D, dtype=torch.float64), "o": torch.eye(H * D, dtype=torch.float64)})
    t["a"] = torch.zeros_like(t["a"])
    h = torch.randn(T, W, dtype=torch.float64)
    got = plain.general_delta(h, t, "", H, D, 1e-5)
    r, k, v = h @ t["r"].T, h @ t["k"].T, h @ t["v"].T
    o = torch.stack([sum((r[i] @ k[j]) * v[j] for j in range(i + 1)) for i in range(T)])
    want = plain.rms(o, 1e-5) * torch.sigmoid(h @ t["g"].T)
    assert torch.allclose(got, want, atol=1e-9)
