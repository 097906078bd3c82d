"""The Lomopel configuration: config.json's keys in, the same keys out; optional keys; what is refused;
the manifest that follows from it; random model folders (CPU only)."""
import json
import os

import pytest
import torch

from vllm_oxide_b200 import models  # noqa: F401  (registers the architectures)
from vllm_oxide_b200.config import LomopelConfig, architecture_for
from vllm_oxide_b200.errors import ConfigError, WeightsError
from vllm_oxide_b200.models import lomopel_manifest


def _dict():
    return {
        "architecture": "Lomopel", "vocab": 90, "width": 40, "embedding": {"scale": 2.5}, "norm": {"eps": 1e-6},
        "layers": [
            {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 12, "vdim": 20, "scale": 0.3,
                                            "q_temp": {"coef": 0.25, "every": 32}, "v_mix": True}, "mlp": {"kind": "dense", "ff": 64}},
            {"type": "parallel", "mixer": {
                "left": {"heads": 2, "kv_heads": 1, "dim": 16, "vdim": 8, "scale": 0.25, "mask": {"size": 11}, "rot": {"dims": 8, "base": 300.0}},
                "right": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "conv": 3, "decay_rank": 5, "gate_rank": 6},
                "left_scale": 1.5, "right_scale": 0.5}, "mlp": None},
            {"type": "attention", "mixer": {"heads": 2, "kv_heads": 2, "dim": 8, "vdim": 20, "scale": 0.5, "v_mix": True}, "mlp": None},
        ]}


def test_keys_in_keys_out_and_the_registry():
    d = _dict()
    arch = architecture_for(d)
    assert arch.name == "Lomopel"
    cfg = arch.config_cls.from_dict(d)
    assert isinstance(cfg, LomopelConfig)
    assert cfg.to_dict() == d
    assert LomopelConfig.from_dict(cfg.to_dict()) == cfg
    a, par = cfg.layers[0].attention, cfg.layers[1]
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.q_temp, a.v_mix, a.window, a.rot_dims) == (4, 2, 12, 20, 0.3, (0.25, 32), True, 0, 0)
    assert (par.left.window, par.left.rot_dims, par.left.rot_base, par.right.conv, par.left_scale, par.right_scale, par.ff) == (11, 8, 300.0, 3, 1.5, 0.5, 0)
    assert cfg.embedding_scale == 2.5 and cfg.norm_eps == 1e-6 and cfg.first_mixing_layer() == 0
    assert cfg.param_count() == sum(torch.Size(s.shape).numel() for s in lomopel_manifest(cfg).values())


def test_optional_keys():
    d = _dict()
    del d["embedding"]
    del d["layers"][0]["mixer"]["q_temp"]
    del d["layers"][0]["mixer"]["v_mix"]
    del d["layers"][1]["mixer"]["left"]["rot"]
    del d["layers"][1]["mixer"]["left"]["mask"]
    del d["layers"][1]["mixer"]["right"]["decay_rank"]
    cfg = LomopelConfig.from_dict(d)
    assert cfg.embedding_scale == 1.0 and cfg.layers[0].attention.q_temp is None and not cfg.layers[0].attention.v_mix
    assert cfg.layers[1].left.rot_dims == 0 and cfg.layers[1].left.window == 0 and cfg.layers[1].right.decay_rank is None
    m = lomopel_manifest(cfg)
    assert m["l1.mix.right.a1"].shape == (-1, 40) and m["l1.mix.right.a2"].shape == (32, -1)      # taken from the stored tensor
    assert m["l0.mix.vmix"].optional and not m["l2.mix.vmix"].optional


@pytest.mark.parametrize("path,value", [
    (("layers", 0, "type"), "sliding"), (("layers", 0, "mixer", "kv_heads"), 3), (("layers", 1, "mixer", "left", "rot", "dims"), 7),
    (("layers", 1, "mixer", "left", "rot", "dims"), 18), (("layers", 1, "mixer", "left", "mask", "size"), 0),
    (("layers", 1, "mixer", "right", "conv"), 0), (("layers", 0, "mixer", "q_temp", "every"), 0), (("layers", 0, "mlp", "kind"), "moe"),
    (("layers", 2, "mixer", "vdim"), 16), (("layers", 0, "mixer", "scale"), "big"), (("layers", 1, "mixer", "left", "v_mix"), True),
    (("norm",), None), (("layers",), [])])
def test_what_is_refused(path, value):
    d = _dict()
    at = d
    for k in path[:-1]:
        at = at[k]
    at[path[-1]] = value
    with pytest.raises(ConfigError):
        LomopelConfig.from_dict(d)


def test_manifest_names_and_shapes():
    m = lomopel_manifest(LomopelConfig.from_dict(_dict()))
    assert m["embed"].shape == (90, 40) and m["head"].shape == (90, 40) and m["final.norm"].shape == (40,)
    assert m["l0.mix.q"].shape == (48, 40) and m["l0.mix.q.b"].shape == (48,) and m["l0.mix.k"].shape == (24, 40)
    assert m["l0.mix.v"].shape == (40, 40) and m["l0.mix.o"].shape == (40, 80) and m["l0.mix.o.b"].shape == (40,)
    assert m["l0.mix.sink"].shape == (4,) and m["l0.mix.vmix"].shape == ()
    assert m["l1.mix.left.g"].shape == (16, 40) and m["l1.mix.left.o"].shape == (40, 16) and m["l1.mix.left.k"].shape == (16, 40)
    assert m["l1.mix.right.q"].shape == (16, 40) and m["l1.mix.right.q.conv"].shape == (16, 3) and m["l1.mix.right.v.conv"].shape == (48, 3)
    assert m["l1.mix.right.b"].shape == (4, 40) and m["l1.mix.right.A_log"].shape == (4,) and m["l1.mix.right.norm"].shape == (12,)
    assert m["l1.mix.right.a1"].shape == (5, 40) and m["l1.mix.right.a2"].shape == (32, 5) and m["l1.mix.right.dt_bias"].shape == (32,)
    assert m["l1.mix.right.g1"].shape == (6, 40) and m["l1.mix.right.g2"].shape == (48, 6) and m["l1.mix.right.o"].shape == (40, 48)
    assert m["l0.mlp.gate"].shape == (64, 40) and m["l0.ls2"].shape == (40,) and not m["l0.norm2"].optional
    assert m["l1.norm2"].optional and m["l1.ls2"].optional and "l1.mlp.gate" not in m and m["l1.ls1"].shape == (40,)


def test_a_random_model_folder_reads_back_and_a_wrong_one_is_refused(tmp_path):
    from vllm_oxide_b200.weights import load_safetensors_weights, write_random_model
    from vllm_oxide_b200.weights.safetensors_io import SafetensorsFile, write_safetensors
    cfg = LomopelConfig.from_dict(_dict())
    d = str(tmp_path / "m")
    write_random_model(d, cfg, seed=3, std=0.1)
    assert json.load(open(os.path.join(d, "config.json"))) == _dict()
    manifest = lomopel_manifest(cfg)
    ws = load_safetensors_weights(d, manifest)
    assert not ws.has("l1.norm2") and ws.take("l0.mix.vmix").shape == () and ws.take("l2.mix.vmix").shape == ()
    # a checkpoint may hold a tensor the model does not use where the manifest says so, but nothing else
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    tensors["l1.ls2"] = torch.zeros(40, dtype=torch.bfloat16)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    assert load_safetensors_weights(d, manifest).has("l1.ls2")
    tensors["l1.mix.left.sink"] = torch.zeros(2, dtype=torch.bfloat16)
    del tensors["l0.mix.sink"]
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    with pytest.raises(WeightsError) as e:
        load_safetensors_weights(d, manifest)
    assert e.value.missing == ["l0.mix.sink"] and e.value.unexpected == ["l1.mix.left.sink"]
