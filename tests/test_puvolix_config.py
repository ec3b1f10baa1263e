"""Configuration, specification and tensor list of the Puvolix decoder (no GPU)."""

import copy

import pytest

from quanta_b200.config import ConfigError, PuvolixConfig
from quanta_b200.config.registry import resolve
from tests.plain import puvolix_plain as P


def _layer(mlp):
    return {"type": "parallel", "mlp": mlp, "mixer": {
        "left": {"heads": 4, "kv_heads": 2, "dim": 12, "vdim": 20, "conv": 2, "scale": 0.3,
                 "rot": {"dims": 8, "base": 100.0, "scaling": {"factor": 3.0, "low": 1.0, "high": 3.0, "original": 40}}},
        "right": {"heads": 6, "kv_heads": 3, "dim": 10, "vdim": 14, "conv": 5}}}


RAW = {"architecture": "Puvolix", "vocab": 50, "width": 36, "norm": {"eps": 1e-4, "groups": 3}, "logit_softcap": 9.0,
       "layers": [_layer({"kind": "dense", "ff": 24}), _layer(None),
                  _layer({"kind": "moe", "router": {"experts": 5, "top": 2}, "expert": {"ff": 16, "limit": 1.1},
                          "shared": {"ff": 8, "limit": 0.6}}),
                  _layer({"kind": "moe", "router": {"experts": 3, "top": 3}, "expert": {"ff": 8, "limit": 2.0}, "shared": None})]}


def test_registry_finds_the_architecture_by_its_key():
    assert resolve(RAW).name == "Puvolix"
    assert resolve({"architectures": ["Puvolix"]}).config_cls is PuvolixConfig


def test_fields_and_round_trip():
    cfg = PuvolixConfig.from_dict(RAW)
    assert (cfg.vocab, cfg.width, cfg.norm_eps, cfg.norm_groups, cfg.logit_softcap) == (50, 36, 1e-4, 3, 9.0)
    assert [l.mlp and l.mlp["kind"] for l in cfg.layers] == ["dense", None, "moe", "moe"]
    again = PuvolixConfig.from_dict(cfg.to_dict())
    assert again == cfg and again.to_dict() == cfg.to_dict()
    bare = PuvolixConfig.from_dict({k: v for k, v in RAW.items() if k != "logit_softcap"} | {"norm": {"eps": 1e-5}})
    assert (bare.norm_groups, bare.logit_softcap) == (1, 0.0)


@pytest.mark.parametrize("change,what", [
    (lambda r: r["layers"][0].update(type="attention"), "type"),
    (lambda r: r["layers"][0]["mlp"].update(kind="gated"), "kind"),
    (lambda r: r["layers"][0]["mixer"].pop("right"), "right"),
    (lambda r: r["layers"][0]["mixer"]["left"].pop("scale"), "lacks"),
    (lambda r: r["layers"][0]["mixer"]["left"].update(kv_heads=3), "multiple"),
    (lambda r: r["layers"][0]["mixer"]["right"].update(kv_heads=4), "multiple"),
    (lambda r: r["layers"][0]["mixer"]["right"].update(dim=300), "between"),
    (lambda r: r["layers"][0]["mixer"]["left"]["rot"].update(dims=7), "even"),
    (lambda r: r["layers"][0]["mixer"]["left"]["rot"]["scaling"].pop("low"), "scaling"),
    (lambda r: r["layers"][0]["mixer"]["left"]["rot"]["scaling"].update(high=0.5), "low < high"),
    (lambda r: r["layers"][2]["mlp"]["router"].update(top=6), "top"),
    (lambda r: r["layers"][2]["mlp"]["expert"].update(limit=0.0), "limit"),
    (lambda r: r["layers"][2]["mlp"]["shared"].update(ff=0), "shared"),
    (lambda r: r["norm"].update(groups=5), "groups"),
    (lambda r: r.pop("norm"), "norm"),
])
def test_refusals(change, what):
    raw = copy.deepcopy(RAW)
    change(raw)
    with pytest.raises(ConfigError, match=what):
        PuvolixConfig.from_dict(raw)


def test_the_specification_names_every_tensor_with_its_shape():
    """The tensors the parts ask for are those the plain implementation draws (its list is written from the layout
    of a model folder), and the layers' needs of cache and state follow the configuration."""
    from quanta_b200.engine.model import Model
    from quanta_b200.models.puvolix import build_spec
    cfg = PuvolixConfig.from_dict(RAW)
    model = Model(build_spec(cfg), dtype="float32", device="cpu")
    assert {s.name: tuple(s.shape) for s in model.tensor_specs()} == P.tensor_shapes(RAW)
    assert "l1.norm2" in model.spec.ignorable_names           # a layer without a feed-forward
    need = model.cache_needs()[0]
    assert [(st.name, st.heads, st.width) for st in need.streams] == [("k", 2, 12), ("v", 2, 20)] and need.window is None
    state = model.state_needs()[0]
    assert state["gated_delta_state"][0] == (6, 10, 14)
    assert state["attention_conv_inputs"][0] == (1, 4 * 12 + 2 * 12 + 2 * 20)
    assert state["gated_delta_conv_inputs"][0] == (4, 2 * 3 * 10 + 6 * 14)
    # one tap needs no state
    one = copy.deepcopy(RAW)
    one["layers"][0]["mixer"]["left"]["conv"] = 1
    assert "attention_conv_inputs" not in Model(build_spec(PuvolixConfig.from_dict(one)), dtype="float32", device="cpu").state_needs()[0]


def test_random_weights_mode_writes_a_folder_the_loader_accepts(tmp_path):
    import json

    from quanta_b200.engine.model import write_random_model
    from quanta_b200.weights.safetensors_io import CheckpointFolder
    out = write_random_model(PuvolixConfig.from_dict(RAW), 3, tmp_path / "m")
    assert json.loads((out / "config.json").read_text())["norm"] == {"eps": 1e-4, "groups": 3}
    ckpt = CheckpointFolder(out)
    try:
        assert {n: tuple(ckpt.meta(n)[1]) for n in ckpt.names()} == P.tensor_shapes(RAW)
    finally:
        ckpt.close()
