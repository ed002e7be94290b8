"""Kemitar without a GPU: the typed configuration (keys, checks, the model in parts, the tensors it
declares), the registry, random model folders, and properties of the plain implementation that the GPU
tests lean on."""
import copy

import pytest
import torch

import plain_kemitar as P
from tiny_configs import TINY, make_model_dir


def typed(raw):
    from flyweight_b200.config.kemitar import KemitarConfig
    return KemitarConfig.from_dict(raw)


def test_the_registry_finds_the_architecture_by_either_key():
    import flyweight_b200.models  # noqa: F401
    from flyweight_b200.config import architecture_name, lookup
    raw = TINY["KA"]
    assert architecture_name(raw) == "Kemitar"
    assert architecture_name({"architectures": ["Kemitar"]}) == "Kemitar"
    assert lookup("Kemitar").config_class.from_dict(raw).to_dict() == typed(raw).to_dict()


@pytest.mark.parametrize("name", ["KA", "KB"])
def test_the_model_in_parts_follows_the_configuration(name):
    raw = TINY[name]
    config = typed(raw)
    assert config.to_dict() == raw
    spec = config.model_spec()
    assert spec.vocab_size == raw["vocab"] and spec.hidden_size == raw["width"]
    assert spec.embedding.params["buckets"] == raw["embedding"]["bigram"]["buckets"]
    assert [entry.cache_of for entry in spec.schedule] == [layer["mixer"].get("kv_from") for layer in raw["layers"]]
    for layer, given in zip(spec.layers, raw["layers"]):
        m = given["mixer"]
        p = layer.parts["mixer"].params
        assert (p["num_heads"], p["dim"], p["rot_dim"], p["vdim"], p["kv_rank"], p["scale"]) == \
            (m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["scale"])
        assert p["position"].params["theta"] == m["rot"]["base"] and p["eps"] == raw["norm"]["eps"]
        assert ("feed_forward" in layer.parts) == (given["mlp"] is not None)
        assert ("dkv" in layer.parts["mixer"].tensors) == ("kv_from" not in m)


def test_declared_tensors_and_their_shapes():
    from flyweight_b200.models import KemitarForCausalLM
    from flyweight_b200.parts import Precision
    raw = TINY["KA"]
    model = KemitarForCausalLM(typed(raw), Precision("float32"), torch.device("cpu"))
    declared = {name: tuple(decl.shape) for name, decl in model.declare().items()}
    W = raw["width"]
    assert declared["embed"] == (raw["vocab"], W) and declared["head"] == (raw["vocab"], W)
    assert declared["bigram"] == (raw["embedding"]["bigram"]["buckets"] + 1, W)
    assert declared["final.norm"] == () and declared["l0.norm1"] == () and declared["l0.shift"] == (W,)
    m = raw["layers"][1]["mixer"]
    assert declared["l1.mix.q"] == (m["heads"] * (m["dim"] + m["rot_dim"]), W)
    assert declared["l1.mix.uk"] == (m["heads"] * m["dim"], m["kv_rank"])
    assert declared["l1.mix.uv"] == (m["heads"] * m["vdim"], m["kv_rank"])
    assert declared["l1.mix.o"] == (W, m["heads"] * m["vdim"]) and declared["l1.mix.sink"] == (m["heads"],)
    assert "l1.mix.dkv" not in declared and "l1.norm2" not in declared and "l1.mlp.gate" not in declared
    assert declared["l0.mix.dkv"] == (40 + 8, W) and declared["l0.mix.dkv.norm"] == (40,)
    assert declared["l3.mlp.down"] == (W, 96)
    # what each schedule position keeps: pages for a layer with a projection of its own, and the
    # token shift's row for every layer; one more entry for the embedding's last token
    specs = model.state_specs()
    assert len(specs) == len(raw["layers"]) + 1
    assert model.cache_sources() == [None, 0, 0, None]


@pytest.mark.parametrize("damage,message", [
    (lambda c: c["layers"][1]["mixer"].update(kv_from=1), "no earlier layer"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "no earlier layer"),
    (lambda c: c["layers"][1]["mixer"].update(kv_rank=48), "must agree"),
    (lambda c: c["layers"][0].update(type="ring"), "unknown type"),
    (lambda c: c["layers"][0]["mlp"].update(kind="experts"), "unknown feed-forward"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "missing scale"),
    (lambda c: c.pop("width"), "missing width"),
    (lambda c: c["embedding"]["bigram"].update(buckets=0), "buckets"),
])
def test_a_wrong_configuration_is_refused_with_its_reason(damage, message):
    from flyweight_b200.config.lfm2 import ConfigError
    raw = copy.deepcopy(TINY["KA"])
    damage(raw)
    with pytest.raises(ConfigError, match=message):
        typed(raw)


def test_random_model_folders_load_in_the_plain_implementation(tmp_path):
    path = make_model_dir(tmp_path / "m", TINY["KB"], seed=1, preset="unit", dtype=torch.bfloat16)
    cfg, w = P.load_model_dir(path)
    assert cfg == TINY["KB"]
    logits = P.forward(cfg, w, [1, 2, 3, 4])
    assert logits.shape == (4, TINY["KB"]["vocab"]) and bool(torch.isfinite(logits).all())


def test_the_plain_implementation_is_causal_and_keeps_its_state_in_the_prefix(tmp_path):
    """Logits at a place depend on the tokens up to it only, and on all of them: the one before (pair
    table, token shift) and the first."""
    path = make_model_dir(tmp_path / "m", TINY["KA"], seed=2, preset="unit", dtype=torch.float32)
    cfg, w = P.load_model_dir(path)
    tokens = [5, 9, 200, 17, 3, 88, 41]
    full = P.forward(cfg, w, tokens)
    assert torch.allclose(P.forward(cfg, w, tokens[:4]), full[:4], atol=1e-12)
    changed = P.forward(cfg, w, [6] + tokens[1:])
    assert float((changed[-1] - full[-1]).abs().max()) > 1e-6
    assert P.hashed_pair_rows([4, 4, 7], 97, 31, 5) == [97, (4 * 31 + 4 * 5) % 97, (4 * 31 + 7 * 5) % 97]


def test_the_sink_takes_weight_from_the_keys():
    scores = torch.zeros(1, 2, 2, dtype=torch.float64)
    weights = P.softmax_with_sink(scores, torch.tensor([0.0], dtype=torch.float64))
    assert torch.allclose(weights[0], torch.tensor([[0.5, 0.0], [1 / 3, 1 / 3]], dtype=torch.float64))


def test_tensors_of_a_sublayer_that_a_layer_leaves_out_are_passed_over():
    """A checkpoint may carry the output norm of a feed-forward that a layer does not have, or the latent
    projection of a layer that reads another's rows; anything else that is not declared is refused."""
    from flyweight_b200.models import KemitarForCausalLM
    from flyweight_b200.parts import Precision
    from flyweight_b200.weights import WeightError, bind, random_tensors
    model = KemitarForCausalLM(typed(TINY["KA"]), Precision("float32"), torch.device("cpu"))
    declared = model.declare()
    stored = dict(random_tensors(declared, 1, "unit", torch.float32, "cpu"))
    stored["l1.norm2"] = torch.ones(())
    stored["l1.mix.dkv"] = torch.zeros(48, 80)
    assert set(bind(declared, stored, model.spec.unused_tensors)) == set(declared)
    stored["l0.norm3"] = torch.ones(())
    with pytest.raises(WeightError, match="l0.norm3"):
        bind(declared, stored, model.spec.unused_tensors)


def test_a_layer_that_reads_anothers_rows_may_leave_their_sizes_unsaid():
    raw = copy.deepcopy(TINY["KA"])
    for key in ("kv_rank", "rot_dim", "rot"):
        raw["layers"][1]["mixer"].pop(key)
    assert typed(raw).to_dict() == TINY["KA"]
