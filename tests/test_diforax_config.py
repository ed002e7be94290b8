"""Diforax without a GPU: the typed configuration (keys, checks, the model in parts, the tensors it
declares), the registry, random model folders, and properties of the plain implementation that the GPU
tests lean on."""
import copy

import pytest
import torch

import plain_diforax as P
from tiny_configs import TINY, make_model_dir

F64 = torch.float64


def typed(raw):
    from flyweight_b200.config.diforax import DiforaxConfig
    return DiforaxConfig.from_dict(raw)


def test_the_registry_finds_the_architecture_by_either_key():
    import flyweight_b200.models  # noqa: F401
    from flyweight_b200.config import architecture_name, lookup
    raw = TINY["DA"]
    assert architecture_name(raw) == "Diforax"
    assert architecture_name({"architectures": ["Diforax"]}) == "Diforax"
    assert lookup("Diforax").config_class.from_dict(raw).to_dict() == typed(raw).to_dict()


@pytest.mark.parametrize("name", ["DA", "DB", "DC"])
def test_the_model_in_parts_follows_the_configuration(name):
    raw = TINY[name]
    config = typed(raw)
    assert config.to_dict() == raw
    spec = config.model_spec()
    assert spec.vocab_size == raw["vocab"] and spec.hidden_size == raw["width"] and spec.head_tensor == "head"
    assert [entry.cache_of for entry in spec.schedule] == [layer["mixer"].get("kv_from") for layer in raw["layers"]]
    for layer, given in zip(spec.layers, raw["layers"]):
        assert layer.arrangement == "sandwich_residual"
        m, p = given["mixer"], layer.parts["mixer"].params
        if given["type"] == "attention":
            assert layer.parts["mixer"].kind == "gqa_attention"
            assert (p["num_heads"], p["num_kv_heads"], p["head_dim"], p["value_dim"], p["scale"], p["chunk"]) == \
                (m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["scale"], m["mask"]["size"])
            assert p["qk_unit_rms_eps"] == raw["norm"]["eps"] and p["qk_norm_eps"] is None
            assert p["position"].params == {"theta": m["rot"]["base"], "rotary_dim": m["rot"]["dims"],
                                            "pairing": "half_split"}
            assert ("k" in layer.parts["mixer"].tensors) == ("kv_from" not in m)
        else:
            assert layer.parts["mixer"].kind == "gated_delta_rule"
            assert (p["num_heads"], p["num_kv_heads"], p["dim"], p["vdim"], p["taps"], p["eps"]) == \
                (m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"], raw["norm"]["eps"])
        mlp = given["mlp"]
        assert ("feed_forward" in layer.parts) == (mlp is not None) == ("ffn_out_norm" in layer.parts)
        if mlp is not None and mlp["kind"] == "dense":
            assert layer.parts["feed_forward"].params == {"hidden_size": raw["width"], "ffn_dim": mlp["ff"],
                                                          "activation": "gelu_tanh"}
        elif mlp is not None:
            f, r = layer.parts["feed_forward"].params, mlp["router"]
            groups = r.get("groups", {"count": 1, "keep": 1})
            assert (f["experts"], f["identity"], f["top"], f["groups"], f["keep_groups"], f["ffn_dim"], f["activation"]) \
                == (r["experts"], r["identity"], r["top"], groups["count"], groups["keep"], mlp["expert"]["ff"], "silu")


def test_declared_tensors_and_their_shapes():
    from flyweight_b200.models import DiforaxForCausalLM
    from flyweight_b200.parts import Precision
    raw = TINY["DA"]
    model = DiforaxForCausalLM(typed(raw), Precision("float32"), torch.device("cpu"))
    declared = {name: tuple(decl.shape) for name, decl in model.declare().items()}
    W = raw["width"]
    assert declared["embed"] == (raw["vocab"], W) and declared["head"] == (raw["vocab"], W)
    assert declared["final.norm"] == (W,)
    for name in ("norm1", "norm1b", "norm2", "norm2b"):
        assert declared[f"l0.{name}"] == (W,)
    assert "l2.norm2" not in declared and "l2.norm2b" not in declared and "l2.mlp.gate" not in declared
    d = raw["layers"][0]["mixer"]
    assert declared["l0.mix.q"] == declared["l0.mix.k"] == (d["kv_heads"] * d["dim"], W)
    assert declared["l0.mix.v"] == declared["l0.mix.g"] == (d["heads"] * d["vdim"], W)
    assert declared["l0.mix.q.conv"] == (d["kv_heads"] * d["dim"], d["conv"])
    assert declared["l0.mix.v.conv"] == (d["heads"] * d["vdim"], d["conv"])
    assert declared["l0.mix.b"] == declared["l0.mix.a"] == (d["heads"], W)
    assert declared["l0.mix.A_log"] == declared["l0.mix.dt_bias"] == (d["heads"],)
    assert declared["l0.mix.norm"] == (d["vdim"],) and declared["l0.mix.o"] == (W, d["heads"] * d["vdim"])
    r = raw["layers"][0]["mlp"]
    outputs = r["router"]["experts"] + r["router"]["identity"]
    assert declared["l0.mlp.router"] == (outputs, W) and declared["l0.mlp.correction"] == (outputs,)
    assert declared[f"l0.mlp.e{r['router']['experts'] - 1}.down"] == (W, r["expert"]["ff"])
    assert f"l0.mlp.e{r['router']['experts']}.gate" not in declared          # identity experts have no tensors
    a = raw["layers"][1]["mixer"]
    assert declared["l1.mix.q"] == (a["heads"] * a["dim"], W) and declared["l1.mix.k"] == (a["kv_heads"] * a["dim"], W)
    assert declared["l1.mix.v"] == (a["kv_heads"] * a["vdim"], W) and declared["l1.mix.o"] == (W, a["heads"] * a["vdim"])
    assert "l2.mix.k" not in declared and "l2.mix.v" not in declared and "l2.mix.q" in declared
    assert declared["l1.mlp.gate"] == (raw["layers"][1]["mlp"]["ff"], W)
    # the state one request keeps in a delta layer: the matrices and the convolution's last inputs
    state = model.layers[0].state_spec()
    entries = d["heads"] * d["dim"] * d["vdim"] + (2 * d["kv_heads"] * d["dim"] + d["heads"] * d["vdim"]) * (d["conv"] - 1)
    assert state.shape == (-(-entries // 4) * 4,)                     # slots start on 16-byte borders
    pages = model.layers[1].state_spec()
    assert (pages.n_kv_heads, pages.head_dim, pages.window) == (a["kv_heads"], max(a["dim"], a["vdim"]), 0)
    assert model.layers[2].state_spec() is None


def _broken(edit):
    raw = copy.deepcopy(TINY["DA"])
    edit(raw)
    return raw


@pytest.mark.parametrize("edit,message", [
    (lambda r: r.pop("width"), "missing width"),
    (lambda r: r["layers"][0].update(type="mamba"), "unknown type"),
    (lambda r: r["layers"][1]["mixer"].pop("scale"), "missing scale"),
    (lambda r: r["layers"][1]["mixer"].update(heads=7), "multiple of kv_heads"),
    (lambda r: r["layers"][1]["mixer"]["rot"].update(dims=34), "rot.dims"),
    (lambda r: r["layers"][1]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda r: r["layers"][2]["mixer"].update(kv_from=2), "no earlier attention layer"),
    (lambda r: r["layers"][2]["mixer"].update(kv_from=0), "no earlier attention layer"),
    (lambda r: r["layers"][2]["mixer"].update(dim=16), "must agree"),
    (lambda r: r["layers"][0]["mixer"].pop("conv"), "missing conv"),
    (lambda r: r["layers"][0]["mlp"]["router"]["groups"].update(count=3), "equal groups"),
    (lambda r: r["layers"][0]["mlp"]["router"].update(top=5), "top does not fit"),
    (lambda r: r["layers"][1]["mlp"].update(kind="sparse"), "unknown feed-forward"),
    (lambda r: r["layers"][1]["mixer"]["mask"].update(size=0), "size must be positive"),
])
def test_a_configuration_that_does_not_fit_is_refused_with_its_reason(edit, message):
    from flyweight_b200.config import ConfigError
    with pytest.raises(ConfigError, match=message):
        typed(_broken(edit))


def test_a_layer_that_reads_anothers_keys_may_leave_their_sizes_unsaid():
    raw = copy.deepcopy(TINY["DA"])
    for key in ("kv_heads", "dim", "vdim", "rot"):
        raw["layers"][2]["mixer"].pop(key)
    assert typed(raw).layers[2]["mixer"]["rot"] == TINY["DA"]["layers"][1]["mixer"]["rot"]
    assert typed(raw).model_spec().layers[2].parts["mixer"].params["head_dim"] == 32


def test_a_random_model_folder_loads_and_runs_in_the_plain_implementation(tmp_path):
    make_model_dir(tmp_path / "m", TINY["DB"], seed=1, preset="unit", dtype=torch.bfloat16)
    config, weights = P.load_model_dir(tmp_path / "m")
    assert config == TINY["DB"]
    logits = P.forward(config, weights, [1, 2, 3, 4, 5])
    assert logits.shape == (5, TINY["DB"]["vocab"]) and torch.isfinite(logits).all()


# ------------------------------------------------------------------ the plain implementation itself
def test_plain_a_query_sees_its_own_chunk_only():
    seen = P.chunk_visible(torch.arange(10), torch.arange(10), 4)
    assert seen[3].tolist() == [True] * 4 + [False] * 6
    assert seen[4].tolist() == [False] * 4 + [True] + [False] * 5
    assert seen[9].tolist() == [False] * 8 + [True, True]


def test_plain_delta_rule_cut_anywhere_gives_the_same():
    g = torch.Generator().manual_seed(1)
    H, G, d, e, L, W, T = 4, 2, 8, 6, 3, 32, 40
    w = {"q": torch.randn(G * d, W, generator=g, dtype=F64), "k": torch.randn(G * d, W, generator=g, dtype=F64),
         "v": torch.randn(H * e, W, generator=g, dtype=F64), "g": torch.randn(H * e, W, generator=g, dtype=F64),
         "b": torch.randn(H, W, generator=g, dtype=F64), "a": torch.randn(H, W, generator=g, dtype=F64),
         "o": torch.randn(W, H * e, generator=g, dtype=F64), "A_log": torch.randn(H, generator=g, dtype=F64),
         "dt_bias": torch.randn(H, generator=g, dtype=F64), "norm": torch.rand(e, generator=g, dtype=F64) + 0.5,
         "q.conv": torch.randn(G * d, L, generator=g, dtype=F64), "k.conv": torch.randn(G * d, L, generator=g, dtype=F64),
         "v.conv": torch.randn(H * e, L, generator=g, dtype=F64)}
    h = torch.randn(T, W, generator=g, dtype=F64) * 0.3
    whole, _ = P.delta_mixer(h, w, H, G, d, e, 1e-6)
    state, parts = None, []
    for a, b in ((0, 1), (1, 3), (3, 20), (20, 21), (21, 40)):
        out, state = P.delta_mixer(h[a:b], w, H, G, d, e, 1e-6, state)
        parts.append(out)
    assert torch.allclose(torch.cat(parts), whole, rtol=0, atol=1e-12)
    # a change of a late token leaves the early outputs alone, a change of an early one reaches the late
    h2 = h.clone()
    h2[30] += 1
    again, _ = P.delta_mixer(h2, w, H, G, d, e, 1e-6)
    assert torch.equal(again[:30], whole[:30]) and not torch.allclose(again[30:], whole[30:])
    h2 = h.clone()
    h2[2] += 1
    assert not torch.allclose(P.delta_mixer(h2, w, H, G, d, e, 1e-6)[0][39], whole[39])


def test_plain_router_groups_corrections_and_identity_experts():
    h = torch.eye(4, dtype=F64)[:1] * 0                                   # all scores equal: 1/6 each
    router = torch.zeros(6, 4, dtype=F64)
    correction = torch.tensor([0.0, 0.5, -0.9, -0.8, 0.4, 0.3], dtype=F64)
    ids, weights = P.route(h, router, correction, 3, 2, 3)
    # groups (0,1) (2,3) (4,5): the middle one is out although its members are not the smallest of all
    assert sorted(ids[0].tolist()) == [1, 4, 5] and torch.allclose(weights, torch.full((1, 3), 1 / 6, dtype=F64))
    ids, _ = P.route(h, router, torch.tensor([-5.0, -4.0, -9.0, -8.0, -7.0, -6.0], dtype=F64), 3, 1, 2)
    assert sorted(ids[0].tolist()) == [0, 1]                              # negative choice values still win their group
    x = torch.randn(3, 4, generator=torch.Generator().manual_seed(0), dtype=F64)
    out = P.moe(x, torch.zeros(2, 4, dtype=F64), torch.zeros(2, dtype=F64), [], 2, 1, 1, 2)
    assert torch.allclose(out, x)                                         # two identity experts at 1/2 each
