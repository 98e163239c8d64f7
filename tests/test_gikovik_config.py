"""Gikovik's configuration reader, its description as parts, its tensor names, and the plain
implementation's own pieces on cases done by hand (no GPU)."""
import json
import math
import os

import pytest
import torch

import gikovik_configs as C
from plain import gikovik_plain as P

import poor_mans_mamba_b200.architectures  # noqa: F401  (registration)
from poor_mans_mamba_b200.config import ConfigError, resolve_architecture
from poor_mans_mamba_b200.config.gikovik import GikovikConfig
from poor_mans_mamba_b200.config.registry import open_model_dir
from poor_mans_mamba_b200.engine.model import Model
from poor_mans_mamba_b200.weights.loader import check_tensors
from poor_mans_mamba_b200.weights.safetensors_io import ModelFiles

F64 = torch.float64


@pytest.mark.parametrize("which", ["A", "B", "C", "M"])
def test_every_size_and_constant_is_read(which):
    data = C.config(which)
    cfg = GikovikConfig.from_dict(data)
    assert (cfg.vocab_size, cfg.hidden_size, cfg.norm_eps) == (data["vocab"], data["width"], data["norm"]["eps"])
    assert cfg.side_dim == (data["token_side"]["dim"] if data.get("token_side") else 0)
    if data.get("loop"):
        assert (cfg.loop.start, cfg.loop.stop, cfg.loop.times) == tuple(data["loop"][k] for k in ("start", "stop", "times"))
    else:
        assert cfg.loop is None
    for layer, raw in zip(cfg.layers, data["layers"]):
        m = raw["mixer"]
        assert layer.type == raw["type"]
        assert (layer.mixer.heads, layer.mixer.dim, layer.mixer.vdim, layer.mixer.q_rank, layer.mixer.kv_rank,
                layer.mixer.scale) == tuple(m[k] for k in ("heads", "dim", "vdim", "q_rank", "kv_rank", "scale"))
        if raw["type"] == "latent_attention_2":
            assert (layer.mixer.rot_dim, layer.mixer.rot_dims, layer.mixer.rot_base) == (
                m["rot_dim"], m["rot"]["dims"], m["rot"]["base"])
        else:
            assert layer.mixer.rot_dim == 0 and layer.mixer.rot_dims == 0
        mlp = raw["mlp"]
        if mlp is None:
            assert layer.dense is None and layer.routed is None
        elif mlp["kind"] == "dense":
            assert layer.dense.ff == mlp["ff"] and layer.routed is None
        else:
            r, groups = mlp["router"], mlp["router"].get("groups")
            assert (layer.routed.experts, layer.routed.top, layer.routed.expert_ff) == (r["experts"], r["top"], mlp["expert"]["ff"])
            assert layer.routed.scale == r.get("scale", 1.0)
            assert (layer.routed.groups, layer.routed.keep) == ((groups["count"], groups["keep"]) if groups else (1, 1))
            assert layer.routed.shared_ff == (mlp["shared"]["ff"] if mlp.get("shared") else 0)


def test_the_architecture_is_chosen_by_its_name():
    assert resolve_architecture(C.config("A")).name == "Gikovik"


@pytest.mark.parametrize("path,value,needle", [
    (("layers", 0, "mixer", "heads"), 0, "layers[0].mixer.heads"),
    (("layers", 1, "mixer", "rot", "dims"), 7, "layers[1].mixer.rot.dims"),
    (("layers", 1, "mixer", "rot", "dims"), 14, "layers[1].mixer.rot.dims"),
    (("layers", 1, "mixer", "rot", "base"), 0.0, "layers[1].mixer.rot.base"),
    (("layers", 1, "mlp", "router", "top"), 5, "layers[1].mlp.router.top"),
    (("layers", 1, "mlp", "router", "groups", "count"), 4, "layers[1].mlp.router.groups.count"),
    (("layers", 1, "mlp", "router", "groups", "keep"), 4, "layers[1].mlp.router.groups.keep"),
    (("layers", 0, "mlp", "kind"), "glu", "layers[0].mlp.kind"),
    (("layers", 2, "type"), "attention", "layers[2].type"),
    (("loop", "stop"), 5, "loop"),
    (("loop", "start"), 3, "loop"),
    (("loop", "times"), 0, "loop.times"),
    (("token_side", "dim"), 0, "token_side.dim"),
    (("width",), 0, "width"),
])
def test_errors_name_the_key(path, value, needle):
    data = C.config("A")
    node = data
    for k in path[:-1]:
        node = node[k]
    node[path[-1]] = value
    with pytest.raises(ConfigError) as exc:
        GikovikConfig.from_dict(data)
    assert needle in str(exc.value)


def test_missing_keys_are_refused_and_optional_ones_default():
    data = C.config("A")
    del data["layers"][1]["mixer"]["rot_dim"]
    with pytest.raises(ConfigError, match="rot_dim"):
        GikovikConfig.from_dict(data)
    data = C.config("A")
    del data["layers"][0]["mixer"]["scale"]
    with pytest.raises(ConfigError, match="scale"):
        GikovikConfig.from_dict(data)
    data = C.config("A")
    data["loop"], data["token_side"] = None, None
    del data["layers"][1]["mlp"]["router"]["groups"], data["layers"][1]["mlp"]["router"]["scale"], data["layers"][1]["mlp"]["shared"]
    cfg = GikovikConfig.from_dict(data)
    r = cfg.layers[1].routed
    assert cfg.loop is None and cfg.side_dim == 0 and (r.groups, r.keep, r.scale, r.shared_ff) == (1, 1, 1.0, 0)


@pytest.mark.parametrize("which", ["A", "B", "C", "M"])
def test_every_run_of_a_looped_layer_has_a_cache_of_its_own(which):
    data = C.config(which)
    cfg = GikovikConfig.from_dict(data)
    spec = resolve_architecture(data).model_spec(cfg)
    runs = P.layer_runs(data)
    assert [(c.layer, c.enters) for c in spec.order] == [(i, first) for i, first in runs]
    assert [c.cache_of for c in spec.order] == list(range(len(runs)))
    assert (spec.reentry is not None) == bool(data.get("loop"))
    model = Model(spec)
    states = model.state_specs()
    assert sorted(states) == list(range(len(runs)))
    for run, (i, _) in enumerate(runs):
        m = data["layers"][i]["mixer"]
        need = m["kv_rank"] + m.get("rot_dim", 0)
        by_name = dict(states[run])
        kv = by_name["mix.kv"]
        assert kv.kind == "paged" and kv.width >= need and kv.width % 16 == 0 and kv.width < 2 * max(need, 16)


@pytest.mark.parametrize("which", ["A", "B", "C"])
def test_tensor_names_and_shapes_match_a_model_folder(which, tmp_path):
    d, cfg, weights = C.make_model_dir(which, str(tmp_path))
    arch, typed = open_model_dir(d)
    model = Model(arch.model_spec(typed))
    specs = model.param_specs()
    assert set(specs) == set(weights)
    for name, spec in specs.items():
        assert tuple(spec.shape) == tuple(weights[name].shape), name
    files = ModelFiles(d)
    try:
        assert check_tensors(specs, model.ignored_names(), files, strict=True) == []
    finally:
        files.close()


def test_random_weights_mode_writes_a_loadable_folder(tmp_path):
    from poor_mans_mamba_b200.weights import write_random_model
    d = write_random_model(C.config("C"), seed=5, out_dir=str(tmp_path))
    arch, typed = open_model_dir(d)
    model = Model(arch.model_spec(typed))
    files = ModelFiles(d)
    try:
        assert check_tensors(model.param_specs(), model.ignored_names(), files, strict=True) == []
        w = {k: files.tensor(k).float() for k in files.keys()}
    finally:
        files.close()
    logits = P.forward(json.load(open(os.path.join(d, "config.json"))), w, [1, 2, 3, 4, 5])
    assert logits.shape == (5, 97) and bool(torch.isfinite(logits).all())


# ----------------------------------------------------------------------------- the plain pieces by hand
def test_plain_rotation_turns_neighbouring_pairs():
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0, 6.0]]], dtype=F64)  # one token, one head, 6 entries, 4 of them turn
    out = P.rotate_pairs(x, torch.tensor([3]), 4, 100.0)
    a0, a1 = 3.0, 3.0 * 100.0 ** (-0.5)
    want = [1 * math.cos(a0) - 2 * math.sin(a0), 2 * math.cos(a0) + 1 * math.sin(a0),
            3 * math.cos(a1) - 4 * math.sin(a1), 4 * math.cos(a1) + 3 * math.sin(a1), 5.0, 6.0]
    assert torch.allclose(out[0, 0], torch.tensor(want, dtype=F64))
    assert torch.equal(P.rotate_pairs(x, torch.tensor([0]), 4, 100.0), x)


def test_plain_softmax_sink_counts_once_and_is_not_scaled():
    q = torch.tensor([[[2.0]], [[2.0]]], dtype=F64)
    k = torch.tensor([[[1.0]], [[3.0]]], dtype=F64)
    v = torch.tensor([[[10.0]], [[20.0]]], dtype=F64)
    out = P.causal_softmax_attention(q, k, v, 0.5, torch.tensor([0.25], dtype=F64))
    e1, e3, es = math.exp(1.0), math.exp(3.0), math.exp(0.25)
    assert torch.allclose(out.view(-1), torch.tensor([10 * e1 / (e1 + es), (10 * e1 + 20 * e3) / (e1 + e3 + es)], dtype=F64))
    out = P.causal_softmax_attention(q, k, v, 0.5, None)
    assert torch.allclose(out.view(-1), torch.tensor([10.0, (10 * e1 + 20 * e3) / (e1 + e3)], dtype=F64))


def test_plain_router_groups_corrections_and_weights():
    sg = lambda z: 1.0 / (1.0 + math.exp(-z))
    # six experts in three groups of two; choice scores s + correction; the two best groups are kept
    z = torch.tensor([[0.0, 0.0, 2.0, -2.0, 1.0, 1.0]], dtype=F64)
    corr = torch.tensor([0.0, 0.0, 0.0, 0.0, -0.4, -0.4], dtype=F64)
    # group sums: 1.0;  sg(2) + sg(-2) = 1.0 exactly ... make the first group lose clearly instead
    corr[0] = -0.3
    ids, w = P.route(z, corr, 2, {"count": 3, "keep": 2}, 2.0)
    # groups: {0.2, 0.5} = 0.7; {0.88, 0.12} = 1.0; {0.33, 0.33} = 0.66 -> groups 1 and 0; best two: experts 2 and 1
    assert sorted(ids[0].tolist()) == [1, 2]
    s1, s2 = sg(0.0), sg(2.0)
    got = dict(zip(ids[0].tolist(), w[0].tolist()))
    assert abs(got[1] - 2.0 * s1 / (s1 + s2)) < 1e-12 and abs(got[2] - 2.0 * s2 / (s1 + s2)) < 1e-12
    # an expert outside the kept groups is not chosen although its score is the largest of all
    z = torch.tensor([[3.0, 3.0, 3.5, -9.0, -9.0, -9.0]], dtype=F64)
    ids, _ = P.route(z, None, 2, {"count": 3, "keep": 1}, 1.0)
    assert sorted(ids[0].tolist()) == [0, 1]
    # negative choice scores inside a kept group still beat every expert outside it
    z = torch.tensor([[0.0, 0.0, 0.0, 0.0]], dtype=F64)
    corr = torch.tensor([-5.0, -6.0, -7.0, -100.0], dtype=F64)
    ids, w = P.route(z, corr, 2, {"count": 2, "keep": 1}, 1.0)
    assert sorted(ids[0].tolist()) == [0, 1] and torch.allclose(w, torch.full((1, 2), 0.5, dtype=F64))


def test_plain_experts_token_input_and_loop_order():
    up, down = torch.tensor([[1.0, -1.0]], dtype=F64), torch.tensor([[2.0], [3.0]], dtype=F64)
    y = P.ungated_expert(torch.tensor([[3.0, 1.0], [1.0, 3.0]], dtype=F64), up, down)
    assert y.tolist() == [[8.0, 12.0], [0.0, 0.0]]
    W = {"side.embed": torch.tensor([[9.0, 9.0, 1.0, 2.0]], dtype=F64), "l1.side.gate": torch.tensor([[1.0, 0.0], [0.0, 1.0]], dtype=F64),
         "l1.side.proj": torch.tensor([[1.0, 0.0], [0.0, 1.0]], dtype=F64), "l1.side.norm": torch.tensor([2.0, 3.0], dtype=F64)}
    x = torch.tensor([[0.5, -1.0]], dtype=F64)
    g = P.gelu_tanh(x) * torch.tensor([[1.0, 2.0]], dtype=F64)
    want = x + g / torch.sqrt((g * g).mean() + 0.1) * W["l1.side.norm"]
    assert torch.allclose(P.token_input(x, torch.tensor([0]), W, 1, 2, 0.1), want)
    cfg = {"layers": [None] * 5, "loop": {"start": 1, "stop": 3, "times": 2}}
    assert P.layer_runs(cfg) == [(0, False), (1, True), (2, False), (1, True), (2, False), (3, False), (4, False)]
    assert P.layer_runs({"layers": [None] * 2}) == [(0, False), (1, False)]


def test_plain_forward_depends_on_every_branch():
    """Every tensor of configuration A moves the logits: a branch that the plain forward left out would not."""
    cfg = C.config("A")
    w = C.make_weights(cfg, 3)
    toks = C.sequences(cfg, (12,), seed=1)[0]
    base = P.forward(cfg, w, toks)
    for name in w:
        if ".mlp.e" in name:
            continue  # an expert that no token of this prompt chose changes nothing
        other = dict(w)
        other[name] = w[name] * 1.5 + 0.1
        assert float((P.forward(cfg, other, toks) - base).abs().max()) > 1e-6, name
