"""Sorovik's configuration reader, its description as parts, its tensor names, what the cache manager keeps
for it, and the plain implementation's own pieces on cases done by hand (no GPU)."""
import json
import math
import os

import pytest
import torch

import sorovik_configs as C
from plain import sorovik_plain as P

import poor_mans_mamba_b200.architectures  # noqa: F401  (registration)
from poor_mans_mamba_b200.cache import CacheManager
from poor_mans_mamba_b200.config import ConfigError, resolve_architecture
from poor_mans_mamba_b200.config.registry import open_model_dir
from poor_mans_mamba_b200.config.sorovik import SorovikConfig
from poor_mans_mamba_b200.engine.model import Model
from poor_mans_mamba_b200.parts.base import StateSpec
from poor_mans_mamba_b200.weights.loader import check_tensors
from poor_mans_mamba_b200.weights.safetensors_io import ModelFiles

F64 = torch.float64


@pytest.mark.parametrize("which", ["A", "B", "C", "M"])
def test_every_size_and_constant_is_read(which):
    data = C.config(which)
    cfg = SorovikConfig.from_dict(data)
    assert (cfg.vocab_size, cfg.hidden_size, cfg.norm_eps) == (data["vocab"], data["width"], data["norm"]["eps"])
    for layer, raw in zip(cfg.layers, data["layers"]):
        m = raw["mixer"]
        assert layer.type == raw["type"]
        mask, rot = m.get("mask") or {}, m.get("rot") or {"dims": 0, "base": 1.0}
        if raw["type"] == "latent_attention":
            x = layer.latent
            assert layer.attention is None
            assert (x.heads, x.dim, x.rot_dim, x.vdim, x.kv_rank, x.scale) == tuple(
                m[k] for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale"))
            assert (x.rot_dims, x.rot_base, x.window, x.kv_from) == (rot["dims"], rot["base"], mask.get("size", 0), m.get("kv_from"))
        else:
            x = layer.attention
            assert layer.latent is None
            assert (x.heads, x.kv_heads, x.dim, x.scale, x.conv) == (m["heads"], m["kv_heads"], m["dim"], m["scale"], m.get("conv", 0))
            assert (x.rot_dims, x.window, x.keep_first) == (rot["dims"], mask.get("size", 0), mask.get("keep_first", 0))
            if rot["dims"]:
                assert x.rot_base == rot["base"]
        mlp = raw["mlp"]
        if mlp is None:
            assert layer.dense is None and layer.routed is None
        elif mlp["kind"] == "dense":
            assert layer.dense.ff == mlp["ff"] and layer.routed is None
        else:
            r, groups = mlp["router"], mlp["router"].get("groups")
            assert (layer.routed.experts, layer.routed.top, layer.routed.expert_ff) == (r["experts"], r["top"], mlp["expert"]["ff"])
            assert (layer.routed.groups, layer.routed.keep) == ((groups["count"], groups["keep"]) if groups else (1, 1))


def test_the_architecture_is_chosen_by_its_name():
    assert resolve_architecture(C.config("A")).name == "Sorovik"


@pytest.mark.parametrize("path,value,needle", [
    (("layers", 0, "mixer", "heads"), 0, "layers[0].mixer.heads"),
    (("layers", 0, "mixer", "kv_heads"), 3, "layers[0].mixer.kv_heads"),
    (("layers", 0, "mixer", "vdim"), 16, "layers[0].mixer.vdim"),
    (("layers", 0, "mixer", "rot", "dims"), 7, "layers[0].mixer.rot.dims"),
    (("layers", 0, "mixer", "rot", "dims"), 26, "layers[0].mixer.rot.dims"),
    (("layers", 1, "mixer", "rot", "dims"), 14, "layers[1].mixer.rot.dims"),
    (("layers", 1, "mixer", "rot", "base"), 0.0, "layers[1].mixer.rot.base"),
    (("layers", 0, "mixer", "mask", "size"), -1, "layers[0].mixer.mask.size"),
    (("layers", 0, "mixer", "mask", "keep_first"), -2, "layers[0].mixer.mask.keep_first"),
    (("layers", 2, "mixer", "kv_from"), 2, "layers[2].mixer.kv_from"),
    (("layers", 2, "mixer", "kv_from"), 0, "layers[2].mixer.kv_from"),
    (("layers", 4, "mixer", "kv_from"), 2, "layers[4].mixer.kv_from"),
    (("layers", 4, "mixer", "kv_from"), 3, "layers[4].mixer.kv_from"),
    (("layers", 2, "mixer", "kv_rank"), 24, "layers[2].mixer.kv_from"),
    (("layers", 0, "mlp", "router", "top"), 5, "layers[0].mlp.router.top"),
    (("layers", 0, "mlp", "router", "groups", "count"), 4, "layers[0].mlp.router.groups.count"),
    (("layers", 0, "mlp", "router", "groups", "keep"), 4, "layers[0].mlp.router.groups.keep"),
    (("layers", 1, "mlp", "kind"), "glu", "layers[1].mlp.kind"),
    (("layers", 2, "type"), "latent_attention_2", "layers[2].type"),
    (("width",), 0, "width"),
])
def test_errors_name_the_key(path, value, needle):
    data = C.config("A")
    node = data
    for k in path[:-1]:
        node = node[k]
    node[path[-1]] = value
    with pytest.raises(ConfigError) as exc:
        SorovikConfig.from_dict(data)
    assert needle in str(exc.value)


def test_missing_keys_are_refused_and_optional_ones_default():
    for layer, key in ((0, "kv_heads"), (0, "scale"), (1, "kv_rank"), (1, "scale"), (1, "vdim")):
        data = C.config("A")
        del data["layers"][layer]["mixer"][key]
        with pytest.raises(ConfigError, match=key):
            SorovikConfig.from_dict(data)
    data = C.config("A")
    a = data["layers"][0]["mixer"]
    del a["conv"], a["rot"], a["mask"], a["vdim"], data["layers"][0]["mlp"]["router"]["groups"], data["layers"][1]["mixer"]["mask"]
    data["layers"][0]["mlp"]["router"]["top"] = 6
    cfg = SorovikConfig.from_dict(data)
    x, r = cfg.layers[0].attention, cfg.layers[0].routed
    assert (x.conv, x.rot_dims, x.window, x.keep_first, r.groups, r.keep, r.top) == (0, 0, 0, 0, 1, 1, 6)
    assert cfg.layers[1].latent.window == 0


@pytest.mark.parametrize("which", ["A", "B", "C", "M"])
def test_layers_that_read_another_layers_rows_run_on_its_cache(which):
    """A layer with kv_from declares no state and runs on the owner's cache; the owner's rows are kept for the
    widest window of all their readers (for ever if one of them has none)."""
    data = C.config(which)
    cfg = SorovikConfig.from_dict(data)
    spec = resolve_architecture(data).model_spec(cfg)
    assert [c.layer for c in spec.order] == list(range(len(data["layers"])))
    model = Model(spec)
    states = model.state_specs()
    for i, raw in enumerate(data["layers"]):
        m = raw["mixer"]
        src = m.get("kv_from")
        assert spec.order[i].cache_of == (i if src is None else src)
        if src is not None:
            assert model.layers[i].state_specs() == []
            continue
        by_name = dict(states[i])
        kv = by_name["mix.kv"]
        if raw["type"] == "latent_attention":
            readers = [l["mixer"] for j, l in enumerate(data["layers"]) if j == i or l["mixer"].get("kv_from") == i]
            sizes = [(r.get("mask") or {}).get("size", 0) for r in readers]
            assert kv.window == (0 if 0 in sizes else max(sizes)) and kv.keep_first == 0
            need = m["kv_rank"] + m["rot_dim"]
            assert kv.width >= need and kv.width % 16 == 0 and kv.width < 2 * max(need, 16)
            assert "mix.conv" not in by_name
        else:
            mask = m.get("mask") or {}
            assert (kv.window, kv.keep_first) == (mask.get("size", 0), mask.get("keep_first", 0) if mask.get("size", 0) else 0)
            assert kv.width == m["kv_heads"] * ((m["dim"] + 15) // 16 * 16)
            if m.get("conv"):
                assert by_name["mix.conv"].shape == (m["conv"] - 1, (m["heads"] + m["kv_heads"]) * m["dim"])
            else:
                assert "mix.conv" not in by_name


def test_the_first_pages_stay_where_first_tokens_are_kept():
    """Pages of 4 tokens, a window of 6 with 5 first tokens kept beside a plain window of 6: the plain group gives
    back every page the window has passed, the other all but the two pages that hold the first five tokens."""
    specs = {0: [("a.kv", StateSpec.paged("kv", 2, 16, window=6, keep_first=5))],
             1: [("b.kv", StateSpec.paged("kv", 2, 16, window=6))]}
    cache = CacheManager(specs, page_size=4, num_pages=12, num_slots=2, dtype=torch.float32, device="cpu")
    assert len(cache.groups) == 2
    kept = next(g for g in cache.groups.values() if g.keep_first == 5)
    plain = next(g for g in cache.groups.values() if g.keep_first == 0)
    assert kept.kept_blocks() == 2 and plain.kept_blocks() == 0
    cache.admit("r")
    cache.grow("r", 9)
    cache.advance("r", 9)         # next position 9 reads 4..9: block 0 is behind both windows
    assert [p >= 0 for p in kept.tables["r"]] == [True, True, True]
    assert [p >= 0 for p in plain.tables["r"]] == [False, True, True]
    for n in range(10, 31):
        cache.grow("r", n)
        cache.advance("r", 1)
    # next position 30 reads 25..30: blocks 6 and 7; the kept group also holds blocks 0 and 1
    assert [p >= 0 for p in kept.tables["r"]] == [True, True, False, False, False, False, True, True]
    assert [p >= 0 for p in plain.tables["r"]] == [False, False, False, False, False, False, True, True]
    cache.check()
    cache.release("r")
    assert kept.pool.n_free == 12 and plain.pool.n_free == 12
    # a window without kept tokens and one with them never share pages, whatever else is equal
    assert StateSpec.paged("kv", 2, 16, window=0, keep_first=5).keep_first == 0


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
def test_plain_rotation_turns_halves():
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0, 6.0]]], dtype=F64)  # one token, one head, 6 entries, 4 of them turn
    out = P.rotate_halves(x, torch.tensor([3]), 4, 100.0)
    a0, a1 = 3.0, 3.0 * 100.0 ** (-0.5)
    want = [1 * math.cos(a0) - 3 * math.sin(a0), 2 * math.cos(a1) - 4 * math.sin(a1),
            3 * math.cos(a0) + 1 * math.sin(a0), 4 * math.cos(a1) + 2 * math.sin(a1), 5.0, 6.0]
    assert torch.allclose(out[0, 0], torch.tensor(want, dtype=F64))
    assert torch.equal(P.rotate_halves(x, torch.tensor([0]), 4, 100.0), x)


def test_plain_window_keeps_the_first_tokens():
    m = P.window_mask(7, 3, 2)
    assert m[6].tolist() == [True, True, False, False, True, True, True]
    assert m[3].tolist() == [True, True, True, True, False, False, False]
    assert P.window_mask(4, 0)[3].tolist() == [True] * 4
    assert P.window_mask(5, 1)[4].tolist() == [False, False, False, False, True]


def test_plain_convolution_starts_from_zeros():
    u = torch.tensor([[1.0, 10.0], [2.0, 20.0], [3.0, 30.0]], dtype=F64)
    w = torch.tensor([[0.5, 1.0, 2.0], [1.0, 0.0, -1.0]], dtype=F64)   # the last tap multiplies the newest input
    y = P.causal_conv(u, w)
    assert torch.allclose(y[:, 0], torch.tensor([2.0, 1.0 + 4.0, 0.5 + 2.0 + 6.0], dtype=F64))
    assert torch.allclose(y[:, 1], torch.tensor([-10.0, -20.0, 10.0 - 30.0], dtype=F64))


def test_plain_softmax_one_more_in_the_denominator():
    q = torch.tensor([[[1.0]], [[1.0]]], dtype=F64)
    k = torch.tensor([[[0.0]], [[math.log(3.0)]]], dtype=F64)
    v = torch.tensor([[[2.0]], [[4.0]]], dtype=F64)
    out = P.masked_softmax_attention(q, k, v, 1.0, P.window_mask(2, 0), torch.zeros(1, dtype=F64))
    assert torch.allclose(out[:, 0, 0], torch.tensor([2.0 / 2.0, (2.0 + 3.0 * 4.0) / 5.0], dtype=F64))
    out = P.masked_softmax_attention(q, k, v, 1.0, P.window_mask(2, 0), torch.tensor([math.log(4.0)], dtype=F64))
    assert torch.allclose(out[:, 0, 0], torch.tensor([2.0 / 5.0, (2.0 + 3.0 * 4.0) / 8.0], dtype=F64))


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
