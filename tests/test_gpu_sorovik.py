"""Sorovik through the engine against the plain implementation (GPU): every way of cutting the
work, tiny configurations that differ in every size and option, float32 and bfloat16."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import gpu_harness as H
import sorovik_configs as C
from plain import sorovik_plain as P

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
F32_FRAC = 2e-5
LENGTHS = (1, 2, 9, 40, 77, 131, 203)


def check_rows(got, ref, dtype, what, f32_frac=F32_FRAC):
    return H.check_rows(got, ref, dtype, what, f32_frac=f32_frac)


def refs_of(cfg, weights, seqs):
    return [P.forward(cfg, weights, s, torch.float64) for s in seqs]


class Case:
    """A configuration with two sets of weights: freely routed tokens for float32, decisive routers for
    bfloat16 (see sorovik_configs.decisive_routers)."""

    def __init__(self, which, tmp, lengths=LENGTHS, seq_seed=7, seed=None, edit=None, patch=None):
        self.which = which if isinstance(which, str) else "custom"
        seed = ord(self.which[0]) if seed is None else seed
        self.by_dtype = {}
        for dtype, routers in (("float32", None), ("bfloat16", C.decisive_routers)):
            def both(w, routers=routers):
                if edit:
                    edit(w)
                if routers:
                    routers(w)
            d, cfg, weights = C.make_model_dir(which, str(tmp / dtype), seed=seed, edit=both, patch=patch)
            self.cfg = cfg
            self.seqs = C.sequences(cfg, lengths, seed=seq_seed)
            self.by_dtype[dtype] = (d, weights, refs_of(cfg, weights, self.seqs))

    def of(self, dtype):
        return self.by_dtype[dtype]


@pytest.fixture(scope="module", params=["A", "B", "C"])
def case(request, tmp_path_factory):
    return Case(request.param, tmp_path_factory.mktemp(f"sv{request.param}"))


def test_the_stream_after_every_layer(case):
    """The float32 residual stream after every layer against the plain implementation: the first
    difference names the layer."""
    d, weights, refs = case.of("float32")
    seq = case.seqs[4]
    want = []
    P.forward(case.cfg, weights, seq, torch.float64, layers_out=want)
    runner = H.make_runner(d, "float32", page_size=16, num_pages=8, num_slots=1)
    got = []
    for layer in runner.model.layers:
        def forward(stream, ctx, cache, orig=layer.forward):
            orig(stream, ctx, cache)
            got.append(stream.flush().clone())
        layer.forward = forward
    H.run_script(runner, [seq], H.script_whole([seq]))
    assert len(got) == len(want) == len(case.cfg["layers"])
    for i, (g, w) in enumerate(zip(got, want)):
        err = float((g.double().cpu() - w).abs().max())
        assert err <= 2e-5 * max(1.0, float(w.abs().max())), f"{case.which}: stream after layer {i}: {err:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cutting", ["whole", "tail", "portions", "mixed"])
def test_cuttings_agree_with_plain(case, dtype, cutting):
    which, seqs = case.which, case.seqs
    d, weights, refs = case.of(dtype)
    page_size = 16
    if cutting == "mixed":
        # so few pages and slots that they are used again
        budget = max((len(s) + page_size - 1) // page_size for s in seqs) + 5
        runner = H.make_runner(d, dtype, page_size=page_size, num_pages=budget, num_slots=3)
        script = H.script_mixed(seqs, max_live=3, seed=5, budget_pages=budget, page_size=page_size)
        assert any(len(p) > 1 and any(n == 1 for _, _, n in p) and any(n > 1 for _, _, n in p) for p, _ in script)
    else:
        runner = H.make_runner(d, dtype, page_size=page_size, num_pages=16, num_slots=2)
        script = {"whole": H.script_whole, "portions": H.script_portions,
                  "tail": lambda s: H.script_tail_one_by_one(s, tail=70)}[cutting](seqs)
    out = H.run_script(runner, seqs, script)
    for i, ref in enumerate(refs):
        check_rows(out[i], ref, dtype, f"{which} {dtype} {cutting} seq {i} (len {len(seqs[i])})")
    for g in runner.cache.groups.values():
        assert g.pool.n_free == g.num_pages  # every page came back
    assert runner.cache.free_slots == runner.cache.num_slots


@pytest.mark.parametrize("page_size", [16, 64])
def test_portions_of_two_tokens_and_page_borders(case, page_size):
    """Every portion is two tokens long (then three, so that both parities of a page's and a window's edge
    are met), against the whole prompt."""
    which, seqs = case.which, case.seqs
    d, weights, refs = case.of("float32")
    i = 5
    for width in (2, 3):
        runner = H.make_runner(d, "float32", page_size=page_size, num_pages=max(4, 256 // page_size), num_slots=1)
        n = len(seqs[i])
        script = [([(i, a, min(width, n - a))], [i] if a + width >= n else []) for a in range(0, n, width)]
        out = H.run_script(runner, seqs, script)
        check_rows(out[i], refs[i], "float32", f"{which} portions of {width}")


def test_long_decoding_from_the_first_token(case):
    """One prompt token, then 202 tokens one by one: windows pass over decoded tokens, pages are given back
    while the first ones stay, the convolution's window starts from zeros."""
    which, seqs = case.which, case.seqs
    for dtype in ("float32", "bfloat16"):
        d, weights, refs = case.of(dtype)
        runner = H.make_runner(d, dtype, page_size=16, num_pages=16, num_slots=1)
        out = H.run_script(runner, seqs[6:7], H.script_tail_one_by_one(seqs[6:7], tail=len(seqs[6]) - 1))
        check_rows(out[0], refs[6], dtype, f"{which} {dtype} long decoding")


def test_batch_of_unequal_requests_equals_each_alone(case):
    which, seqs = case.which, case.seqs
    for dtype in ("float32", "bfloat16"):
        d, weights, refs = case.of(dtype)
        runner = H.make_runner(d, dtype, page_size=16, num_pages=40, num_slots=4)
        pick = [1, 3, 4, 6]
        half = {i: len(seqs[i]) // 2 for i in pick}
        script = [([(i, 0, half[i]) for i in pick], []),
                  ([(i, half[i], len(seqs[i]) - half[i]) for i in pick], pick)]
        out = H.run_script(runner, seqs, script)
        for i in pick:
            check_rows(out[i], refs[i], dtype, f"{which} {dtype} batched seq {i}")


def test_slot_and_pages_used_again_start_clean(case):
    """A request that takes the slot and pages of a finished one sees nothing of it (neither its keys nor the
    last inputs of its convolution)."""
    which, seqs = case.which, case.seqs
    d, weights, refs = case.of("float32")
    runner = H.make_runner(d, "float32", page_size=16, num_pages=13, num_slots=1)
    script = [([(6, 0, 203)], [6]), ([(5, 0, 50)], []), ([(5, 50, 81)], [5]), ([(3, 0, 40)], [3])]
    out = H.run_script(runner, seqs, script)
    for i in (6, 5, 3):
        check_rows(out[i], refs[i], "float32", f"{which} reuse seq {i}")


def test_windowed_pages_come_back_and_first_pages_stay(tmp_path):
    """While a long request decodes, the pages behind every window are given back, except those that hold
    kept first tokens; a pool far smaller than the request is enough."""
    case = Case("A", tmp_path, lengths=(400,), seq_seed=5, seed=17)
    seqs = case.seqs
    d, weights, refs = case.of("float32")
    # windows of 24 (3 kept) and of up to 70 tokens on pages of 16: a request never holds more than 7 pages a group
    runner = H.make_runner(d, "float32", page_size=16, num_pages=9, num_slots=1)
    script = [([(0, 0, 100)], [])] + [([(0, p, min(7, 400 - p))], [0] if p + 7 >= 400 else []) for p in range(100, 400, 7)]
    held, first_held = [], []
    orig = runner.cache.advance

    def advance(req, n):
        out = orig(req, n)
        held.append({k: sum(1 for p in g.tables[req] if p >= 0) for k, g in runner.cache.groups.items()})
        first_held.append({k: g.tables[req][0] >= 0 for k, g in runner.cache.groups.items()})
        return out
    runner.cache.advance = advance
    out = H.run_script(runner, seqs, script)
    check_rows(out[0], refs[0], "float32", "pages given back")
    kept = 0
    for key, g in runner.cache.groups.items():
        assert g.window > 0 and max(h[key] for h in held) <= 7
        # the first page stays to the end only where first tokens are kept
        assert first_held[-1][key] == (g.keep_first > 0)
        kept += g.keep_first > 0
    assert kept == 1


def _loud(weights, cfg):
    """Weights under which a lost key, a window that is one token off, a sink left out or a wrong angle cannot
    hide.  In the first layer of either kind the first head's query and key are made large along one
    unrotated entry, so that single scores stand out by far wherever their keys lie (the last one inside a
    window, a kept first token hundreds back); the rotated parts are made large as a whole, so that positions
    decide scores; the sinks are raised to the level of those scores."""
    seen = set()
    for i, layer in enumerate(cfg["layers"]):
        if layer["type"] in seen or layer["mixer"].get("kv_from") is not None:
            continue
        seen.add(layer["type"])
        m, p = layer["mixer"], f"l{i}.mix."
        d = m["dim"]
        if layer["type"] == "latent_attention":
            rd = m["rot_dim"]
            weights[p + "q"][d - 1] *= 3.0
            weights[p + "uk"][d - 1] *= 3.0
            weights[p + "q"][d:d + rd] *= 2.0
            weights[p + "dkv"][m["kv_rank"]:] *= 2.0
            weights[p + "sink"] += 3.0
        else:
            weights[p + "q.norm"][d - 1] *= 3.0
            weights[p + "k.norm"][d - 1] *= 3.0
            weights[p + "q.norm"][:m["rot"]["dims"]] *= 1.5


@pytest.mark.parametrize("which", ["A", "B"])
def test_loud_far_keys_sinks_windows_and_positions(which, tmp_path):
    case = Case(which, tmp_path, lengths=(300,), seq_seed=3, seed=11, edit=lambda w: _loud(w, C.CONFIGS[which]))
    seqs, cfg = case.seqs, case.cfg
    for dtype in ("float32", "bfloat16"):
        d, weights, refs = case.of(dtype)
        ref = refs[0]
        # the oracle itself: with windows one token longer or shorter, one more or one fewer first token kept,
        # without the sinks, or with the one in the denominator left out, the logits move visibly
        def moved(change):
            other = json.loads(json.dumps(cfg))
            w2 = dict(weights)
            change(other, w2)
            return float((P.forward(other, w2, seqs[0], torch.float64) - ref).abs().max())
        def window_by(delta):
            def change(c, w):
                for layer in c["layers"]:
                    if layer["mixer"].get("mask", {}).get("size"):
                        layer["mixer"]["mask"]["size"] += delta
            return change
        def keep_by(delta):
            def change(c, w):
                for layer in c["layers"]:
                    if "keep_first" in layer["mixer"].get("mask", {}):
                        layer["mixer"]["mask"]["keep_first"] += delta
            return change
        def no_sink(c, w):
            for k in list(w):
                if k.endswith("mix.sink"):
                    w[k] = w[k] - 50.0
        assert moved(window_by(1)) > 0.5 and moved(window_by(-1)) > 0.5
        assert moved(keep_by(1)) > 0.5 and moved(keep_by(-1)) > 0.5
        assert moved(no_sink) > 0.5
        for script in (H.script_whole(seqs), H.script_tail_one_by_one(seqs, tail=100), H.script_portions(seqs, seed=2)):
            runner = H.make_runner(d, dtype, page_size=16, num_pages=24, num_slots=1)
            out = H.run_script(runner, seqs, script)
            if dtype == "float32":
                check_rows(out[0], ref, dtype, f"loud {which} {dtype}", f32_frac=4e-5)
                continue
            # loud scores magnify bfloat16 rounding at a few positions: all rows within twice the usual bound
            # (a fault moves them by three times as much and more), all but one in fifty within the bound itself
            frac = (out[0].double() - ref).abs().max(dim=1).values / float(ref.abs().max())
            assert bool(torch.isfinite(out[0]).all()) and float(frac.max()) <= 2 * H.BF16_FRAC, f"loud {which}: {float(frac.max()):.3f}"
            assert int((frac > H.BF16_FRAC).sum()) <= len(frac) // 50, f"loud {which}: {int((frac > H.BF16_FRAC).sum())} rows over"


def test_options_that_one_model_leaves_equal(tmp_path):
    """Configuration A with a latent layer that has no window while the layers that read its rows have one,
    an attention layer that keeps first tokens but as many as its window, a router without groups that takes
    every expert, and no feed-forward in the first layer."""
    def patch(cfg):
        del cfg["layers"][1]["mixer"]["mask"]
        cfg["layers"][0]["mixer"]["mask"] = {"size": 8, "keep_first": 8}
        cfg["layers"][0]["mlp"] = None
        cfg["layers"][3]["mlp"]["router"]["top"] = 5
    case = Case(C.SV_A, tmp_path, lengths=(57, 18), patch=patch, seed=31)
    seqs = case.seqs
    for dtype in ("float32", "bfloat16"):
        d, weights, refs = case.of(dtype)
        for script in (H.script_whole(seqs), H.script_portions(seqs, seed=4), H.script_tail_one_by_one(seqs, tail=30)):
            runner = H.make_runner(d, dtype, page_size=16, num_pages=8, num_slots=1)
            out = H.run_script(runner, seqs, script)
            for i, ref in enumerate(refs):
                check_rows(out[i], ref, dtype, f"options {dtype} seq {i}")


def test_sizes_that_are_multiples_of_nothing(tmp_path):
    """A width that is no multiple of 4, head sizes that are no multiples of 8, a latent of 6 entries beside 2
    rotated ones, a convolution of 6 taps, 7 experts in one group, an odd vocabulary: the scalar forms of the
    kernels and the float products."""
    cfg = {"architecture": "Sorovik", "vocab": 77, "width": 50, "norm": {"eps": 1e-5}, "layers": [
        C.layer(C.attention(3, 3, 10, 0.3, conv=6, rot=(6, 40.0), window=7, keep_first=2), C.moe(7, 3, 9)),
        C.layer(C.latent(3, 5, 2, 7, 6, 0.4, 2, 30.0, window=11), C.dense(33)),
        C.layer(C.latent(2, 9, 2, 3, 6, 0.3, 2, 30.0, window=19, kv_from=1), C.moe(6, 2, 10, groups=(3, 2))),
    ]}
    case = Case(cfg, tmp_path, lengths=(45, 3), seed=13)
    seqs = case.seqs
    for dtype in ("float32", "bfloat16"):
        d, weights, refs = case.of(dtype)
        for script in (H.script_whole(seqs), H.script_portions(seqs, seed=6), H.script_tail_one_by_one(seqs, tail=25)):
            runner = H.make_runner(d, dtype, page_size=16, num_pages=8, num_slots=1)
            out = H.run_script(runner, seqs, script)
            for i, ref in enumerate(refs):
                check_rows(out[i], ref, dtype, f"odd sizes {dtype} seq {i}")


def test_greedy_generation_through_the_engine(case):
    """Engine.generate (scheduler, sampler, decode graphs) against greedy decoding with the plain
    implementation, float32; bfloat16 with graphs against bfloat16 step by step."""
    from poor_mans_mamba_b200.entry import Engine
    which, seqs, cfg = case.which, case.seqs, case.cfg
    d, weights, refs = case.of("float32")
    prompts = [seqs[2], seqs[3][:23], seqs[1]]
    n_new = 12
    eng = Engine(d, dtype="float32", max_tokens=1024, max_seqs=4, page_size=16, max_batched_tokens=32)
    got = eng.generate(prompts, max_new_tokens=n_new, eos_token_id=-1)
    for p, g in zip(prompts, got):
        toks = list(p)
        for _ in range(n_new):
            lg = P.forward(cfg, weights, toks, torch.float64)[-1]
            top2 = torch.topk(lg, 2).values
            if float(top2[0] - top2[1]) < 1e-3:
                break  # a near tie: the two may disagree from here on without either being wrong
            toks.append(int(lg.argmax()))
        want = toks[len(p):]
        assert g[:len(want)] == want
    d = case.of("bfloat16")[0]
    a = Engine(d, dtype="bfloat16", max_tokens=1024, max_seqs=4, page_size=16, cuda_graphs=True).generate(
        prompts, max_new_tokens=n_new, eos_token_id=-1)
    b = Engine(d, dtype="bfloat16", max_tokens=1024, max_seqs=4, page_size=16, cuda_graphs=False).generate(
        prompts, max_new_tokens=n_new, eos_token_id=-1)
    assert a == b


def test_trace_program_replays_a_schedule(case, tmp_path):
    which, seqs, cfg = case.which, case.seqs, case.cfg
    if which != "A":
        pytest.skip("one configuration is enough for the program")
    steps = [
        {"step": 0, "entries": [{"id": "x", "tokens": seqs[3][:17], "want": [0, 16]},
                                {"id": "y", "tokens": seqs[2], "want": [8]}], "end": ["y"]},
        {"step": 1, "entries": [{"id": "x", "tokens": seqs[3][17:19], "want": []}], "end": []},
        {"step": 2, "entries": [{"id": "x", "tokens": seqs[3][19:], "want": [len(seqs[3]) - 20]},
                                {"id": "z", "tokens": seqs[1], "want": [1]}], "end": ["x", "z"]},
    ]
    for dtype in ("float32", "bfloat16"):
        d, weights, refs = case.of(dtype)
        out_dir = str(tmp_path / f"out_{dtype}")
        proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype,
                               "--out", out_dir, "--max-tokens", "128"],
                              input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
                              timeout=600)
        assert proc.returncode == 0, proc.stderr[-2000:]
        assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
        V = cfg["vocab"]
        s0 = np.fromfile(os.path.join(out_dir, "0.f32"), dtype="<f4").reshape(-1, V)
        s2 = np.fromfile(os.path.join(out_dir, "2.f32"), dtype="<f4").reshape(-1, V)
        assert not os.path.exists(os.path.join(out_dir, "1.f32"))
        want0 = torch.stack([refs[3][0], refs[3][16], refs[2][8]])
        want2 = torch.stack([refs[3][-1], refs[1][1]])
        check_rows(torch.from_numpy(s0), want0, dtype, "trace step 0")
        check_rows(torch.from_numpy(s2), want2, dtype, "trace step 2")


def test_command_line_generates_from_a_model_folder(case):
    which, seqs, cfg = case.which, case.seqs, case.cfg
    d, weights, refs = case.of("float32")
    if which != "B":
        pytest.skip("one configuration is enough for the program")
    prompt = ",".join(str(t) for t in seqs[2])
    proc = subprocess.run([sys.executable, "-m", "poor_mans_mamba_b200", d, "64", "GPU", "1", "2", "5", "--dtype", "float32",
                           "--prompt-ids", prompt, "--page-size", "16"], capture_output=True, text=True, timeout=600,
                          cwd=ROOT)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [l for l in proc.stdout.splitlines() if l.startswith("req_id=")]
    assert len(lines) == 2 and all("gen_tokens=5" in l for l in lines)
    toks = list(seqs[2])
    for _ in range(5):
        toks.append(int(P.forward(cfg, weights, toks, torch.float64)[-1].argmax()))
    assert str(toks[len(seqs[2]):]) in lines[0]


def test_medium_sizes_where_the_tensor_core_forms_run(tmp_path):
    """Cache rows and heads of 64 and 128 entries, prompts long enough for the tcgen05 attention, expert rows
    that the tensor-core grouped products take, pages of 64 tokens: whole, in portions that cut pages and
    windows anywhere, and with a long tail decoded through the decode attention."""
    case = Case("M", tmp_path, lengths=(700, 333), seq_seed=9, seed=21)
    seqs = case.seqs
    for dtype in ("float32", "bfloat16"):
        d, weights, refs = case.of(dtype)
        for name, script in (("whole", H.script_whole(seqs)),
                             ("tail", H.script_tail_one_by_one(seqs, tail=120)),
                             ("portions", [([(0, 0, 257)], []), ([(0, 257, 2), (1, 0, 130)], []),
                                           ([(0, 259, 300), (1, 130, 1)], []), ([(0, 559, 141), (1, 131, 202)], [0, 1])])):
            runner = H.make_runner(d, dtype, page_size=64, num_pages=20, num_slots=2)
            out = H.run_script(runner, seqs, script)
            for i, ref in enumerate(refs):
                check_rows(out[i], ref, dtype, f"medium {dtype} {name} seq {i}", f32_frac=4e-5)


def _random_config(seed):
    """A configuration drawn at random from the ranges a small model of this design may take: every size, the
    order of the layers, which layers read whose latent rows, windows, kept tokens, convolutions, groups."""
    import random
    rng = random.Random(2000 + seed)
    layers, owners = [], []
    for i in range(rng.randint(2, 6)):
        kind = rng.choice(["latent_attention", "latent_attention", "attention"])
        if kind == "latent_attention":
            dim = rng.choice([8, 16, 32, 48, 64])
            if owners and rng.random() < 0.5:
                j = rng.choice(owners)
                src = layers[j]["mixer"]
                rd, kv_rank, rot = src["rot_dim"], src["kv_rank"], dict(src["rot"])
                kv_from = j
            else:
                rd = rng.choice([4, 8, 16, 32])
                kv_rank = rng.choice([16, 24, 48, 64, 96, 112, 160, 200])
                rot = {"dims": rng.choice([rd, rd, rd // 2]), "base": rng.choice([100.0, 1e4, 1e6])}
                kv_from = None
                owners.append(i)
            mixer = {"heads": rng.randint(1, 8), "dim": dim, "rot_dim": rd, "vdim": rng.choice([8, 16, 32, 64]),
                     "kv_rank": kv_rank, "scale": (dim + rd) ** -0.5, "rot": rot}
            if rng.random() < 0.8:
                mixer["mask"] = {"size": rng.choice([1, 7, 16, 33, 64, 100])}
            if kv_from is not None:
                mixer["kv_from"] = kv_from
        else:
            dim = rng.choice([8, 16, 24, 32, 64, 128])
            G = rng.choice([1, 2, 3])
            mixer = {"heads": G * rng.randint(1, 4), "kv_heads": G, "dim": dim, "vdim": dim, "scale": dim ** -0.5}
            if rng.random() < 0.8:
                mixer["conv"] = rng.randint(1, 4)
            if rng.random() < 0.8:
                mixer["rot"] = {"dims": rng.choice([dim, dim // 2, dim // 4 * 2]), "base": rng.choice([100.0, 5e4])}
            if rng.random() < 0.8:
                mixer["mask"] = {"size": rng.choice([1, 5, 16, 40, 65])}
                if rng.random() < 0.8:
                    mixer["mask"]["keep_first"] = rng.choice([0, 1, 4, 17, 70])
        what = rng.choice(["dense", "moe", "moe", None])
        mlp = None
        if what == "dense":
            mlp = {"kind": "dense", "ff": 8 * rng.randint(8, 60)}
        elif what == "moe":
            experts = rng.choice([4, 6, 8, 12, 16])
            count = rng.choice([c for c in (1, 2, 3, 4, experts) if experts % c == 0])
            keep = rng.randint(1, count)
            router = {"experts": experts, "top": rng.randint(1, min(6, keep * (experts // count)))}
            if count > 1 or rng.random() < 0.5:
                router["groups"] = {"count": count, "keep": keep}
            mlp = {"kind": "moe", "router": router, "expert": {"ff": 8 * rng.randint(2, 16)}}
        layers.append({"type": kind, "mixer": mixer, "mlp": mlp})
    return {"architecture": "Sorovik", "vocab": rng.randint(100, 700), "width": rng.choice([96, 136, 160, 200, 256, 328]),
            "norm": {"eps": rng.choice([1e-6, 1e-5])}, "layers": layers}


@pytest.mark.parametrize("seed", range(8))
def test_configurations_drawn_at_random(seed, tmp_path):
    cfg = _random_config(seed)
    case = Case(cfg, tmp_path, lengths=(150, 37, 70), seq_seed=seed, seed=50 + seed)
    seqs = case.seqs
    for dtype in ("float32", "bfloat16"):
        d, weights, refs = case.of(dtype)
        for name, script in (("whole", H.script_whole(seqs)),
                             ("mixed", H.script_mixed(seqs, max_live=3, seed=seed, budget_pages=8, page_size=64))):
            runner = H.make_runner(d, dtype, page_size=64, num_pages=8, num_slots=3)
            out = H.run_script(runner, seqs, script)
            for i, ref in enumerate(refs):
                check_rows(out[i], ref, dtype, f"random {seed} {dtype} {name} seq {i}: {json.dumps(cfg)[:300]}", f32_frac=4e-5)
