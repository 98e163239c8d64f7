"""Each mechanism of the Gikovik parts alone against its plain function (GPU): the kernels and parts
are called as the model calls them, on inputs made so that a fault shows."""
import math
import types

import pytest
import torch

from plain import gikovik_plain as P

from poor_mans_mamba_b200.engine.workspace import Workspace
from poor_mans_mamba_b200.kernels import ops as K
from poor_mans_mamba_b200.parts.base import PartSpec, build_part
import poor_mans_mamba_b200.parts  # noqa: F401  (registration)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def rnd(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16).float()


def close(got, want, dtype, what, f32=2e-5, bf16=2e-2):
    got, want = got.double().cpu(), want.double()
    tol = (f32 if dtype == torch.float32 else bf16) * max(1.0, float(want.abs().max()))
    err = float((got - want).abs().max())
    assert err <= tol, f"{what}: {err:.3e} > {tol:.3e}"


def inv_freq(dims, base):
    i = torch.arange(dims // 2, dtype=torch.float64)
    return torch.pow(torch.tensor(base, dtype=torch.float64), -2.0 * i / dims).float().to(DEV)


# ----------------------------------------------------------------------------- latents into the pages
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("q_rank,kv_rank,rot_dim,rot_dims", [(20, 28, 0, 0), (36, 20, 12, 8), (8, 140, 0, 0), (24, 40, 8, 8),
                                                             (128, 112, 16, 16), (16, 24, 40, 16), (5, 3, 2, 2)])
def test_normed_latents_and_the_rotated_key_part_in_their_pages(dtype, q_rank, kv_rank, rot_dim, rot_dims):
    """Positions up to 1,000 in two sequences whose pages are not in order: the normed query latent, and what the
    pages hold afterwards (key row [normed latent | turned part | 0], value row [normed latent | 0])."""
    page, eps, base = 16, 1e-3, 300.0
    Dp = K.latent_padded_dim(kv_rank, rot_dim)
    positions = [0, 1, 15, 16, 17, 999, 1000, 5, 31, 32]
    seq = [0, 0, 0, 0, 0, 0, 0, 1, 1, 1]
    T = len(positions)
    # the projections of a step come as column blocks of one wider matrix
    wide = rnd(T, q_rank + kv_rank + rot_dim + 3, seed=1, scale=2.0).to(DEV, dtype)
    ql, kvl = wide[:, :q_rank], wide[:, q_rank:q_rank + kv_rank + rot_dim]
    qw, kw = rnd(q_rank, seed=2) + 1.0, rnd(kv_rank, seed=3) + 1.0
    n_blocks = 1000 // page + 1
    perm = torch.randperm(2 * n_blocks, generator=torch.Generator().manual_seed(7)).to(torch.int32)
    table = perm.view(2, n_blocks).to(DEV)
    pool = torch.full((2 * n_blocks, 2, page, Dp), 7.0, dtype=dtype, device=DEV)  # a page used before: no zeros in it
    cq = torch.empty(T, q_rank, dtype=dtype, device=DEV)
    inv = inv_freq(rot_dims, base) if rot_dims else None
    pos_t = torch.tensor(positions, dtype=torch.int32, device=DEV)
    K.latent_norm_store(ql, kvl, qw.to(DEV), kw.to(DEV), eps, inv, pos_t, torch.tensor(seq, dtype=torch.int32, device=DEV),
                        table, pool, cq, kv_rank, rot_dim, rot_dims)
    q64, kv64 = ql.double().cpu(), kvl.double().cpu()
    close(cq, P.rms_norm(q64, qw.double(), eps), dtype, "query latent")
    c = P.rms_norm(kv64[:, :kv_rank], kw.double(), eps)
    turned = P.rotate_pairs(kv64[:, None, kv_rank:], torch.tensor(positions), rot_dims, base)[:, 0]
    for t in range(T):
        pg = int(table[seq[t], positions[t] // page])
        row_k, row_v = pool[pg, 0, positions[t] % page], pool[pg, 1, positions[t] % page]
        close(row_k[:kv_rank], c[t], dtype, "latent in the key row")
        close(row_v[:kv_rank], c[t], dtype, "latent in the value row")
        if rot_dim:
            close(row_k[kv_rank:kv_rank + rot_dim], turned[t], dtype, "turned key part", f32=3e-5)
        assert float(row_k[kv_rank + rot_dim:].abs().max()) == 0.0 if Dp > kv_rank + rot_dim else True
        assert float(row_v[kv_rank:].abs().max()) == 0.0 if Dp > kv_rank else True


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,dim,rot_dim,rot_dims,kv_rank", [(3, 24, 12, 8, 20), (5, 16, 8, 8, 40), (1, 40, 40, 16, 24),
                                                            (8, 48, 16, 16, 112), (4, 16, 0, 0, 28)])
def test_rotated_query_part_beside_the_absorbed_one(dtype, H, dim, rot_dim, rot_dims, kv_rank):
    Dp, base = K.latent_padded_dim(kv_rank, rot_dim), 1000.0
    positions = [0, 1, 2, 63, 64, 500, 4095]
    T = len(positions)
    q = rnd(T, H * (dim + rot_dim), seed=4).to(DEV, dtype)
    out = torch.full((T, H * Dp), 3.0, dtype=dtype, device=DEV)
    K.latent_query_rot(q, inv_freq(rot_dims, base) if rot_dims else None, torch.tensor(positions, dtype=torch.int32, device=DEV),
                       out, H, dim, rot_dim, rot_dims, kv_rank, Dp)
    got = out.view(T, H, Dp)
    assert bool((got[:, :, :kv_rank] == 3.0).all())  # the absorbed part is another kernel's
    if rot_dim:
        want = P.rotate_pairs(q.double().cpu().view(T, H, dim + rot_dim)[:, :, dim:], torch.tensor(positions), rot_dims, base)
        close(got[:, :, kv_rank:kv_rank + rot_dim], want, dtype, "turned query part", f32=3e-5)
    if Dp > kv_rank + rot_dim:
        assert float(got[:, :, kv_rank + rot_dim:].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
def test_head_gate_per_head_products_and_the_squared_relu(dtype):
    T, H, dv = 7, 5, 24
    a, g = rnd(T, H * dv, seed=1), rnd(T, H + 3, seed=2, scale=2.0)
    gd = g.to(DEV, dtype)[:, 1:1 + H]  # a column block of the step's projections
    out = torch.empty(T, H * dv, dtype=dtype, device=DEV)
    K.head_gate(a.to(DEV, dtype), gd, 1.0, out, H, dv)
    want = a.double().view(T, H, dv) * torch.sigmoid(g[:, 1:1 + H].double())[:, :, None]
    close(out, want.reshape(T, H * dv), dtype, "gate")
    x, w = rnd(T, H, 12, seed=3), rnd(H, 12, 20, seed=4)
    buf = torch.zeros(T, H, 32, dtype=dtype, device=DEV)
    K.head_linear(x.to(DEV, dtype), w.to(DEV, dtype), buf[:, :, :20])
    close(buf[:, :, :20], torch.einsum("thk,hkn->thn", x.double(), w.double()), dtype, "per-head product")
    assert float(buf[:, :, 20:].abs().max()) == 0.0
    z = rnd(T, 37, seed=5, scale=2.0)
    act = torch.empty(T, 37, dtype=dtype, device=DEV)
    K.relu_squared(z.to(DEV, dtype), act)
    close(act, P.relu_squared(z.double()), dtype, "squared relu")


# ----------------------------------------------------------------------------- the whole mixer on one sequence
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rotated", [False, True])
def test_latent_mixer_on_a_prompt_and_then_token_by_token(dtype, rotated, tmp_path):
    """The mixer of a one-layer model, its result taken where the layer receives it: a prompt of 70 tokens in
    one step and 30 more one by one, against keys and values made head by head from the latents.  One head's
    query and key are loud along one entry, and the sink (or the turned part) is large enough to move the
    result."""
    import gikovik_configs as C
    import gpu_harness as H
    mixer = {"heads": 3, "dim": 16, "vdim": 24, "q_rank": 20, "kv_rank": 36, "scale": 0.2}
    if rotated:
        mixer.update({"rot_dim": 12, "rot": {"dims": 8, "base": 50.0}})
    cfg = {"architecture": "Gikovik", "vocab": 150, "width": 56, "norm": {"eps": 1e-5},
           "layers": [{"type": "latent_attention_2" if rotated else "latent_attention", "mixer": mixer, "mlp": None}]}

    def edit(w):
        w["l0.mix.uq"][15] *= 6.0
        w["l0.mix.uk"][15] *= 6.0
        if rotated:
            w["l0.mix.uq"][16:28] *= 3.0
            w["l0.mix.dkv"][36:] *= 3.0
        else:
            w["l0.mix.sink"] += 3.0
    d, cfg, w = C.make_model_dir(cfg, str(tmp_path), seed=5, edit=edit)
    toks = C.sequences(cfg, (100,), seed=2)[0]
    W = {k: v.double() for k, v in w.items()}
    n = P.rms_norm(W["embed"][torch.tensor(toks)], W["l0.norm1"], 1e-5)
    want = P.latent_attention(n, W, "l0.mix.", mixer, 1e-5, torch.arange(100))
    if not rotated:  # the sink moves the result
        other = dict(W)
        other["l0.mix.sink"] = W["l0.mix.sink"] - 50.0
        assert float((P.latent_attention(n, other, "l0.mix.", mixer, 1e-5, torch.arange(100)) - want).abs().max()) > 0.05
    runner = H.make_runner(d, dtype, page_size=16, num_pages=8, num_slots=1)
    part, got = runner.model.layers[0].mixer, []

    def forward(x, ctx, cache, out, orig=part.forward):
        orig(x, ctx, cache, out)
        got.append(out.float().clone())
    part.forward = forward
    H.run_script(runner, [toks], H.script_tail_one_by_one([toks], tail=30))
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    close(torch.cat(got), want, tdt, "latent mixer", f32=3e-5, bf16=3e-2)


# ----------------------------------------------------------------------------- the token input and the re-entry
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D,R,layers,layer,T", [(72, 6, 4, 2, 9), (100, 1, 3, 0, 9), (44, 3, 2, 1, 9), (384, 24, 3, 2, 9),
                                                 (1031, 16, 2, 1, 9), (1024, 32, 2, 1, 9), (320, 16, 2, 0, 1030), (72, 6, 3, 1, 1027),
                                                 (1024, 32, 2, 1, 1100), (192, 64, 2, 0, 1025)])
def test_token_input_with_waiting_branches(dtype, D, R, layers, layer, T):
    """Rows read one entry and four entries at a time, one token and four tokens a block (a step of many tokens, its
    last block short)."""
    V, eps = 50, 1e-4
    h = rnd(T, D, seed=1, scale=2.0)
    a, b = rnd(T, D, seed=2), rnd(T, D, seed=3, scale=0.5)
    table = rnd(V, layers * R, seed=4)
    wg, wp, nw = rnd(R, D, seed=5, scale=1.5 / math.sqrt(D)), rnd(D, R, seed=6, scale=1.0 / math.sqrt(R)), rnd(D, seed=7) * 0.2 + 0.5
    tokens = torch.tensor([3, 49, 0, 3, 17, 8, 8, 21, 30] * (T // 9 + 1))[:T]
    W = {"side.embed": table.double(), f"l{layer}.side.gate": wg.double(), f"l{layer}.side.proj": wp.double(),
         f"l{layer}.side.norm": nw.double()}
    ad, bd = a.to(DEV, dtype), b.to(DEV, dtype)
    for branches, x in (([], h.double()), ([(ad, 1.0)], h.double() + ad.double().cpu()),
                        ([(ad, 1.0), (bd, 0.5)], h.double() + ad.double().cpu() + 0.5 * bd.double().cpu())):
        want = P.token_input(x, tokens, W, layer, R, eps)
        # with the matrix as stored, bfloat16 steps of many tokens take the tensor-core form where the sizes allow
        for rows in (None, wp.to(DEV, dtype)):
            hd = h.to(DEV).clone()
            K.token_gated_update(hd, branches, tokens.to(DEV, torch.int32), table.to(DEV, dtype), layer * R, wg.to(DEV, dtype),
                                 wp.t().contiguous().to(DEV, dtype), nw.to(DEV), eps, w_proj_rows=rows)
            # the stream itself is float in both storage types; only the small products read rounded operands
            close(hd, want, torch.float32, f"token input, {len(branches)} branches", f32=3e-5 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D", [44, 72, 384])
def test_embedding_reentry_replaces_the_stream(dtype, D):
    T = 11
    h, x0 = rnd(T, D, seed=1, scale=2.0), rnd(T, D, seed=2)
    w = rnd(D, 2 * D, seed=3, scale=1.0 / math.sqrt(2 * D))
    part = build_part("stream_update", PartSpec("embedding_reentry", "loop", {"tensor": "in"}), hidden_size=D)
    part.bind({"in": w.to(DEV, dtype)})
    ctx = types.SimpleNamespace(workspace=Workspace(torch.device(DEV)), dtype=dtype)
    both = torch.zeros(T, 2 * D, dtype=dtype, device=DEV)
    both[:, D:] = x0.to(DEV, dtype)
    a = rnd(T, D, seed=4).to(DEV, dtype)
    stream = types.SimpleNamespace(h=h.to(DEV).clone(), reentry=both, pending=[(a, 1.0)])
    stream.take_pending = lambda n: (stream.pending, setattr(stream, "pending", []))[0]
    part.forward(stream, ctx)
    x = h.double() + a.double().cpu()
    xin = x if dtype == torch.float32 else x.to(torch.bfloat16).double()
    want = torch.cat([xin, x0.double()], dim=-1) @ w.double().t()
    close(stream.h, want, dtype, "re-entry", f32=3e-5)
    assert stream.h.dtype == torch.float32


# ----------------------------------------------------------------------------- the scored router and its experts
def _scored_case(D, E, F, Fs, seed, T):
    names = {"router": (E, D), "correction": (E,)}
    for e in range(E):
        names.update({f"e{e}.up": (F, D), f"e{e}.down": (D, F)})
    if Fs:
        names.update({"shared.up": (Fs, D), "shared.down": (D, Fs), "shared.sg": (1, D)})
    w = {}
    for i, (n, shape) in enumerate(names.items()):
        gain = 2.0 if n in ("router", "shared.sg") else 1.5
        w[n] = rnd(*shape, seed=seed * 1000 + i, scale=gain / math.sqrt(shape[-1]) if len(shape) > 1 else 0.3)
    return w, rnd(T, D, seed=seed + 7)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D,E,top,F,Fs,T,groups,keep,scale", [
    (72, 6, 3, 40, 24, 33, 3, 2, 1.5),      # rows of whole 16-byte groups: the tensor-core products in bfloat16
    (100, 5, 2, 20, 0, 7, 1, 1, 1.0),       # no groups, no shared expert, float products
    (44, 12, 5, 12, 8, 300, 6, 3, 2.5),     # groups of two: a group's score is the sum of both
    (44, 9, 3, 8, 0, 50, 9, 4, 1.0),        # groups of one
    (64, 16, 1, 48, 80, 1, 4, 1, 0.5),      # a single token, one expert a token
    (128, 8, 4, 96, 32, 517, 2, 1, 2.0),    # several row tiles, a ragged last one, every expert of the kept group
    (256, 8, 2, 192, 64, 700, 4, 2, 1.25),  # rows of whole 128-byte pieces and many pairs: the tcgen05 products in bfloat16
    (128, 4, 4, 64, 0, 900, 1, 1, 3.0),     # every expert for every token
])
def test_scored_router_and_ungated_experts_against_the_plain_sum(dtype, D, E, top, F, Fs, T, groups, keep, scale):
    w, x = _scored_case(D, E, F, Fs, seed=3, T=T)
    part = build_part("feed_forward", PartSpec("routed_scored", "mlp", {
        "experts": E, "top": top, "expert_ff": F, "scale": scale, "groups": groups, "keep": keep, "correction": True,
        "shared_ff": Fs, "shared_gate": True}), hidden_size=D)
    params = {}
    for ps in part.param_specs():
        t = w[ps.name].to(DEV)
        params[ps.name] = t if ps.kind == "vector" else t.to(dtype)
    part.bind(params)
    part.finalize(dtype, torch.device(DEV))
    ctx = types.SimpleNamespace(workspace=Workspace(torch.device(DEV)), dtype=dtype)
    xd = x.to(DEV, dtype)
    out = torch.full((T, D), float("nan"), dtype=dtype, device=DEV)
    part.forward(xd, ctx, out)
    cfg = {"router": {"experts": E, "top": top, "scale": scale, "groups": {"count": groups, "keep": keep}}, "expert": {"ff": F}}
    if Fs:
        cfg["shared"] = {"ff": Fs}
    # the router's choice itself, where neither the groups nor the experts are a close call
    z = x.double() @ w["router"].double().t()
    choice = torch.sigmoid(z) + w["correction"].double()
    per = choice.view(T, groups, E // groups)
    gs = per.topk(min(2, E // groups), dim=-1).values.sum(-1)
    gsort = gs.sort(dim=-1, descending=True).values
    sure = (gsort[:, keep - 1] - gsort[:, keep]) > 1e-3 if keep < groups else torch.ones(T, dtype=torch.bool)
    want_ids, want_w = P.route(z, w["correction"].double(), top, {"count": groups, "keep": keep}, scale)
    allowed = torch.zeros(T, groups, dtype=torch.bool).scatter_(1, gs.topk(keep, dim=-1).indices, True)
    masked = choice.masked_fill(~allowed[:, :, None].expand(T, groups, E // groups).reshape(T, E), -math.inf)
    csort = masked.sort(dim=-1, descending=True).values
    gaps = csort[:, :top] - csort[:, 1:top + 1] if top < E else csort[:, :top - 1] - csort[:, 1:top]
    if gaps.numel():
        sure &= gaps.min(dim=-1).values > 1e-3
    ids = torch.empty(T, top, dtype=torch.int32, device=DEV)
    pw = torch.empty(T, top, dtype=torch.float32, device=DEV)
    gate = torch.empty(T, dtype=torch.float32, device=DEV)
    K.moe_route(xd, params["router"], None, top, ids, pw, scored=True, correction=params["correction"], groups=groups,
                keep=keep, scale=scale, gate_w=params["shared.sg"].reshape(-1) if Fs else None, gate_out=gate if Fs else None)
    got_sorted, order = ids.cpu().long().sort(dim=-1)
    want_sorted, want_order = want_ids.sort(dim=-1)
    assert torch.equal(got_sorted[sure], want_sorted[sure])
    assert T < 8 or int(sure.sum()) >= T // 2  # (most tokens are far from a close call)
    if bool(sure.any()):
        close(pw.cpu().gather(1, order)[sure], want_w.gather(1, want_order)[sure], torch.float32, "router weights", f32=1e-5)
    if Fs:
        close(gate, torch.sigmoid(x.double() @ w["shared.sg"].double().t()).view(-1), torch.float32, "shared expert's gate", f32=1e-5)
    # the output: tokens on a close call may take either side, so only the sure ones are compared
    want = P.routed_ffn(x.double(), {"mlp." + k: v.double() for k, v in w.items()}, "mlp.", cfg)
    close(out[sure.to(DEV)], want[sure], dtype, "routed feed-forward", f32=3e-5, bf16=3e-2)
