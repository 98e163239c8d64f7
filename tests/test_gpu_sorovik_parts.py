"""Each mechanism of the Sorovik parts alone against its plain function (GPU): the kernels are called as
the model calls them, on inputs made so that a fault shows."""
import math

import pytest
import torch

from plain import sorovik_plain as P

from poor_mans_mamba_b200.kernels import ops as K
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


def i32(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


# ----------------------------------------------------------------------------- norms
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D", [44, 72, 328, 1030])
def test_embedding_with_its_norm(dtype, D):
    V, eps = 50, 1e-3
    table, w = rnd(V, D, seed=1, scale=3.0), rnd(D, seed=2) * 0.2 + 1.0
    tokens = [0, 49, 7, 7, 23]
    out = torch.empty(len(tokens), D, dtype=torch.float32, device=DEV)
    K.embed(out, table.to(DEV, dtype), i32(tokens), 1.0, w.to(DEV), eps)
    close(out, P.rms_norm(table.double()[tokens], w.double(), eps), torch.float32, "normed embedding")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D,branches", [(44, 1), (72, 2), (328, 1), (1030, 2), (2048, 1), (3072, 2), (5000, 2), (9000, 1)])
def test_post_norm_of_a_sublayer_and_norm_of_the_stream_in_one_launch(dtype, D, branches):
    """x <- x + rms(sum of branches) * w_post, out = rms(x) * w: for all rows, for chosen rows (the stream is
    then left alone), without a following norm, and without a stream."""
    T, eps_p, eps = 9, 1e-2, 1e-5
    h0 = rnd(T, D, seed=1, scale=2.0)
    bs = [(rnd(T, D, seed=2 + i, scale=0.5 + i), 1.0 - 0.5 * i) for i in range(branches)]
    wp, w = rnd(D, seed=7) * 0.3 + 0.5, rnd(D, seed=8) * 0.2 + 1.0
    dev_b = [(b.to(DEV, dtype), s) for b, s in bs]
    total = sum(s * b.to(dtype).double() for b, s in bs)
    x = h0.double() + P.rms_norm(total, wp.double(), eps_p)
    want = P.rms_norm(x, w.double(), eps)
    h = h0.to(DEV).clone()
    out = torch.empty(T, D, dtype=dtype, device=DEV)
    K.add_postnorm_rmsnorm(h, dev_b, wp.to(DEV), eps_p, w.to(DEV), eps, out)
    close(h, x, torch.float32, "stream")
    close(out, want, dtype, "normed stream", bf16=1e-2)
    rows = [7, 0, 3]
    h = h0.to(DEV).clone()
    out = torch.empty(len(rows), D, dtype=dtype, device=DEV)
    K.add_postnorm_rmsnorm(h, dev_b, wp.to(DEV), eps_p, w.to(DEV), eps, out, i32(rows))
    assert torch.equal(h.cpu(), h0)
    close(out, want[rows], dtype, "chosen rows", bf16=1e-2)
    h = h0.to(DEV).clone()
    K.add_postnorm_rmsnorm(h, dev_b, wp.to(DEV), eps_p, None, 0.0, None)
    close(h, x, torch.float32, "stream, nothing normed")
    out = torch.empty(T, D, dtype=dtype, device=DEV)
    K.add_postnorm_rmsnorm(None, dev_b, wp.to(DEV), eps_p, None, 0.0, out)
    close(out, P.rms_norm(total, wp.double(), eps_p), dtype, "post norm alone", bf16=1e-2)


# ----------------------------------------------------------------------------- activation and router
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("F", [12, 88, 520])
def test_gate_with_the_tanh_form_of_gelu(dtype, F):
    T = 5
    gu = rnd(T, 2 * F + 4, seed=1, scale=2.5)
    dev = gu.to(DEV, dtype)[:, :2 * F] if F % 8 else gu[:, :2 * F].contiguous().to(DEV, dtype)
    out = torch.empty(T, F, dtype=dtype, device=DEV)
    K.gelu_tanh_mul(dev, 1.0, out)
    g, u = dev.double().cpu()[:, :F], dev.double().cpu()[:, F:]
    close(out, P.gelu_tanh(g) * u, dtype, "gelu gate")
    z = torch.tensor([-3.0, -1.0, 0.0, 0.5, 2.0], dtype=torch.float64)   # values done by hand
    by_hand = [0.5 * v * (1 + math.tanh(math.sqrt(2 / math.pi) * (v + 0.044715 * v ** 3))) for v in z.tolist()]
    assert torch.allclose(P.gelu_tanh(z), torch.tensor(by_hand, dtype=torch.float64))


def test_gelu_gate_in_the_epilogue_of_the_tensor_core_product():
    """The dense feed-forward's [gate | up] product of a prompt step with the activation in its epilogue, against
    the product followed by the activation launch and against the plain functions."""
    T, D, F = 600, 448, 512
    x, w = rnd(T, D, seed=1).to(DEV, torch.bfloat16), rnd(2 * F, D, seed=2, scale=D ** -0.5 * 2).to(DEV, torch.bfloat16)
    if not K.tc_gemm_supported(x, w, F, True):
        pytest.skip("sizes the tcgen05 product does not take")
    out = torch.empty(T, F, dtype=torch.bfloat16, device=DEV)
    K.tc_gemm_gelu_glu(x, w, 1.0, out)
    torch.cuda.synchronize()
    assert K.tc_gemm_status(x.device) == 0
    gu = x.double().cpu() @ w.double().cpu().t()
    close(out, P.gelu_tanh(gu[:, :F]) * gu[:, F:], torch.bfloat16, "gelu gate in the epilogue")


@pytest.mark.parametrize("E,top,groups,keep", [(8, 3, 2, 1), (6, 2, 3, 2), (12, 5, 6, 3), (9, 3, 9, 4), (4, 4, 1, 1),
                                               (16, 1, 4, 1), (5, 2, 1, 1), (64, 6, 8, 3)])
@pytest.mark.parametrize("T", [7, 700])
def test_router_softmax_over_all_groups_by_their_largest_score(E, top, groups, keep, T):
    """Choice and weights where no call is close: the scores are the softmax over ALL experts, a group counts
    by its largest score, the weights are the chosen scores themselves (they do not sum to one)."""
    D = 40
    x, w = rnd(T, D, seed=E + T), rnd(E, D, seed=top, scale=0.6)
    ids = torch.empty(T, top, dtype=torch.int32, device=DEV)
    weights = torch.empty(T, top, dtype=torch.float32, device=DEV)
    K.moe_route(x.to(DEV), w.to(DEV), None, top, ids, weights, scored="softmax", groups=groups, keep=keep)
    z = x.double() @ w.double().t()
    checked = 0
    for t in range(T):
        gaps = (z[t][:, None] - z[t][None, :]).abs() + torch.eye(E, dtype=torch.float64)
        if float(gaps.min()) < 1e-4:
            continue  # a close call: either choice is right
        chosen, ws = P.route(z[t], top, groups, keep)
        assert ids[t].tolist() == chosen, f"token {t}"
        close(weights[t], torch.stack(ws), torch.float32, "weights", f32=1e-5)
        checked += 1
    assert checked > T // 2
    assert float(weights.sum(dim=1).max()) <= 1.0 + 1e-5
    if top < E:
        assert float(weights.sum(dim=1).min()) < 0.999  # not divided by their sum


def test_plain_router_by_hand():
    # scores 0.1 0.2 | 0.45 0.05 | 0.15 0.05: two groups kept -> groups 1 and 0; top 3 -> experts 2, 1, 0
    z = torch.log(torch.tensor([0.1, 0.2, 0.45, 0.05, 0.15, 0.05], dtype=torch.float64))
    chosen, ws = P.route(z, 3, 3, 2)
    assert chosen == [2, 1, 0] and torch.allclose(torch.stack(ws), torch.tensor([0.45, 0.2, 0.1], dtype=torch.float64))
    chosen, ws = P.route(z, 2, 3, 1)
    assert chosen == [2, 3]
    chosen, ws = P.route(z, 3, 1, 1)
    assert chosen == [2, 1, 4]


# ----------------------------------------------------------------------------- queries, keys and values into place
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,d,rot_dims,bias", [(4, 2, 24, 16, False), (3, 3, 16, 16, True), (6, 2, 8, 4, False),
                                                 (4, 1, 40, 0, False), (8, 2, 64, 32, False)])
def test_norm_over_the_whole_projection_then_rotation_into_the_pages(dtype, H, G, d, rot_dims, bias):
    """Positions up to 1,000 in two sequences whose pages are not in order: the queries, and what the pages hold
    afterwards (key rows normed over all heads at once and turned in halves, value rows the keys as they came)."""
    page, eps, base = 16, 1e-3, 300.0
    Dp = (d + 15) // 16 * 16
    positions = [0, 1, 15, 16, 17, 999, 1000, 5, 31, 32]
    seq = [0, 0, 0, 0, 0, 0, 0, 1, 1, 1]
    T = len(positions)
    wide = rnd(T, (H + G) * d + 5, seed=1, scale=2.0).to(DEV, dtype)
    q, k = wide[:, :H * d], wide[:, H * d:(H + G) * d]
    qn, kn = rnd(H * d, seed=2) * 0.3 + 1.0, rnd(G * d, seed=3) * 0.3 + 1.0
    qb, kb = rnd(H * d, seed=4), rnd(G * d, seed=5)
    n_blocks = 1000 // page + 1
    table = torch.randperm(2 * n_blocks, generator=torch.Generator().manual_seed(7)).to(torch.int32).view(2, n_blocks).to(DEV)
    pool = torch.full((2 * n_blocks, 2, page, G * Dp), 7.0, dtype=dtype, device=DEV)  # pages used before
    q_out = torch.full((T, H * Dp), 5.0, dtype=dtype, device=DEV)
    biases = (qb.to(DEV), kb.to(DEV), kb.to(DEV)) if bias else None
    K.rope_pairs_store(q, k, k, inv_freq(rot_dims, base) if rot_dims else None, rot_dims, i32(positions), i32(seq), table,
                       pool, q_out, H, G, d, d, Dp, half_layout=True, biases=biases, qk_norm=(qn.to(DEV), kn.to(DEV), eps))
    q64 = q.double().cpu() + (qb.double() if bias else 0.0)
    k64 = k.double().cpu() + (kb.double() if bias else 0.0)
    pos = torch.tensor(positions)
    want_q = P.rotate_halves(P.rms_norm(q64, qn.double(), eps).view(T, H, d), pos, rot_dims, base)
    want_k = P.rotate_halves(P.rms_norm(k64, kn.double(), eps).view(T, G, d), pos, rot_dims, base)
    close(q_out.view(T, H, Dp)[:, :, :d], want_q, dtype, "queries", f32=3e-5)
    for t in range(T):
        pg = int(table[seq[t], positions[t] // page])
        row_k = pool[pg, 0, positions[t] % page].view(G, Dp)
        row_v = pool[pg, 1, positions[t] % page].view(G, Dp)
        close(row_k[:, :d], want_k[t], dtype, "key row", f32=3e-5)
        close(row_v[:, :d], k64[t].view(G, d), dtype, "value row: the key before norm and rotation")
        if Dp > d:
            assert float(row_k[:, d:].abs().max()) == 0.0 and float(row_v[:, d:].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kv_rank,rot_dim,rot_dims", [(20, 12, 8), (100, 20, 20), (140, 4, 4), (112, 16, 16), (24, 8, 0)])
def test_latent_rows_with_halves_turned_and_queries_without_a_latent(dtype, kv_rank, rot_dim, rot_dims):
    page, eps, base, H, dim = 16, 1e-3, 300.0, 3, 8
    Dp = K.latent_padded_dim(kv_rank, rot_dim)
    positions = [0, 1, 15, 16, 17, 999, 1000, 5, 31, 32]
    seq = [0, 0, 0, 0, 0, 0, 0, 1, 1, 1]
    T = len(positions)
    wide = rnd(T, kv_rank + rot_dim + 3, seed=1, scale=2.0).to(DEV, dtype)
    kvl = wide[:, 2:2 + kv_rank + rot_dim]
    kw = rnd(kv_rank, seed=3) + 1.0
    n_blocks = 1000 // page + 1
    table = torch.randperm(2 * n_blocks, generator=torch.Generator().manual_seed(9)).to(torch.int32).view(2, n_blocks).to(DEV)
    pool = torch.full((2 * n_blocks, 2, page, Dp), 7.0, dtype=dtype, device=DEV)
    inv = inv_freq(rot_dims, base) if rot_dims else None
    K.latent_norm_store(None, kvl, None, kw.to(DEV), eps, inv, i32(positions), i32(seq), table, pool, None, kv_rank, rot_dim,
                        rot_dims, half_layout=True)
    kv64 = kvl.double().cpu()
    c = P.rms_norm(kv64[:, :kv_rank], kw.double(), eps)
    turned = P.rotate_halves(kv64[:, kv_rank:], torch.tensor(positions), rot_dims, base)
    for t in range(T):
        pg = int(table[seq[t], positions[t] // page])
        row_k, row_v = pool[pg, 0, positions[t] % page], pool[pg, 1, positions[t] % page]
        close(row_k[:kv_rank], c[t], dtype, "latent in the key row")
        close(row_v[:kv_rank], c[t], dtype, "latent in the value row")
        close(row_k[kv_rank:kv_rank + rot_dim], turned[t], dtype, "turned key part", f32=3e-5)
    q = rnd(T, H * (dim + rot_dim) + 8, seed=4).to(DEV, dtype)[:, :H * (dim + rot_dim)]
    out = torch.full((T, H * Dp), 3.0, dtype=dtype, device=DEV)
    K.latent_query_rot(q, inv, i32(positions), out, H, dim, rot_dim, rot_dims, kv_rank, Dp, half_layout=True)
    want = P.rotate_halves(q.double().cpu().view(T, H, dim + rot_dim)[:, :, dim:], torch.tensor(positions), rot_dims, base)
    close(out.view(T, H, Dp)[:, :, kv_rank:kv_rank + rot_dim], want, dtype, "turned query part", f32=3e-5)
    # both in one launch: the rows and the queries' turned parts
    pool2 = torch.full_like(pool, 7.0)
    out2 = torch.full((T, H * Dp), 3.0, dtype=dtype, device=DEV)
    K.latent_norm_store(None, kvl, None, kw.to(DEV), eps, inv, i32(positions), i32(seq), table, pool2, None, kv_rank, rot_dim,
                        rot_dims, half_layout=True, queries=(q, out2, H, dim))
    used = sorted({int(table[seq[t], positions[t] // page]) for t in range(T)})
    assert torch.equal(pool2[used], pool[used]) and torch.equal(out2, out)


# ----------------------------------------------------------------------------- window with kept first tokens
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window,keep,page", [(40, 4, 16), (5, 1, 16), (17, 20, 16), (24, 3, 64), (64, 0, 16), (33, 70, 16), (1, 2, 16)])
def test_window_with_kept_first_tokens_and_one_more_in_the_denominator(dtype, window, keep, page):
    """A sequence of 300 keys in pages that are not in order, queries at the first positions, around the edges of
    the window and of the kept tokens, at page borders and at the end.  Key 0 (kept), the first key outside the
    kept ones and the keys just inside and just outside the window are loud: one of them wrongly seen or lost
    changes the result by far more than the tolerance.  Pages that the window has passed point to the spare
    page, as the cache manager leaves them."""
    H, G, d, n, scale = 4, 2, 16, 300, 0.3
    keys, vals = rnd(n, G, d, seed=1), rnd(n, G, d, seed=2)
    qpos = sorted({0, 1, 2, keep, keep + 1, window - 1, window, window + 1, window + keep, 63, 64, 65, 150, 298, 299} - {-1})
    qpos = [p for p in qpos if 0 <= p < n]
    q = rnd(len(qpos), H, d, seed=3)
    for t, p in enumerate(qpos):     # every query shouts at four keys: two that it must see and two that it must not
        for j, amp in ((0, 6.0), (keep, 6.0), (p - window + 1, 6.0), (p - window, 6.0)):
            if 0 <= j <= p:
                keys[j, :, 3] = 4.0
        q[t, :, 3] = 3.0
    n_blocks = (n + page - 1) // page
    table = torch.randperm(n_blocks, generator=torch.Generator().manual_seed(5)).to(torch.int32)
    pool = torch.full((n_blocks + 1, 2, page, G * d), 9.0, dtype=dtype, device=DEV)   # the spare page holds no zeros
    for j in range(n):
        pool[int(table[j // page]), 0, j % page] = keys[j].reshape(-1).to(dtype)
        pool[int(table[j // page]), 1, j % page] = vals[j].reshape(-1).to(dtype)
    sink = torch.zeros(H, dtype=torch.float32, device=DEV)
    mask = P.window_mask(n, window, keep)
    k_h = keys.double().repeat_interleave(H // G, dim=1)
    v_h = vals.double().repeat_interleave(H // G, dim=1)
    for t, p in enumerate(qpos):
        s = torch.einsum("hd,jhd->hj", q[t].double(), k_h[:p + 1]) * scale
        s = s.masked_fill(~mask[p, :p + 1][None, :], -math.inf)
        e = torch.exp(s)
        want = torch.einsum("hj,jhd->hd", e / (1.0 + e.sum(dim=1, keepdim=True)), v_h[:p + 1])
        # block-table row as the cache manager leaves it: pages between the kept ones and the window are gone
        row = table.clone()
        first_needed = max(0, p - window + 1) // page
        kept_blocks = (keep + page - 1) // page
        row[kept_blocks:max(kept_blocks, first_needed)] = n_blocks
        out = torch.empty(1, H * d, dtype=dtype, device=DEV)
        K.paged_attention(q[t].reshape(1, -1).to(DEV, dtype), pool, row.view(1, -1).to(DEV), i32([p]), i32([0]), out, H, G, d,
                          scale, window=window, sink=sink, keep_first=keep)
        close(out.view(H, d), want, dtype, f"query at {p}", f32=3e-5)


@pytest.mark.parametrize("d,window,keep", [(64, 96, 4), (128, 200, 70), (64, 64, 1), (32, 40, 5)])
def test_kept_first_tokens_on_the_tensor_core_kernels(d, window, keep):
    """bfloat16, pages of 64: a portion of 300 tokens at positions 400..699 through the tcgen05 kernel (head sizes
    64 and 128) and the mma.sync kernel, and the last token alone through the decode kernels; the window is attended
    by the tensor-core kernel, the kept first keys that it has left are added by the merge launch.  Key 0 and
    the keys at both edges of the first row's window are loud."""
    H, G, n, page, scale, dtype = 4, 2, 700, 64, 0.25, torch.bfloat16
    keys, vals = rnd(n, G, d, seed=1), rnd(n, G, d, seed=2)
    t0 = 400
    T = n - t0
    q = rnd(T, H, d, seed=3)
    keys[[0, keep - 1, keep, t0 - window, t0 - window + 1], :, 3] = 4.0
    q[:, :, 3] = 2.0
    n_blocks = (n + page - 1) // page
    table = torch.randperm(n_blocks, generator=torch.Generator().manual_seed(5)).to(torch.int32)
    pool = torch.full((n_blocks + 1, 2, page, G * d), 9.0, dtype=dtype, device=DEV)
    for j in range(n):
        pool[int(table[j // page]), 0, j % page] = keys[j].reshape(-1).to(dtype)
        pool[int(table[j // page]), 1, j % page] = vals[j].reshape(-1).to(dtype)
    sink = torch.zeros(H, dtype=torch.float32, device=DEV)
    mask = P.window_mask(n, window, keep)
    k_h, v_h = keys.double().repeat_interleave(H // G, dim=1), vals.double().repeat_interleave(H // G, dim=1)
    want = torch.zeros(T, H, d, dtype=torch.float64)
    for t in range(T):
        p = t0 + t
        sc = torch.einsum("hd,jhd->hj", q[t].double(), k_h[:p + 1]) * scale
        sc = sc.masked_fill(~mask[p, :p + 1][None, :], -math.inf)
        mx = sc.max(dim=1, keepdim=True).values.clamp(min=0.0)
        e = torch.exp(sc - mx)
        want[t] = torch.einsum("hj,jhd->hd", e / (torch.exp(-mx) + e.sum(dim=1, keepdim=True)), v_h[:p + 1])
    kept_blocks = (keep + page - 1) // page

    def row_for(first_pos):     # pages between the kept ones and the window of the step's first token are gone
        row = table.clone()
        row[kept_blocks:max(kept_blocks, max(0, first_pos - window + 1) // page)] = n_blocks
        return row.view(1, -1).to(DEV)

    qd = q.reshape(T, H * d).to(DEV, dtype)
    positions, seq_of, cu = i32(list(range(t0, n))), i32([0] * T), i32([0, T])
    counter = torch.zeros(64, dtype=torch.int32, device=DEV)
    ran = 0
    if K.attention_tc_supported(H, G, d, page):
        out, lse = torch.empty(T, H * d, dtype=dtype, device=DEV), torch.empty(T, H, 2, dtype=torch.float32, device=DEV)
        K.attention_tc(qd, pool, row_for(t0), positions, cu, [T], out, H, G, d, scale, window=window, sink=sink,
                       keep_first=keep, lse=lse, seq_of=seq_of, split_counter=counter)
        close(out.view(T, H, d), want, dtype, "tcgen05 prompt kernel")
        ran += 1
    if K.flash_supported(H, G, d):
        out, lse = torch.empty(T, H * d, dtype=dtype, device=DEV), torch.empty(T, H, 2, dtype=torch.float32, device=DEV)
        K.paged_attention(qd, pool, row_for(t0), positions, seq_of, out, H, G, d, scale, window=window, cu_seqlens=cu,
                          new_lens=[T], sink=sink, keep_first=keep, lse=lse, split_counter=counter)
        close(out.view(T, H, d), want, dtype, "mma.sync prompt kernel")
        ran += 1
    if K.flash_decode_supported(H, G, d):
        out, lse = torch.empty(1, H * d, dtype=dtype, device=DEV), torch.empty(1, H, 2, dtype=torch.float32, device=DEV)
        K.flash_decode_attention(qd[T - 1:], None, None, 1.0, 1.0, 1.0, None, pool, row_for(n - 1), positions[T - 1:], out, H, G,
                                 d, scale, window=window, sink=sink, keep_first=keep, lse=lse, seq_of=i32([0]),
                                 split_counter=counter)
        close(out.view(1, H, d), want[T - 1:], dtype, "decode kernel")
        ran += 1
    assert ran >= 2
    # the same without the scratch: the float kernel walks both key ranges itself
    out = torch.empty(T, H * d, dtype=dtype, device=DEV)
    K.paged_attention(qd, pool, row_for(t0), positions, seq_of, out, H, G, d, scale, window=window, sink=sink, keep_first=keep)
    close(out.view(T, H, d), want, dtype, "float kernel")
