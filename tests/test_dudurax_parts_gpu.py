"""Every mechanism of Dudurax alone on the GPU against the plain functions, at sizes of its own: the pair embedding,
the post-norm on a 32-bit stream, gated linear attention through its state slots, latent attention through its pages
(windows inside, at and across page edges), the router, the experts and the dense feed-forward.  Requests run in
portions of many sizes beside one another; slots and pages are freed and used again (freed memory is NaN)."""
import pytest
import torch

from plain import dudurax_plain as P
from test_parts_gpu import cache_for, give_weights, runtime, step_in_portions

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 3e-5, torch.bfloat16: 3e-2}
CUTS = [[37, 0, 9], [5, 20, 1], [1, 1, 1], [2, 3, 1], [64, 2, 1], [1, 30, 2], [200, 200, 200]]
LENGTHS = [130, 61, 40]


def close(got, want, dtype, tol=None):
    got, want = got.double().cpu(), want.double().cpu()
    assert got.shape == want.shape, (got.shape, want.shape)
    assert torch.isfinite(got).all()
    err = float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))
    assert err <= (tol or TOL[dtype]), f"error {err:.3g}"


def inputs(lengths, width, dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(n, width, generator=g).to(dtype) for n in lengths]


def rows_of(xs, spans):
    return torch.cat([xs[r][lo:hi] for r, lo, hi in spans]).cuda()


def f64(stored):
    return {k: v.double() for k, v in stored.items()}


# --------------------------------------------------------------------------- pair embedding and the 32-bit stream
@pytest.mark.parametrize("dtype", DTYPES)
def test_pair_embedding_carries_the_previous_token_across_portions(dtype):
    from logssms_b200.engine import StepEntry
    from logssms_b200.parts import PairEmbedding
    emb = PairEmbedding(50, 24, 3.0, buckets=11, mul_prev=1000003, mul_cur=7)
    w = f64(give_weights(emb, dtype))
    cache, planner = cache_for([emb.cache_needs()], dtype, max_requests=2)
    g = torch.Generator().manual_seed(3)
    for round_ in range(3):                      # slots are used again: a new request must not see the old one's last token
        ids = [torch.randint(0, 50, (n,), generator=g).tolist() for n in (23, 9)]
        reqs, done, got = [cache.admit(), cache.admit()], [0, 0], [[], []]
        for step in ([5, 1], [1, 1], [2, 0], [15, 7]):
            entries = [StepEntry(reqs[r], ids[r][done[r]:done[r] + n]) for r, n in enumerate(step) if n]
            ctx = planner.plan(entries)
            out = emb.forward(ctx.token_ids, ctx, 0)
            assert out.f32.dtype == torch.float32 and out.act.dtype == dtype
            at = 0
            for r, n in enumerate(step):
                if n:
                    got[r].append(out.f32[at:at + n].cpu())
                    done[r] += n
                    at += n
        for r in range(2):
            want = P.embed(ids[r], None, w["embed"], w["bigram"], 3.0, 11, 1000003, 7)
            close(torch.cat(got[r]), want, torch.float32, 1e-6)        # summed in 32-bit whatever the dtype
            cache.release(reqs[r])


@pytest.mark.parametrize("dtype", DTYPES)
def test_post_norm_of_a_32_bit_stream(dtype):
    from logssms_b200.config.specs import NormSpec
    from logssms_b200.ops import kernels as K
    from logssms_b200.parts import RMSNorm
    norm = RMSNorm(NormSpec(72, 3e-6, param_name=""), perturb_init=True)
    w = f64(give_weights(norm, dtype))[""]
    g = torch.Generator().manual_seed(1)
    x = torch.randn(11, 72, generator=g) * 3
    y, extra = (torch.randn(11, 72, generator=g).to(dtype) for _ in range(2))
    scale = torch.rand(11, generator=g)
    stream = K.StreamRows(x.cuda(), x.to(dtype).cuda())
    out = norm.post(stream, y.cuda(), 2.5)
    want = P.rms_norm(2.5 * x.double() + y.double(), w, 3e-6)
    close(out.f32, want, torch.float32, 2e-6)
    close(out.act, want, dtype)
    out = norm.post(stream, y.cuda(), 1.0, extra=extra.cuda(), row_scale=scale.cuda())
    close(out.f32, P.rms_norm(x.double() + y.double() + scale.double()[:, None] * extra.double(), w, 3e-6), torch.float32, 2e-6)
    (h,), _ = norm.forward(stream, None, want_residual=False)           # the norm in front of the head
    assert h.dtype == dtype
    close(h, P.rms_norm(x.double(), w, 3e-6), dtype)


# --------------------------------------------------------------------------- gated linear attention
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, dim, vdim, tau, rank", [(3, 16, 24, 4.0, 8), (1, 48, 40, 16.0, 4), (2, 128, 80, 1.0, 16),
                                                        (5, 8, 8, 64.0, 2), (1, 160, 33, 2.0, 3), (2, 4, 1, 1.0, 1)])
def test_gated_linear_attention_in_portions(dtype, heads, dim, vdim, tau, rank):
    from logssms_b200.config.specs import GLASpec
    from logssms_b200.parts import GatedLinearAttention
    if vdim == 1 and dtype == torch.bfloat16:
        pytest.skip("a norm over one value is the sign of a sum that rounding may move across zero")
    spec = GLASpec(56, heads, dim, vdim, tau, 1e-5, rank)
    part = GatedLinearAttention(spec, perturb_init=True)
    w = f64(give_weights(part, dtype, seed=heads))
    part.setup(runtime(dtype))
    cache, planner = cache_for([part.cache_needs()], dtype, max_requests=3)
    xs = inputs(LENGTHS, 56, dtype)
    for _ in range(2):                           # twice: the second time on slots that were freed (and poisoned)
        got = step_in_portions(planner, cache, LENGTHS, CUTS, lambda ctx, spans: part.forward(rows_of(xs, spans), ctx, 0))
        for x, y in zip(xs, got):
            close(y, P.gla(x.double(), w, {}, heads=heads, dim=dim, vdim=vdim, tau=tau, eps=1e-5), dtype)


@pytest.mark.parametrize("heads, dim, vdim", [(2, 64, 72), (1, 144, 32)])
def test_a_lone_long_prompt_runs_its_segments_side_by_side(heads, dim, vdim):
    """Few long portions: the chunked form cuts them into segments that run side by side with a pass over their states
    between (bfloat16).  Two requests, cut so that a later portion starts from the state the segments left."""
    from logssms_b200.config.specs import GLASpec
    from logssms_b200.ops import kernels as K
    from logssms_b200.parts import GatedLinearAttention
    dtype = torch.bfloat16
    assert K.gla_segmented_pays(600, 2, heads, vdim)
    part = GatedLinearAttention(GLASpec(56, heads, dim, vdim, 8.0, 1e-5, 4), perturb_init=True)
    w = f64(give_weights(part, dtype, seed=3))
    cache, planner = cache_for([part.cache_needs()], dtype, max_requests=2, max_seq_len=2048)
    lengths = [1100, 700]
    xs = inputs(lengths, 56, dtype, seed=4)
    got = step_in_portions(planner, cache, lengths, [[530, 0], [3, 690], [567, 10]], lambda ctx, spans: part.forward(rows_of(xs, spans), ctx, 0))
    for x, y in zip(xs, got):
        close(y, P.gla(x.double(), w, {}, heads=heads, dim=dim, vdim=vdim, tau=8.0, eps=1e-5), dtype)


def test_gated_linear_attention_remembers_a_token_hundreds_of_steps_back():
    """Decays of nearly one: the first token's key/value pair is still most of the state 600 tokens later, through
    prompt portions and single decoded tokens; a state that is lost or started anew anywhere changes every later row."""
    from logssms_b200.config.specs import GLASpec
    from logssms_b200.parts import GatedLinearAttention
    dtype = torch.float32
    part = GatedLinearAttention(GLASpec(32, 2, 16, 8, 8.0, 1e-5, 2))
    stored = give_weights(part, dtype, seed=5)
    stored["a2.b"] = torch.full_like(stored["a2.b"], 9.0)
    from logssms_b200.weights.loader import check_and_place
    part.bind_tree(check_and_place(part, stored, dtype, "cuda"))
    cache, planner = cache_for([part.cache_needs()], dtype, max_requests=2, max_seq_len=1024)
    g = torch.Generator().manual_seed(2)
    x = torch.randn(640, 32, generator=g) * 0.05
    x[0] *= 400.0                                 # the far token: by far the largest key and value
    cuts = [[300], [1], [1], [2], [250]] + [[1]] * 86
    (got,) = step_in_portions(planner, cache, [640], cuts, lambda ctx, spans: part.forward(rows_of([x], spans), ctx, 0))
    want = P.gla(x.double(), f64(stored), {}, heads=2, dim=16, vdim=8, tau=8.0, eps=1e-5)
    close(got, want, dtype)
    blind = P.gla(x[1:].double(), f64(stored), {}, heads=2, dim=16, vdim=8, tau=8.0, eps=1e-5)
    assert float((want[1:] - blind)[-50:].abs().max() / want.abs().max()) > 0.005     # the far token does matter at the end


# --------------------------------------------------------------------------- latent attention
def latent_part(dtype, heads, nope, rot, rot_dims, vdim, rank, window, seed=0, sharp=6.0, page_size=16, max_seq_len=256):
    from logssms_b200.config.specs import LatentAttentionSpec, RopeSpec
    from logssms_b200.parts import LatentAttention
    from logssms_b200.weights.loader import check_and_place
    rope = RopeSpec(rot, rot_dims, 300.0, 4096) if rot_dims else None
    spec = LatentAttentionSpec(56, heads, nope, rot, vdim, rank, 0.3, window, rope, 1e-5)
    part = LatentAttention(spec, perturb_init=True)
    stored = give_weights(part, dtype, seed=seed)
    stored["q"] = (stored["q"].float() * sharp).to(stored["q"].dtype)     # sharp scores: single keys carry the output
    part.bind_tree(check_and_place(part, stored, dtype, "cuda"))
    part.setup(runtime(dtype, max_seq_len=max_seq_len, page_size=page_size))
    kw = dict(heads=heads, dim=nope, rot_dim=rot, vdim=vdim, kv_rank=rank, scale=0.3, window=window or 10 ** 9, base=300.0,
              eps=1e-5, rot_dims=rot_dims)
    return part, f64(stored), kw


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, nope, rot, rot_dims, vdim, rank, window", [
    (2, 16, 8, 8, 24, 40, 20), (3, 8, 16, 8, 16, 24, 17), (4, 32, 32, 32, 8, 72, 1), (1, 8, 64, 64, 48, 136, 16),
    (5, 24, 4, 0, 12, 33, 15), (6, 16, 16, 16, 16, 64, 400), (2, 8, 8, 4, 8, 16, 33)])
def test_latent_attention_in_portions_with_windows_around_page_edges(dtype, heads, nope, rot, rot_dims, vdim, rank, window):
    # (sharp scores multiply bfloat16's rounding of the scores themselves: the 32-bit run is the sharp one)
    part, w, kw = latent_part(dtype, heads, nope, rot, rot_dims, vdim, rank, window, seed=heads, sharp=6.0 if dtype == torch.float32 else 2.0)
    # so few pages that a window layer must give pages back while its requests still run
    pages = 40 if window > 64 else 3 * (-(-(window - 1 + 64) // 16) + 1)
    cache, planner = cache_for([part.cache_needs()], dtype, num_pages=pages, max_requests=3)
    xs = inputs(LENGTHS, 56, dtype, seed=1)
    for _ in range(2):
        got = step_in_portions(planner, cache, LENGTHS, CUTS, lambda ctx, spans: part.forward(rows_of(xs, spans), ctx, 0))
        for x, y in zip(xs, got):
            close(y, P.latent_attention(x.double(), w, {}, **kw), dtype)


@pytest.mark.parametrize("heads, nope, rot, rank, window", [(16, 16, 16, 64, 70), (5, 8, 16, 32, 33), (20, 8, 32, 288, 40), (2, 16, 16, 96, 1000)])
def test_latent_attention_of_long_portions_shares_key_tiles_between_neighbouring_tokens(heads, nope, rot, rank, window):
    """Portions of hundreds of tokens (bfloat16): the form whose CTAs hold up to 64 (token, head) rows, for 16 and more
    heads (a tile is one token), fewer heads (several tokens per tile, uneven when 64 is no multiple), ranks beyond 256
    (two warps share a row tile), beside a short request, with a window shorter and longer than the portions."""
    dtype = torch.bfloat16
    part, w, kw = latent_part(dtype, heads, nope, rot, rot, 8, rank, window, seed=heads, sharp=2.0, page_size=16, max_seq_len=1024)
    cache, planner = cache_for([part.cache_needs()], dtype, num_pages=120, max_requests=3, max_seq_len=1024)
    lengths = [700, 9, 420]
    xs = inputs(lengths, 56, dtype, seed=2)
    got = step_in_portions(planner, cache, lengths, [[300, 2, 0], [250, 1, 420], [150, 6, 0]], lambda ctx, spans: part.forward(rows_of(xs, spans), ctx, 0))
    for x, y in zip(xs, got):
        close(y, P.latent_attention(x.double(), w, {}, **kw), dtype)


@pytest.mark.parametrize("window", [1, 2, 15, 16, 17, 31, 32, 33, 100])
def test_latent_attention_kernel_sees_exactly_the_window(window):
    """Equal scores everywhere and latents that carry their own position: the output's first column is then the mean
    position of the visible keys, which names the window's first key and its length, in a prompt and for decoded tokens."""
    from logssms_b200.ops import kernels as K
    page, n, H, rank, rot = 16, 70, 2, 8, 4
    c = torch.zeros(6, page, rank)
    order = [3, 0, 5, 1, 4]                                         # the request's pages, out of order
    for j in range(n):
        c[order[j // page], j % page, 0] = float(j)
    kr = torch.zeros(6, page, rot)
    table = torch.tensor([order + [-1]], dtype=torch.int32).cuda()
    pos = torch.arange(n, dtype=torch.int32).cuda()
    req = torch.zeros(n, dtype=torch.int32).cuda()
    qa, qr = torch.zeros(n, H, rank).cuda(), torch.zeros(n, H, rot).cuda()
    out = K.latent_attention(qa, qr, c.cuda(), kr.cuda(), table, req, pos, 1.0, window)
    lo = (torch.arange(n) - window + 1).clamp_min(0)
    want = (lo + torch.arange(n)).double() / 2
    assert torch.allclose(out[:, 0, 0].double().cpu(), want, atol=1e-4) and torch.allclose(out[:, 1, 0].double().cpu(), want, atol=1e-4)
    # listed rows only (decoded tokens beside a prompt portion): the other rows stay as they were
    listed = torch.tensor([69, 16, 0], dtype=torch.int32).cuda()
    out2 = K.latent_attention(qa, qr, c.cuda(), kr.cuda(), table, req, pos, 1.0, window, token_list=listed,
                              out=torch.full((n, H, rank), -7.0).cuda())
    assert torch.allclose(out2[listed.long(), 0, 0].double().cpu(), want[[69, 16, 0]], atol=1e-4)
    assert float(out2[5, 0, 0]) == -7.0


@pytest.mark.parametrize("heads", [4, 16])
@pytest.mark.parametrize("window", [1, 2, 16, 17, 31, 32, 33, 64, 65, 100])
def test_tensor_core_latent_attention_sees_exactly_the_window(window, heads):
    """The tensor-core forms (bfloat16), equal scores everywhere, and a mark in the latents of every `window`-th key: any
    `window` keys in a row hold exactly one mark, so the output's first column is 1 / (keys seen) at every position; a
    window one key too wide would see two marks at some positions, one key too narrow none."""
    import numpy as np
    from logssms_b200.ops import kernels as K
    from logssms_b200.parts.context import token_block_list
    page, n, rank, rot = 16, 150, 32, 16
    order = [3, 0, 9, 5, 1, 4, 8, 2, 7, 6]
    c = torch.zeros(11, page, rank)
    for j in range(0, n, window):
        c[order[j // page], j % page, 0] = 1.0
    c, kr = c.to(torch.bfloat16).cuda(), torch.zeros(11, page, rot, dtype=torch.bfloat16).cuda()
    table = torch.tensor([order], dtype=torch.int32).cuda()
    pos = torch.arange(n, dtype=torch.int32).cuda()
    req = torch.zeros(n, dtype=torch.int32).cuda()
    qa = torch.zeros(n, heads, rank, dtype=torch.bfloat16).cuda()
    qr = torch.zeros(n, heads, rot, dtype=torch.bfloat16).cuda()
    want = 1.0 / torch.minimum(torch.arange(n) + 1, torch.tensor(window)).double()
    outs = {"a tile per token": K.latent_attention_mma(qa, qr, c, kr, table, req, pos, None, 1.0, window),
            "key ranges": K.latent_attention_mma(qa, qr, c, kr, table, req, pos, None, 1.0, window, splits=3)}
    for rows in (32, 64):
        blocks = torch.from_numpy(np.ascontiguousarray(token_block_list([n], K.latent_wide_tokens(heads, rows)))).cuda()
        outs[f"wide, {rows} rows"] = K.latent_attention_wide(qa, qr, c, kr, table, req, pos, blocks, 1.0, window, rows=rows)
    small = torch.from_numpy(np.ascontiguousarray(token_block_list([n], max(1, 16 // heads)))).cuda()
    outs["tokens that share a tile"] = K.latent_attention_mma(qa, qr, c, kr, table, req, pos, small, 1.0, window)
    for name, out in outs.items():
        for h in (0, heads - 1):
            got = out[:, h, 0].double().cpu()
            assert torch.allclose(got, want, rtol=2e-2, atol=1e-4), f"{name}, head {h}: first position off {int(((got - want).abs() > 2e-2 * want).nonzero()[0])}"


# --------------------------------------------------------------------------- feed-forwards
@pytest.mark.parametrize("n, experts, top, groups, keep", [(6, 4, 2, 3, 2), (12, 8, 4, 4, 3), (3, 3, 1, 1, 1), (6, 2, 3, 2, 1),
                                                           (64, 60, 8, 8, 4), (2, 1, 2, 2, 2), (5, 0, 2, 1, 1)])
def test_router_chooses_as_the_plain_one(n, experts, top, groups, keep):
    from logssms_b200.ops import kernels as K
    g = torch.Generator().manual_seed(n)
    h = torch.randn(300, 40, generator=g)
    W = torch.randn(n, 40, generator=g) * 0.3
    corr = torch.randn(n, generator=g) * 0.1 - 0.2                     # most choice scores are negative
    dense, chosen, chosen_w, idw = K.moe_route(h.cuda(), W.cuda(), corr.cuda(), experts, top, groups, keep, 1.7)
    want = P.route(h.double(), W.double(), corr.double(), top=top, groups=groups, keep=keep, scale=1.7)
    # rows whose choice hangs on less than 1e-5 may go either way in 32-bit
    s = torch.softmax(h.double() @ W.double().T, -1) + corr.double()
    gaps = (s[:, :, None] - s[:, None, :]).abs() + torch.eye(n) * 9
    sure = gaps.flatten(1).min(-1).values > 1e-5
    assert sure.sum() > 250
    assert torch.equal((dense.cpu() > 0)[sure], (want > 0)[sure])
    assert torch.allclose(dense.cpu().double()[sure], want[sure], atol=1e-6)
    assert torch.allclose(idw.cpu().double()[sure], want[sure][:, experts:].sum(-1), atol=1e-6)
    picked = torch.zeros(300, n).scatter_(1, chosen.cpu().long(), chosen_w.cpu())
    assert torch.equal(picked, dense.cpu())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("experts, identity, top, groups, keep, limit", [(4, 2, 2, 3, 2, 2.0), (3, 0, 1, 1, 1, 0.5), (2, 4, 3, 2, 1, 1.0)])
def test_routed_feed_forward(dtype, experts, identity, top, groups, keep, limit):
    from logssms_b200.config.specs import RoutedMLPSpec
    from logssms_b200.parts import RoutedMLP
    from logssms_b200.weights.loader import check_and_place
    spec = RoutedMLPSpec(56, 40, experts, identity, top, groups, keep, 1.3, limit)
    part = RoutedMLP(spec)
    stored = give_weights(part, dtype, seed=experts)
    n = experts + identity
    stored["correction"] = (0.25 * torch.randperm(n, generator=torch.Generator().manual_seed(1)).float()).to(stored["correction"].dtype)
    part.bind_tree(check_and_place(part, stored, dtype, "cuda"))
    x = torch.randn(77, 56, generator=torch.Generator().manual_seed(2)).to(dtype)
    out = part.forward(x.cuda())
    if isinstance(out, tuple):
        y, h, idw = out
        got = y.double().cpu() + idw.double().cpu()[:, None] * h.double().cpu()
    else:
        got = out
    want = P.moe_ff(x.double(), f64(stored), experts=experts, identity=identity, top=top, groups=groups, keep=keep, scale=1.3, limit=limit)
    close(got, want, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_dense_feed_forward(dtype):
    from logssms_b200.config.specs import DenseMLPSpec
    from logssms_b200.parts import DenseMLP
    part = DenseMLP(DenseMLPSpec(56, 90))
    w = f64(give_weights(part, dtype))
    x = (3 * torch.randn(41, 56, generator=torch.Generator().manual_seed(2))).to(dtype)
    close(part.forward(x.cuda()), P.dense_ff(x.double(), w), dtype)
