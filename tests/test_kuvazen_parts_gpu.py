"""Every mechanism of Kuvazen alone on the GPU against the plain functions, at sizes of its own: the normed embedding
and the kernels of a pre-norm 32-bit stream (layer norm, channel scales, the token's side input), the minGRU through its
state slots (token by token and in chunks), attention over a window and pooled blocks through its two page groups
(windows and blocks inside, at and across page edges), the sigmoid router with input-weighted experts and the clamped
dense layer.  Requests run in portions of many sizes beside one another; slots and pages are freed and used again
(freed memory is NaN)."""
import pytest
import torch

from plain import kuvazen_plain as P
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


# --------------------------------------------------------------------------- the stream's kernels
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind", ["layernorm", "rmsnorm"])
def test_normed_embedding_starts_a_32_bit_stream(dtype, kind):
    from logssms_b200.config.specs import NormSpec
    from logssms_b200.parts import NormedEmbedding
    emb = NormedEmbedding(50, 36, norm=NormSpec(36, 2e-6, kind=kind, param_name="embed.norm"))
    w = f64(give_weights(emb, dtype))
    ids = torch.tensor([3, 49, 0, 3, 17], dtype=torch.int32)
    out = emb.forward(ids.cuda())
    assert out.f32.dtype == torch.float32 and out.act.dtype == dtype and out.normed_by is None
    norm = P.layer_norm if kind == "layernorm" else P.rms_norm
    close(out.f32, norm(w["embed"][ids.long()], w["embed.norm"], 2e-6), torch.float32, 2e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [72, 600, 2050])
def test_channel_scaled_sum_and_norm_of_a_stream(dtype, width):
    from logssms_b200.ops import kernels as K
    g = torch.Generator().manual_seed(1)
    x = torch.randn(7, width, generator=g) * 3 + 0.7            # a mean that a layer norm must take off
    y = torch.randn(7, width, generator=g).to(dtype)
    ls, w = torch.rand(width, generator=g) + 0.5, torch.rand(width, generator=g) + 0.5
    for kind, norm in (("layernorm", P.layer_norm), ("rmsnorm", P.rms_norm)):
        stream = x.clone().cuda()
        same, h = K.stream_add_norm(stream, y.cuda(), ls.cuda(), w.cuda(), 1e-5, kind, dtype)
        want = x.double() + ls.double() * y.double()
        assert same is stream and h.dtype == dtype
        close(stream, want, torch.float32, 2e-6)                 # the sum is 32-bit whatever the dtype
        close(h, norm(want, w.double(), 1e-5), dtype)
        _, h = K.stream_add_norm(stream, None, None, w.cuda(), 1e-5, kind, dtype)       # the norm alone leaves the stream as it is
        close(stream, want, torch.float32, 2e-6)
        close(h, norm(want, w.double(), 1e-5), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows", [9, 300])          # few rows: one kernel; many (bfloat16): the two small products go to the library
@pytest.mark.parametrize("width, dim, layer, layers", [(72, 6, 0, 3), (264, 1, 2, 3), (96, 24, 1, 2), (1030, 40, 3, 4)])
def test_token_side_input_closes_a_layer(dtype, width, dim, layer, layers, rows):
    from logssms_b200.config.specs import NormSpec, TokenSideSpec
    from logssms_b200.parts import LayerNorm, TokenSideInput
    if dim == 1 and rows > 9 and dtype == torch.bfloat16:
        pytest.skip("one column: the side input is +- a fixed vector, by the sign of one product of rounded rows")
    shared = {}
    spec = TokenSideSpec(width, dim, layer * dim, layers * dim, 31, 1e-5)
    side = TokenSideInput(spec, perturb_init=True, shared=shared)
    table = shared["model_parts"]["side."]
    assert TokenSideInput(TokenSideSpec(width, dim, 0, layers * dim, 31, 1e-5), shared=shared).shared_table is table   # one table for all layers
    w = f64(give_weights(side, dtype, seed=layer))
    tw = f64(give_weights(table, dtype, seed=9))["embed"]
    nxt = LayerNorm(NormSpec(width, 1e-6, kind="layernorm", param_name=""), perturb_init=True)
    nw = f64(give_weights(nxt, dtype, seed=4))[""]
    g = torch.Generator().manual_seed(2)
    x = torch.randn(rows, width, generator=g) * 2
    y = torch.randn(rows, width, generator=g).to(dtype)
    ls = torch.rand(width, generator=g) + 0.5
    ids = torch.randint(0, 31, (rows,), generator=g)
    joined = x.double() + ls.double() * y.double()
    want = P.side_input(joined, ids.tolist(), layer, tw, w, dim, 1e-5)
    assert float((want - joined).abs().max()) > 0.1              # the side input does move the stream
    stream = x.clone().cuda()
    _, h = side.close(stream, y.cuda(), ls.cuda(), ids.int().cuda(), nxt, dtype)
    close(stream, want, dtype, 2e-5 if dtype == torch.float32 else 2e-2)    # (bfloat16: the two small matrices are rounded)
    close(h, P.layer_norm(want, nw, 1e-6), dtype)
    stream = x.clone().cuda()
    _, none = side.close(stream, None, None, ids.int().cuda(), None, dtype)     # a layer without a feed-forward, the last layer
    assert none is None
    close(stream, P.side_input(x.double(), ids.tolist(), layer, tw, w, dim, 1e-5), dtype, 2e-5 if dtype == torch.float32 else 2e-2)


# --------------------------------------------------------------------------- minGRU
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [1, 40, 130, 520])
def test_mingru_in_portions(dtype, width):
    from logssms_b200.config.specs import MinGRUSpec
    from logssms_b200.parts import MinGRU
    part = MinGRU(MinGRUSpec(56, width), perturb_init=True)
    w = f64(give_weights(part, dtype, seed=width))
    cache, planner = cache_for([part.cache_needs()], dtype, max_requests=3)
    xs = inputs(LENGTHS, 56, dtype)
    for _ in range(2):                           # twice: the second time on slots that were freed (and poisoned)
        got = step_in_portions(planner, cache, LENGTHS, CUTS, lambda ctx, spans: part.forward(rows_of(xs, spans), ctx, 0))
        for x, y in zip(xs, got):
            close(y, P.mingru(x.double(), w, {}), dtype)


def test_mingru_chunks_of_long_portions_carry_the_state_from_chunk_to_chunk_and_step_to_step():
    """Portions of hundreds of tokens run in chunks side by side; cuts in the middle of a chunk, a short request beside."""
    from logssms_b200.config.specs import MinGRUSpec
    from logssms_b200.parts import MinGRU
    for dtype in DTYPES:
        part = MinGRU(MinGRUSpec(56, 200), perturb_init=True)
        w = f64(give_weights(part, dtype, seed=3))
        cache, planner = cache_for([part.cache_needs()], dtype, max_requests=3, max_seq_len=2048)
        lengths = [1100, 7, 700]
        xs = inputs(lengths, 56, dtype, seed=4)
        got = step_in_portions(planner, cache, lengths, [[530, 2, 0], [3, 1, 690], [567, 4, 10]],
                               lambda ctx, spans: part.forward(rows_of(xs, spans), ctx, 0))
        for x, y in zip(xs, got):
            close(y, P.mingru(x.double(), w, {}), dtype)


def test_mingru_remembers_a_token_hundreds_of_steps_back():
    """Update gates of nearly zero: the first token's candidate is still most of the state 600 tokens later, through
    prompt portions and single decoded tokens; a state that is lost or started anew anywhere changes every later row."""
    from logssms_b200.config.specs import MinGRUSpec
    from logssms_b200.parts import MinGRU
    from logssms_b200.weights.loader import check_and_place
    dtype = torch.float32
    part = MinGRU(MinGRUSpec(32, 24))
    stored = give_weights(part, dtype, seed=5)
    stored["z.b"] = torch.full_like(stored["z.b"], -7.0)
    part.bind_tree(check_and_place(part, stored, dtype, "cuda"))
    cache, planner = cache_for([part.cache_needs()], dtype, max_requests=2, max_seq_len=1024)
    g = torch.Generator().manual_seed(2)
    x = torch.randn(640, 32, generator=g) * 0.05
    x[0] *= 400.0                                 # the far token: an open gate and by far the largest candidate
    cuts = [[300], [1], [1], [2], [250]] + [[1]] * 86
    (got,) = step_in_portions(planner, cache, [640], cuts, lambda ctx, spans: part.forward(rows_of([x], spans), ctx, 0))
    want = P.mingru(x.double(), f64(stored), {})
    close(got, want, dtype)
    blind = P.mingru(x[1:].double(), f64(stored), {})
    assert float((want[1:] - blind)[-50:].abs().max() / want[-50:].abs().max()) > 0.05     # the far token does matter at the end


# --------------------------------------------------------------------------- attention over a window and pooled blocks
def attention_part(dtype, heads, kv_heads, dim, vdim, rot_dims, window, pool, seed=0, sharp=6.0, page_size=16, max_seq_len=256):
    from logssms_b200.config.specs import PooledWindowAttentionSpec, RopeSpec
    from logssms_b200.parts import PooledWindowAttention
    from logssms_b200.weights.loader import check_and_place
    rope = RopeSpec(dim, rot_dims, 300.0, 4096) if rot_dims else None
    spec = PooledWindowAttentionSpec(56, heads, kv_heads, dim, vdim, 0.3, window, pool, rope, RopeSpec(vdim, vdim, 300.0, 4096))
    part = PooledWindowAttention(spec, perturb_init=True)
    stored = give_weights(part, dtype, seed=seed)
    stored["q"] = (stored["q"].float() * sharp).to(stored["q"].dtype)     # sharp scores: single keys and blocks carry the output
    part.bind_tree(check_and_place(part, stored, dtype, "cuda"))
    part.setup(runtime(dtype, max_seq_len=max_seq_len, page_size=page_size))
    kw = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=0.3, window=window, pool=pool, base=300.0, rot_dims=rot_dims)
    return part, f64(stored), kw


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv_heads, dim, vdim, rot_dims, window, pool", [
    (6, 2, 16, 24, 8, 20, 5), (2, 2, 24, 8, 24, 17, 16), (4, 1, 8, 136, 4, 7, 24), (3, 3, 32, 16, 0, 1, 3),
    (2, 1, 16, 12, 16, 40, 1), (5, 5, 8, 6, 8, 33, 7), (8, 2, 64, 80, 64, 16, 16), (1, 1, 2, 2, 2, 400, 2)])
def test_pooled_window_attention_in_portions_with_edges_around_page_borders(dtype, heads, kv_heads, dim, vdim, rot_dims, window, pool):
    # (sharp scores multiply bfloat16's rounding of the scores themselves: the 32-bit run is the sharp one)
    part, w, kw = attention_part(dtype, heads, kv_heads, dim, vdim, rot_dims, window, pool, seed=heads,
                                 sharp=6.0 if dtype == torch.float32 else 2.0)
    # so few pages that the token group must give pages back while its requests still run
    keep = max(window, pool)
    pages = 40 if keep > 64 else 3 * (-(-(keep - 1 + 64) // 16) + 1)
    cache, planner = cache_for([part.cache_needs()], dtype, num_pages=pages, max_requests=3)
    xs = inputs(LENGTHS, 56, dtype, seed=1)
    for _ in range(2):
        got = step_in_portions(planner, cache, LENGTHS, CUTS, lambda ctx, spans: part.forward(rows_of(xs, spans), ctx, 0))
        for x, y in zip(xs, got):
            close(y, P.pooled_window_attention(x.double(), w, {}, **kw), dtype)


@pytest.mark.parametrize("heads, kv_heads, dim, vdim, window, pool", [(16, 4, 64, 64, 70, 8), (5, 5, 16, 24, 33, 5), (12, 2, 32, 136, 40, 16),
                                                                      (2, 1, 128, 32, 300, 64)])
def test_pooled_window_attention_of_long_portions(heads, kv_heads, dim, vdim, window, pool):
    """Portions of hundreds of tokens (both dtypes) beside a short request, windows shorter and longer than a tile of
    queries, cuts that leave a block half filled between two steps."""
    for dtype in DTYPES:
        part, w, kw = attention_part(dtype, heads, kv_heads, dim, vdim, dim, window, pool, seed=heads, sharp=4.0 if dtype == torch.float32 else 2.0,
                                     page_size=16, max_seq_len=1024)
        cache, planner = cache_for([part.cache_needs()], dtype, num_pages=120, max_requests=3, max_seq_len=1024)
        lengths = [700, 9, 420]
        xs = inputs(lengths, 56, dtype, seed=2)
        got = step_in_portions(planner, cache, lengths, [[301, 2, 0], [250, 1, 420], [149, 6, 0]],
                               lambda ctx, spans: part.forward(rows_of(xs, spans), ctx, 0))
        for x, y in zip(xs, got):
            # (float32: the angle position * frequency is a 32-bit product in the engine, exact to half a unit in its last
            # place, which at position 700 is 3e-5 radians; the plain functions compute it in 64-bit)
            close(y, P.pooled_window_attention(x.double(), w, {}, **kw), dtype, 2e-4 if dtype == torch.float32 else None)


def marked_attention(window, pool, n, cuts, dtype=torch.float32):
    """One head whose output NAMES what it saw: equal scores (zero queries), values that carry their position in two
    columns (1 and the position), no rotation of the values' meaning lost because the test turns the output forward
    again.  Returns per position (sum of weights' count, mean position seen)."""
    from logssms_b200.config.specs import PooledWindowAttentionSpec, RopeSpec
    from logssms_b200.parts import PooledWindowAttention
    from logssms_b200.weights.loader import check_and_place
    width = 4
    spec = PooledWindowAttentionSpec(width, 1, 1, 2, 2, 1.0, window, pool, None, RopeSpec(2, 2, 50.0, 4096))
    part = PooledWindowAttention(spec)
    stored = give_weights(part, dtype)
    stored["q"], stored["k"] = torch.zeros(2, width), torch.zeros(2, width)
    stored["v"] = torch.tensor([[1.0, 0, 0, 0], [0, 1.0, 0, 0]])
    stored["o"] = torch.tensor([[1.0, 0], [0, 1.0], [0, 0], [0, 0]])
    part.bind_tree(check_and_place(part, {k: v.to(dtype) for k, v in stored.items()}, dtype, "cuda"))
    part.setup(runtime(dtype, max_seq_len=512, page_size=16))
    cache, planner = cache_for([part.cache_needs()], dtype, num_pages=3 * (-(-(max(window, pool) + 63) // 16) + 1), max_requests=2, max_seq_len=512)
    x = torch.zeros(n, width)
    x[:, 0] = 1.0
    x[:, 1] = torch.arange(n, dtype=torch.float32) / 64.0          # exact in bfloat16 up to 512 positions
    (got,) = step_in_portions(planner, cache, [n], cuts, lambda ctx, spans: part.forward(rows_of([x.to(dtype)], spans), ctx, 0))
    out = got[:, :2].double()
    return torch.stack([P.turn_pairs(out[i], i, 50.0, 2) for i in range(n)])       # forward again: the mean of the turned values


@pytest.mark.parametrize("window, pool", [(6, 4), (16, 16), (17, 5), (1, 3), (5, 9), (48, 1), (33, 32)])
def test_the_output_names_every_token_and_block_that_was_seen(window, pool):
    """Exactly the window's tokens and the blocks wholly behind it, in prompts and in decoded tokens, across pages of 16:
    compared position by position with the sum of the turned values that the rule allows."""
    n = 150
    for cuts in ([[150]], [[70], [3]] + [[1]] * 77, [[2], [2], [31], [1], [1], [64], [49]]):
        got = marked_attention(window, pool, n, cuts)
        for i in range(n):
            first, blocks = max(0, i - window + 1), max(0, (i - window + 1) // pool)
            turned = lambda j: P.turn_pairs(torch.tensor([1.0, j / 64.0], dtype=torch.float64), j, 50.0, 2)
            seen = [turned(j) for j in range(first, i + 1)]
            seen += [torch.stack([turned(j) for j in range(b * pool, (b + 1) * pool)]).mean(0) for b in range(blocks)]
            want = torch.stack(seen).mean(0)
            assert float((got[i] - want).abs().max()) < 2e-5, f"window {window}, pool {pool}, cuts {cuts[0]}: position {i} saw something else"
            # one key more or fewer moves the mean by about 1 / (number seen): far above the tolerance
            if blocks:
                fewer = torch.stack(seen[:-1]).mean(0)
                assert float((fewer - want).abs().max()) > 1e-4


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window, pool", [(6, 4), (16, 16), (17, 5), (1, 3), (5, 9), (48, 1), (33, 32), (64, 8), (70, 64)])
def test_a_histogram_of_what_was_seen_on_the_tensor_cores_and_off(dtype, window, pool):
    """Equal scores (zero queries) and values that are unit vectors by the run of 16 positions a token lies in (modulo
    8), unrotated: a head's output is the histogram of the runs it saw (a block counts as one key with its own
    histogram), exact in bfloat16 up to the output's rounding.  One key or block more or fewer moves an entry by
    1 / (keys seen), far more than that rounding.  Long portions of a bfloat16 engine run on the tensor cores, the
    others and the decoded tokens a warp per row."""
    from logssms_b200.config.specs import PooledWindowAttentionSpec
    from logssms_b200.parts import PooledWindowAttention
    from logssms_b200.weights.loader import check_and_place
    width, n = 16, 300
    spec = PooledWindowAttentionSpec(width, 2, 1, 16, 8, 1.0, window, pool, None, None)
    part = PooledWindowAttention(spec)
    stored = give_weights(part, dtype)
    stored["q"], stored["k"] = torch.zeros(32, width), torch.zeros(16, width)
    stored["v"] = torch.eye(8, width)
    stored["o"] = torch.cat([torch.eye(8), torch.zeros(8, 8)]).repeat(1, 2) * 0.5          # the mean of the two heads
    stored = {k: v.to(dtype) for k, v in stored.items()}
    part.bind_tree(check_and_place(part, stored, dtype, "cuda"))
    part.setup(runtime(dtype, max_seq_len=512, page_size=16))
    x = torch.zeros(n, width)
    mark = lambda j: (j // 16) % 8
    x[torch.arange(n), (torch.arange(n) // 16) % 8] = 1.0
    pages = 3 * (-(-(max(window, pool) + 140) // 16) + 1)
    for cuts in ([[300]], [[131], [3], [70]] + [[1]] * 96, [[2], [2], [31], [1], [1], [64], [129], [70]]):
        cache, planner = cache_for([part.cache_needs()], dtype, num_pages=pages, max_requests=2, max_seq_len=512)
        (got,) = step_in_portions(planner, cache, [n], cuts, lambda ctx, spans: part.forward(rows_of([x.to(dtype)], spans), ctx, 0))
        want = torch.zeros(n, 8, dtype=torch.float64)
        for i in range(n):
            first, blocks = max(0, i - window + 1), max(0, (i - window + 1) // pool)
            for j in range(first, i + 1):
                want[i, mark(j)] += 1.0
            for b in range(blocks):
                for j in range(b * pool, (b + 1) * pool):
                    want[i, mark(j)] += 1.0 / pool
            want[i] /= (i + 1 - first + blocks)
        allowed = 1e-5 if dtype == torch.float32 else 0.006 * want + 2e-4        # (bfloat16: the output is rounded twice)
        err = ((got[:, :8].double() - want).abs() / allowed).max(-1).values
        assert float(err.max()) <= 1.0, \
            f"window {window}, pool {pool}, cuts {cuts[0]}: position {int(err.argmax())} saw something else ({float(err.max()):.3g} of what rounding allows)"


def test_a_far_block_among_hundreds_still_carries_the_output():
    """One token far behind the window has by far the largest key: its BLOCK wins the softmax 500 positions later."""
    from logssms_b200.weights.loader import check_and_place
    dtype = torch.float32
    part, w, kw = attention_part(dtype, 2, 1, 16, 8, 16, 24, 8, seed=3, sharp=1.0, max_seq_len=1024)
    cache, planner = cache_for([part.cache_needs()], dtype, num_pages=40, max_requests=2, max_seq_len=1024)
    g = torch.Generator().manual_seed(6)
    x = torch.randn(600, 56, generator=g) * 0.3
    x[43] *= 40.0
    cuts = [[100], [2], [400]] + [[1]] * 98
    (got,) = step_in_portions(planner, cache, [600], cuts, lambda ctx, spans: part.forward(rows_of([x], spans), ctx, 0))
    want = P.pooled_window_attention(x.double(), w, {}, **kw)
    close(got, want, dtype)
    blind = x.clone()
    blind[43] = 0.0
    other = P.pooled_window_attention(blind.double(), w, {}, **kw)
    assert float((want - other)[-50:].abs().max() / want[-50:].abs().max()) > 0.05


# --------------------------------------------------------------------------- feed-forwards
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows", [5, 100])
@pytest.mark.parametrize("ff, limit", [(96, 1.0), (50, 0.25), (8, 7.0)])
def test_clamped_dense_layer(dtype, rows, ff, limit):
    from logssms_b200.config.specs import ClampedGLUSpec
    from logssms_b200.parts import ClampedGLU
    part = ClampedGLU(ClampedGLUSpec(56, ff, limit))
    w = f64(give_weights(part, dtype, seed=ff))
    g = torch.Generator().manual_seed(1)
    x = (torch.randn(rows, 56, generator=g) * 2).to(dtype)
    close(part.forward(x.cuda()), P.dense_ff(x.double(), w, limit), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("experts, top, ff", [(3, 2, 24), (16, 1, 96), (1, 1, 8), (8, 3, 16), (40, 4, 10)])
def test_sigmoid_router_with_input_weighted_experts(dtype, experts, top, ff):
    from logssms_b200.config.specs import RoutedMLPSpec
    from logssms_b200.parts import RoutedMLP
    from logssms_b200.weights.loader import check_and_place
    spec = RoutedMLPSpec(56, ff, experts, 0, top, 1, 1, 1.0, 0.0, score="sigmoid", expert="silu", weigh="input", correction=False)
    part = RoutedMLP(spec)
    stored = give_weights(part, dtype, seed=experts)
    g = torch.Generator().manual_seed(2)
    # a router whose scores are spaced: no choice is a close call for a bfloat16 engine
    direction = torch.randn(56, generator=g) * 56 ** -0.5
    stored["router"] = ((torch.randperm(experts, generator=g).float() - (experts - 1) / 2)[:, None] * 0.8 * direction[None, :]).to(stored["router"].dtype)
    part.bind_tree(check_and_place(part, stored, dtype, "cuda"))
    for rows in (7, 90):
        x = torch.randn(rows, 56, generator=g).to(dtype)
        close(part.forward(x.cuda()), P.moe_ff(x.double(), f64(stored), experts=experts, top=top), dtype)
