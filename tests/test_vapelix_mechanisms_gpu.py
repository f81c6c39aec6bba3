"""Each mechanism of the Vapelix parts alone, built through the registries and run through the
engine's step machinery, against the plain function in ``plain_vapelix``: latent attention in
portions and single tokens at sizes that are no multiple of anything, with far keys, keys at page
borders and the first tokens made decisive; the router and the routed experts; the gated
feed-forward with the tanh form of gelu; the token's side input.  (The block of two branches is
compared run by run in ``test_vapelix_gpu``.)"""

import math

import pytest
import torch

import plain_vapelix as pv
from gpu_helpers import PartHarness, assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def _spec():
    from distengine_b200.config.model import PartSpec
    return PartSpec


def _gen(seed):
    return torch.Generator().manual_seed(seed)


def _act(dtype):
    return None if dtype == torch.float32 else torch.bfloat16


# ----------------------------------------------------------------------------- latent attention
def _latent(dtype, width, m, eps):
    from distengine_b200.parts import build_mixer
    rot = m["rot"]
    scaling = rot.get("scaling")
    spec = _spec().of("latent_attention", width=width, heads=m["heads"], key_dim=m["dim"],
                      rotary_dim=m["rot_dim"], value_dim=m["vdim"], q_rank=m["q_rank"],
                      kv_rank=m["kv_rank"], scale=m["scale"], theta=rot["base"], eps=eps,
                      scaling=None if scaling is None else tuple(
                          scaling[k] for k in ("factor", "original", "fast", "slow")))
    return build_mixer(spec, dtype, torch.device(DEV))


def _latent_weights(width, m, seed, spread=1.0):
    g = _gen(seed)
    H, per = m["heads"], m["dim"] + m["rot_dim"]
    shapes = {"dq": (m["q_rank"], width), "uq": (H * per, m["q_rank"]),
              "dkv": (m["kv_rank"] + m["rot_dim"], width), "uk": (H * m["dim"], m["kv_rank"]),
              "uv": (H * m["vdim"], m["kv_rank"]), "g": (H * m["vdim"], width),
              "o": (width, H * m["vdim"])}
    w = {k: (torch.randn(s, generator=g) * spread / math.sqrt(s[1])).to(torch.bfloat16).float()
         for k, s in shapes.items()}
    w["dq.norm"] = (torch.rand(m["q_rank"], generator=g) + 0.5).to(torch.bfloat16).float()
    w["dkv.norm"] = (torch.rand(m["kv_rank"], generator=g) + 0.5).to(torch.bfloat16).float()
    return w


def _mixer_sizes(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base=10000.0, scaling=None):
    rot = {"base": base, "dims": rot_dim}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank,
            "kv_rank": kv_rank, "scale": scale, "rot": rot}


def _run_in_portions(mixer, h, xs, portions):
    """Feeds the requests' rows in the given portions ({request: count} per step); returns what
    the mixer gave for every request's rows in order."""
    fed = {rid: 0 for rid in xs}
    got = {rid: [] for rid in xs}
    for step in portions:
        entries = [(rid, n) for rid, n in step if n]
        x = torch.cat([xs[rid][fed[rid]: fed[rid] + n] for rid, n in entries]).to(DEV)
        out = h.run(entries, lambda ctx, b: mixer.forward(x, ctx, b[0]).clone()).float().cpu()
        at = 0
        for rid, n in entries:
            got[rid].append(out[at: at + n])
            at += n
            fed[rid] += n
    assert all(fed[rid] == xs[rid].shape[0] for rid in xs)
    return {rid: torch.cat(parts) for rid, parts in got.items()}


SIZES = [
    # heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base, scaling; page
    ((3, 6, 2, 5, 9, 7, 0.4, 100.0, None), 16),                       # rows of 9: no 16-byte piece
    ((2, 10, 6, 3, 14, 18, 0.3, 10000.0, (4.0, 64, 8.0, 1.0)), 4),
    ((8, 16, 8, 16, 24, 24, 0.25, 50000.0, (8.0, 128, 16.0, 1.0)), 8),  # the one-launch decode
    ((12, 8, 16, 8, 16, 16, 0.2, 1000000.0, (16.0, 48, 32.0, 1.0)), 16),  # more than 8 heads
    ((1, 32, 4, 1, 8, 60, 0.15, 500.0, (2.0, 32, 4.0, 2.0)), 8),      # one head, values of size 1
    ((5, 4, 32, 24, 40, 8, 0.3, 20.0, None), 32),                     # mostly rotated
    # cached rows of 64 and of 128 features: in bfloat16 the prompt portions take the tcgen05
    # attention kernel
    ((6, 24, 16, 20, 32, 48, 0.2, 10000.0, (8.0, 64, 32.0, 1.0)), 16),
    ((4, 32, 32, 16, 24, 96, 0.15, 1000000.0, (4.0, 128, 16.0, 2.0)), 16),
    ((10, 16, 16, 24, 40, 48, 0.2, 10000.0, None), 8),
    ((3, 40, 48, 8, 16, 208, 0.1, 500.0, None), 16),                  # a row of 256 features
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes,page", SIZES)
def test_latent_attention_in_portions(dtype, sizes, page):
    """Two requests in unequal portions beside single tokens, then steps of single tokens only,
    against the plain function over each whole sequence."""
    width, eps = 44, 1e-5
    m = _mixer_sizes(*sizes)
    mixer = _latent(dtype, width, m, eps)
    w = _latent_weights(width, m, sizes[0] * 7 + sizes[5], spread=1.5)
    assert {k: v[0] for k, v in mixer.tensors().items()} == {k: tuple(v.shape) for k, v in w.items()}
    mixer.load(w)
    spec = mixer.cache_spec()
    row = m["kv_rank"] + m["rot_dim"]
    assert (spec.kv_heads, spec.head_dim, spec.v_dim) == (1, row, m["kv_rank"])
    # which kernels the prompt portions take
    tensor = dtype == torch.bfloat16 and row % 16 == 0 and row <= 256
    assert (mixer.launcher is not None) == tensor
    if tensor:
        assert (mixer.launcher.shapes[0].code == 2) == (row in (64, 128))
    g = _gen(5)
    xs = {"a": torch.randn(82, width, generator=g).to(dtype),
          "b": torch.randn(46, width, generator=g).to(dtype)}
    want = {rid: pv.latent_attention(x.double(), {k: v.double() for k, v in w.items()}, "", m, eps,
                                     act=_act(dtype)) for rid, x in xs.items()}
    h = PartHarness([mixer], [spec], dtype, page_size=page, num_pages=4 + 160 // page)
    portions = [[("a", 30), ("b", 1)], [("a", 2), ("b", 1)], [("a", 1), ("b", 17)], [("a", 25)],
                [("a", 17), ("b", 21)]] + [[("a", 1), ("b", 1)]] * 6 + [[("a", 1)]]
    got = _run_in_portions(mixer, h, xs, portions)
    for rid in xs:
        assert_close(got[rid], want[rid], dtype, f"latent attention {rid}")


@pytest.mark.parametrize("decoded", [0, 40])
@pytest.mark.parametrize("far", [0, 1, 15, 16, 17, 200])
def test_one_key_among_hundreds_decides(far, decoded):
    """One key's input row is made large (its rotated part is not normed) and the scale sharp, and
    the input is chosen so that this key (the first token, one at a page border, one far back)
    carries the last token's softmax if it is seen with the right rotation: a lost, misplaced or
    wrongly turned key changes the result."""
    width, eps, T = 40, 1e-6, 420
    m = _mixer_sizes(4, 8, 8, 12, 16, 24, 1.5, 10000.0, (8.0, 64, 32.0, 1.0))
    mixer = _latent(torch.float32, width, m, eps)
    w = _latent_weights(width, m, 31, spread=2.0)
    mixer.load(w)
    wd = {k: v.double() for k, v in w.items()}
    others = torch.cat((torch.arange(far), torch.arange(far + 1, T)))
    for seed in range(40):
        g = _gen(100 * far + seed)
        x = torch.randn(T, width, generator=g)
        x[far] *= 6.0                                   # the unnormed rotated key part grows
        want = pv.latent_attention(x.double(), wd, "", m, eps)
        # whether that key carries weight at the last token shows in what the rest gives alone
        rest = pv.latent_attention(x[others].double(), wd, "", m, eps, positions=others)
        if (want[T - 1] - rest[-1]).abs().max() > 0.05 * want[T - 1].abs().max():
            break
    else:
        raise AssertionError("no input was found whose key decides")
    h = PartHarness([mixer], [mixer.cache_spec()], torch.float32, page_size=16, num_pages=28)
    head = T - decoded
    portions = [[("a", head - 150)], [("a", 150)]] + [[("a", 1)]] * decoded
    got = _run_in_portions(mixer, h, {"a": x}, portions)
    assert_close(got["a"], want, torch.float32, f"key {far}")


def test_pages_are_used_again():
    """Requests come and go in a pool of few pages (freed pages are poisoned): every request's
    result is what it gives alone."""
    width, eps = 32, 1e-5
    m = _mixer_sizes(3, 8, 4, 8, 12, 12, 0.3)
    mixer = _latent(torch.float32, width, m, eps)
    w = _latent_weights(width, m, 9)
    mixer.load(w)
    h = PartHarness([mixer], [mixer.cache_spec()], torch.float32, page_size=8, num_pages=9,
                    max_seqs=3)
    wd = {k: v.double() for k, v in w.items()}
    g = _gen(2)
    for rnd in range(5):
        xs = {f"r{rnd}a": torch.randn(31 + rnd, width, generator=g),
              f"r{rnd}b": torch.randn(20 - rnd, width, generator=g)}
        a, b = sorted(xs)
        got = _run_in_portions(mixer, h, xs, [[(a, 9), (b, 20 - rnd)], [(a, 21 + rnd)], [(a, 1)]])
        for rid, x in xs.items():
            assert_close(got[rid], pv.latent_attention(x.double(), wd, "", m, eps), torch.float32,
                         f"turn {rnd} {rid}")
            h.cache.release(rid)
        h.cache.check_invariants()


# ----------------------------------------------------------------------------- routed experts
def _experts(dtype, width, inner, experts, top):
    from distengine_b200.parts import build_feed_forward
    return build_feed_forward(_spec().of("routed_experts", width=width, inner=inner,
                                         experts=experts, top=top, activation="gelu_erf"), dtype,
                              torch.device(DEV))


def _expert_weights(width, inner, experts, seed, spread=1.5):
    g = _gen(seed)
    bf = lambda t: t.to(torch.bfloat16).float()
    w = {"router": bf(torch.randn(experts, width, generator=g) * spread / math.sqrt(width)),
         "router.b": bf(torch.randn(experts, generator=g) * 0.3)}
    for e in range(experts):
        w[f"e{e}.up"] = bf(torch.randn(inner, width, generator=g) * spread / math.sqrt(width))
        w[f"e{e}.down"] = bf(torch.randn(width, inner, generator=g) * spread / math.sqrt(inner))
    return w


@pytest.mark.parametrize("width,inner,experts,top,n", [
    (42, 11, 5, 2, 37),          # odd sizes
    (64, 16, 4, 4, 20),          # every token through every expert
    (40, 24, 1, 1, 9),           # one expert: its weight is 1
    (48, 32, 16, 3, 300),        # more than 64 pairs an expert: several tiles of one expert
    (32, 8, 33, 5, 70),          # more experts than a warp has lanes
])
def test_routed_experts(width, inner, experts, top, n):
    """The router's choice and weights (32-bit), and the weighted sum of the chosen experts, in
    one step and cut into unequal steps (a token's result does not depend on its neighbours)."""
    ff = _experts(torch.float32, width, inner, experts, top)
    w = _expert_weights(width, inner, experts, 3 * experts + top)
    assert {k: v[0] for k, v in ff.tensors().items()} == {k: tuple(v.shape) for k, v in w.items()}
    ff.load(w)
    x = torch.randn(n, width, generator=_gen(n))
    wd = {k: v.double() for k, v in w.items()}
    want = pv.routed_feed_forward(x.double(), wd, "", experts, top)
    h = PartHarness([ff], [], torch.float32)
    got = h.run([("a", n)], lambda ctx, b: ff.forward(x.to(DEV), ctx).clone())
    assert got.dtype == torch.float32                       # joins the stream unrounded
    assert_close(got, want, torch.float32, "routed experts")
    cut = n // 3
    for part in (slice(0, cut), slice(cut, cut + 1), slice(cut + 1, n)):
        xs = x[part].to(DEV)
        piece = h.run([("a", xs.shape[0])], lambda ctx, b: ff.forward(xs, ctx).clone())
        assert torch.equal(piece, got[part]), "a token's result depends on its step"


def test_the_router_bias_decides_and_ties_go_to_the_lower_index():
    """Equal router rows: the logits differ by the bias alone, so the bias picks the experts; with
    equal biases too, the lowest indices are chosen and share the weight equally."""
    from distengine_b200.kernels import latent as lk
    width, experts, top, n = 24, 7, 3, 13
    g = _gen(4)
    x = torch.randn(n, width, generator=g).to(DEV)
    router = torch.randn(1, width, generator=g).repeat(experts, 1).contiguous().to(DEV)
    chosen = torch.empty(n, top, dtype=torch.int32, device=DEV)
    weight = torch.empty(n, top, device=DEV)
    bias = torch.tensor([0.0, 2.0, -1.0, 0.5, 3.0, 0.25, 1.0], device=DEV)
    lk.experts_route(x, router, bias, top, chosen, weight)
    assert sorted(chosen[0].tolist()) == [1, 4, 6]
    assert bool((chosen == chosen[0]).all())
    order = {e: i for i, e in enumerate(chosen[0].tolist())}
    want = torch.softmax(torch.tensor([3.0, 2.0, 1.0], dtype=torch.float64), 0)
    got = weight[5].cpu().double()
    assert_close(torch.stack([got[order[4]], got[order[1]], got[order[6]]]), want, torch.float32,
                 "weights over the chosen logits alone")
    lk.experts_route(x, router, torch.zeros(experts, device=DEV), top, chosen, weight)
    assert sorted(chosen[3].tolist()) == [0, 1, 2]
    assert_close(weight.cpu(), torch.full((n, top), 1 / 3), torch.float32, "tied weights")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,inner,experts,top,n", [
    (72, 40, 8, 2, 150),         # few pairs: tiles of 64 slots on the CUDA cores
    (72, 40, 8, 2, 700),         # many pairs: in bfloat16, tiles of 128 slots on the tensor cores
    (64, 96, 24, 3, 400),        # tiles that are mostly empty, experts without a token
    (256, 320, 4, 1, 1500),      # several tiles an expert, several tiles of columns
])
def test_routed_experts_in_both_types_with_the_engine_choice(dtype, width, inner, experts, top, n):
    """bfloat16 rounds the products; the plain function is given the engine's choice of experts
    and says how near a tie any other choice was."""
    ff = _experts(dtype, width, inner, experts, top)
    w = _expert_weights(width, inner, experts, 8)
    w["router.b"][1::5] = -50.0                 # experts that no token chooses
    ff.load(w)
    x = torch.randn(n, width, generator=_gen(6)).to(dtype)
    h = PartHarness([ff], [], dtype)
    caught = {}

    def fn(ctx, b):
        out = ff.forward(x.to(DEV), ctx).clone()
        caught["chosen"] = ctx.buffer("experts.chosen", (n, top), torch.int32).clone().cpu()
        return out

    got = h.run([("a", n)], fn)
    slack: list = []
    want = pv.routed_feed_forward(x.double(), {k: v.double() for k, v in w.items()}, "", experts,
                                  top, act=_act(dtype), chosen=caught["chosen"], slack=slack)
    assert max(slack) <= 1e-3
    assert_close(got, want, dtype, "routed experts")


# ----------------------------------------------------------------------------- dense feed-forward
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,inner", [(42, 30), (64, 96), (256, 520)])
def test_gated_feed_forward_with_the_tanh_gelu(dtype, width, inner):
    from distengine_b200.parts import build_feed_forward
    ff = build_feed_forward(_spec().of("gated_mlp", width=width, inner=inner,
                                       activation="gelu_tanh", names=("gate", "up", "down")),
                            dtype, torch.device(DEV))
    g = _gen(width)
    bf = lambda t: t.to(torch.bfloat16).float()
    w = {"gate": bf(torch.randn(inner, width, generator=g) * 2.0 / math.sqrt(width)),
         "up": bf(torch.randn(inner, width, generator=g) / math.sqrt(width)),
         "down": bf(torch.randn(width, inner, generator=g) / math.sqrt(inner))}
    assert {k: v[0] for k, v in ff.tensors().items()} == {k: tuple(v.shape) for k, v in w.items()}
    ff.load(w)
    x = (torch.randn(19, width, generator=g) * 1.5).to(dtype)
    h = PartHarness([ff], [], dtype)
    got = h.run([("a", 19)], lambda ctx, b: ff.forward(x.to(DEV), ctx).clone())
    want = pv.gated_feed_forward(x.double(), {k: v.double() for k, v in w.items()}, "",
                                 act=_act(dtype))
    assert_close(got, want, dtype, "gated feed-forward")
    # the tanh form is not the erf form: at these inputs they differ by more than the tolerance
    other = (pv.gelu_erf(x.double() @ w["gate"].double().t())
             * (x.double() @ w["up"].double().t())) @ w["down"].double().t()
    assert (other - want).abs().max() > 1e-3


# ----------------------------------------------------------------------------- the side input
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,dim,index,layers", [(42, 5, 2, 4), (64, 8, 0, 1), (40, 1, 3, 5)])
def test_token_side_input(dtype, width, dim, index, layers):
    """The layer's part of the token's table row gates a small projection; the result joins the
    stream behind an RMS norm (eps inside the root: rows of tiny y show it)."""
    from distengine_b200.parts.base import build_side_input
    from distengine_b200.parts.context import ResidualStream
    vocab, eps, n = 31, 1e-5, 17
    side = build_side_input(_spec().of("token_side", width=width, dim=dim, index=index,
                                       layers=layers, vocabulary=vocab, eps=eps,
                                       table="/side.embed"), dtype, torch.device(DEV))
    g = _gen(10 * width + dim)
    bf = lambda t: t.to(torch.bfloat16).float()
    w = {"side.embed": bf(torch.randn(vocab, layers * dim, generator=g)),
         "gate": bf(torch.randn(dim, width, generator=g) / math.sqrt(width)),
         "proj": bf(torch.randn(width, dim, generator=g) / math.sqrt(dim)),
         "norm": bf(torch.rand(width, generator=g) + 0.5)}
    w["side.embed"][3] *= 1e-3                   # y so small that eps counts
    side.load({("/side.embed" if k == "side.embed" else k): v for k, v in w.items()})
    ids = [int(t) for t in torch.randint(0, vocab, (n,), generator=g)]
    ids[4] = ids[9] = 3
    x = torch.randn(n, width, generator=g)
    rows = x.to(dtype)                           # the stream as the projections read it
    h = PartHarness([side], [], dtype, vocabulary=vocab)

    def fn(ctx, b):
        stream = ResidualStream(x.to(DEV).clone())
        side.forward(stream, rows.to(DEV), ctx)
        return stream.resid.clone()

    got = h.run([("a", n)], fn, tokens={"a": ids})
    wd = {k: v.double() for k, v in w.items()}
    want = x.double() + pv.token_side(x.double(), torch.tensor(ids), wd, "", index, dim, eps,
                                      act=_act(dtype))
    assert got.dtype == torch.float32
    assert_close(got, want, dtype, "token side input")
    no_eps = pv.token_side(x.double(), torch.tensor(ids), wd, "", index, dim, 0.0)
    with_eps = pv.token_side(x.double(), torch.tensor(ids), wd, "", index, dim, eps)
    assert (no_eps[4] - with_eps[4]).abs().max() > 1e-2
