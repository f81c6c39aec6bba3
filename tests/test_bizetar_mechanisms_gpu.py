"""Each mechanism of the Bizetar parts alone, built through the configuration and the registries
and run through the engine's step machinery, against the plain function in ``plain_bizetar``: both
forms of sink attention in portions and single tokens at sizes that are no multiple of anything,
with one key among hundreds made decisive (the first token, keys on both sides of a page border, a
far one), the sink's share, the distance bias, the query's growth, the mixing of values between
layers, pages and slots that are used again; the row kernels of the block; the learned cubic
activation; the router's scores, its correction, the outputs that hand the input on, and the gated
experts.  (The block is compared layer by layer in ``test_bizetar_gpu``.)"""

import math

import pytest
import torch

import bizetar_configs as bc
import plain_bizetar as pb
from gpu_helpers import PartHarness, assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def _gen(seed):
    return torch.Generator().manual_seed(seed)


def _act(dtype):
    return None if dtype == torch.float32 else torch.bfloat16


def _build(config, dtype):
    """The mixers and feed-forwards of a configuration's layers, built as the model builds them,
    with the plain implementation's random weights."""
    from distengine_b200.config.bizetar import BizetarConfig
    from distengine_b200.parts import build_feed_forward, build_mixer
    specs = BizetarConfig.from_json(config).layer_specs()
    weights = pb.random_weights(config, 5, spread=1.5)
    mixers, feeds = [], []
    for i, spec in enumerate(specs):
        for part_spec, prefix, out in ((spec.mixer, f"l{i}.mix.", mixers),
                                       (spec.feed_forward, f"l{i}.mlp.", feeds)):
            if part_spec is None:
                out.append(None)
                continue
            build = build_mixer if out is mixers else build_feed_forward
            part = build(part_spec, dtype, torch.device(DEV))
            part.load({local: weights[prefix + local] for local in part.tensors()})
            out.append(part)
    return mixers, feeds, {k: v.double() for k, v in weights.items()}


def _model(width, layers, eps=1e-5):
    return {"architecture": "Bizetar", "vocab": 16, "width": width, "norm": {"eps": eps},
            "layers": layers}


def _run_in_portions(mixers, h, xs, portions):
    """Feeds the requests' rows in the given portions through all mixers one after the other (each
    on the same input rows: only the values of the first reach the later ones); returns every
    mixer's result for every request's rows in order."""
    fed = {rid: 0 for rid in xs}
    got = [{rid: [] for rid in xs} for _ in mixers]
    for step in portions:
        entries = [(rid, n) for rid, n in step if n]
        x = torch.cat([xs[rid][fed[rid]: fed[rid] + n] for rid, n in entries]).to(DEV)

        def run(ctx, bindings):
            return torch.stack([m.forward(x, ctx, b).float().clone()
                                for m, b in zip(mixers, bindings)])

        out = h.run(entries, run).cpu()
        at = 0
        for rid, n in entries:
            for index in range(len(mixers)):
                got[index][rid].append(out[index, at: at + n])
            at += n
            fed[rid] += n
    assert all(fed[rid] == xs[rid].shape[0] for rid in xs)
    return [{rid: torch.cat(parts) for rid, parts in g.items()} for g in got]


def _plain_mixers(config, wd, x, act=None):
    """Every layer's mixer on the same input x, values handed on as in the model."""
    outs, v_first = [], None
    for i, entry in enumerate(config["layers"]):
        m = entry["mixer"]
        fn = pb.attention if entry["type"] == "attention" else pb.attention_2
        y, v = fn(x, wd, f"l{i}.mix.", m, config["norm"]["eps"],
                  v_first if m.get("v_mix") else None, act)
        if m.get("v_mix") and v_first is None:
            v_first = v
        outs.append(y)
    return outs


PORTIONS = [[("a", 30), ("b", 1)], [("a", 2), ("b", 1)], [("a", 1), ("b", 17)], [("a", 25)],
            [("a", 17), ("b", 21)]] + [[("a", 1), ("b", 1)]] * 6 + [[("a", 1)]]

MIXERS = [
    # rows that are no 16-byte piece; two kv heads; the query grows every third position
    (bc.layer("attention", bc.first(6, 2, 5, 3, 0.4, q_temp=(0.7, 3)), None), 16),
    (bc.layer("attention_2", bc.second(6, 2, 10, 3, 0.3, conv=2,
                                       rot=(100.0, 6, (4.0, 16, 8.0, 1.0))), None), 4),
    # whole pieces, up to 8 heads a kv head: single tokens take the one-block kernel
    (bc.layer("attention", bc.first(8, 1, 16, 8, 0.25, q_temp=(0.3, 1)), None), 8),
    (bc.layer("attention_2", bc.second(8, 2, 16, 16, 0.25, conv=3,
                                       rot=(30000.0, 16, (8.0, 32, 16.0, 1.0))), None), 8),
    # more than 8 heads a kv head; no convolution, rotation of a part without stretch
    (bc.layer("attention_2", bc.second(12, 1, 8, 8, 0.3, rot=(1000000.0, 4)), None), 16),
    # one head, values of size 1, five taps, nothing rotated
    (bc.layer("attention_2", bc.second(1, 1, 32, 1, 0.15, conv=5), None), 8),
    (bc.layer("attention", bc.first(5, 5, 4, 24, 0.3), None), 32),
    # a single tap is a weight on every channel
    (bc.layer("attention_2", bc.second(4, 4, 24, 20, 0.2, conv=1, rot=(500.0, 24)), None), 16),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("entry,page", MIXERS)
def test_sink_attention_in_portions(dtype, entry, page):
    """Two requests in unequal portions beside single tokens, then steps of single tokens only,
    against the plain function over each whole sequence."""
    config = _model(44, [entry])
    (mixer,), _, wd = _build(config, dtype)
    g = _gen(5)
    xs = {"a": torch.randn(82, 44, generator=g).to(dtype),
          "b": torch.randn(46, 44, generator=g).to(dtype)}
    want = {rid: _plain_mixers(config, wd, x.double(), _act(dtype))[0] for rid, x in xs.items()}
    h = PartHarness([mixer], [mixer.cache_spec()], dtype, page_size=page,
                    num_pages=4 + 160 // page)
    got = _run_in_portions([mixer], h, xs, PORTIONS)[0]
    for rid in xs:
        assert_close(got[rid], want[rid], dtype, f"sink attention {rid}")


def test_values_are_mixed_between_layers():
    """Four mixers in one step: the first gives its values, the second takes them with its own
    lambda, the third stays out, the fourth takes them with as many numbers a token in another
    split into heads; what a taker caches is the mixed value (decoded tokens read it back)."""
    config = _model(40, [
        bc.layer("attention", bc.first(4, 2, 8, 6, 0.3), None),
        bc.layer("attention_2", bc.second(6, 2, 4, 6, 0.4, conv=3, rot=(100.0, 4)), None),
        bc.layer("attention_2", bc.second(2, 1, 8, 5, 0.4, v_mix=False, conv=2), None),
        bc.layer("attention_2", bc.second(3, 1, 8, 12, 0.4), None)])
    mixers, _, wd = _build(config, torch.float32)
    assert [m.value_mix for m in mixers] == ["give", "take", None, "take"]
    g = _gen(8)
    xs = {"a": torch.randn(60, 40, generator=g), "b": torch.randn(33, 40, generator=g)}
    h = PartHarness(mixers, [m.cache_spec() for m in mixers], torch.float32, page_size=8,
                    num_pages=30)
    portions = [[("a", 20), ("b", 3)], [("a", 1), ("b", 29)], [("a", 38)], [("a", 1), ("b", 1)]]
    got = _run_in_portions(mixers, h, xs, portions)
    for rid, x in xs.items():
        want = _plain_mixers(config, wd, x.double())
        for index in range(4):
            assert_close(got[index][rid], want[index], torch.float32, f"mixer {index} {rid}")
    # without the mixing the second mixer gives something else
    plain = dict(config["layers"][1]["mixer"], v_mix=False)
    alone, _ = pb.attention_2(xs["a"].double(), wd, "l1.mix.", plain, 1e-5, None)
    assert (alone - got[1]["a"].double()).abs().max() > 1e-2


@pytest.mark.parametrize("kind", ["attention", "attention_2"])
@pytest.mark.parametrize("decoded", [0, 40])
@pytest.mark.parametrize("far", [0, 1, 15, 16, 17, 200])
def test_one_key_among_hundreds_decides(kind, far, decoded):
    """The query matrix reads one half of the input as the key matrix reads the other, and the
    last token's first half is the far token's second: that key (the first token, one at a page
    border, one far back) carries the last token's softmax if it is seen, at the right distance
    and turned by the right position, and its value is its own; a lost or misplaced key changes
    the result."""
    width, T, dk = 40, 420, 32
    if kind == "attention":
        entry = bc.layer(kind, bc.first(4, 1, dk, 12, 1.0, q_temp=(0.4, 96)), None)
    else:
        entry = bc.layer(kind, bc.second(4, 1, dk, 12, 1.0,
                                         rot=(10000.0, 4, (8.0, 64, 32.0, 1.0))), None)
    config = _model(width, [entry])
    from distengine_b200.config.bizetar import BizetarConfig
    from distengine_b200.parts import build_mixer
    weights = pb.random_weights(config, 31, spread=2.0)
    half = width // 2
    wq = torch.zeros(dk, width)
    wq[:, :half] = weights["l0.mix.k"][:, half:]
    weights["l0.mix.k"][:, :half] = 0
    weights["l0.mix.q"] = wq.repeat(4, 1)                          # every head asks for its like
    if kind == "attention":
        weights["l0.mix.q.norm"] = weights["l0.mix.k.norm"].repeat(4)
        weights["l0.mix.sink"] = torch.full((4,), 2.0)
    else:
        weights["l0.mix.q.b"] = weights["l0.mix.k.b"].repeat(4)
        weights["l0.mix.q.norm"] = weights["l0.mix.k.norm"].clone()
    mixer = build_mixer(BizetarConfig.from_json(config).layer_specs()[0].mixer, torch.float32,
                        torch.device(DEV))
    mixer.load({local: weights[f"l0.mix.{local}"] for local in mixer.tensors()})
    wd = {k: v.double() for k, v in weights.items()}
    fn = pb.attention if kind == "attention" else pb.attention_2
    for seed in range(40):
        g = _gen(100 * far + seed)
        x = torch.randn(T, width, generator=g)
        x[T - 1, :half] = x[far, half:]
        want, _ = fn(x.double(), wd, "l0.mix.", entry["mixer"], 1e-5, None)
        # that the key carries weight at the last token shows in what another input there gives
        other = x.clone()
        other[far] = torch.randn(width, generator=g)
        moved, _ = fn(other.double(), wd, "l0.mix.", entry["mixer"], 1e-5, None)
        if (want[T - 1] - moved[T - 1]).abs().max() > 0.3 * want[T - 1].abs().max():
            break
    else:
        raise AssertionError("no input was found whose key decides")
    h = PartHarness([mixer], [mixer.cache_spec()], torch.float32, page_size=16, num_pages=28)
    head = T - decoded
    portions = [[("a", head - 150)], [("a", 150)]] + [[("a", 1)]] * decoded
    got = _run_in_portions([mixer], h, {"a": x}, portions)[0]
    assert_close(got["a"], want, torch.float32, f"key {far}")


@pytest.mark.parametrize("sink,share", [(-30.0, 0.0), (0.0, None), (30.0, 1.0)])
def test_the_sink_takes_its_share(sink, share):
    """A sink far below every score leaves the plain softmax, one far above takes all the weight
    (the result vanishes), one between is counted once whatever the step's cut."""
    entry = bc.layer("attention_2", bc.second(3, 1, 8, 8, 0.3), None)
    config = _model(24, [entry])
    (mixer,), _, wd = _build(config, torch.float32)
    mixer.sink.fill_(sink)
    wd["l0.mix.sink"] = torch.full((3,), sink, dtype=torch.float64)
    x = torch.randn(50, 24, generator=_gen(3))
    want = _plain_mixers(config, wd, x.double())[0]
    h = PartHarness([mixer], [mixer.cache_spec()], torch.float32, page_size=8, num_pages=10)
    got = _run_in_portions([mixer], h, {"a": x}, [[("a", 33)], [("a", 2)]] + [[("a", 1)]] * 15)[0]
    assert_close(got["a"], want, torch.float32, f"sink {sink}")
    if share == 1.0:
        assert got["a"].abs().max() < 1e-6
    if share == 0.0:
        assert (got["a"][0] - got["a"][1]).abs().max() > 1e-3    # the first token sees itself alone


def test_pages_and_slots_are_used_again():
    """Requests come and go in a pool of few pages and three slots (freed pages are poisoned, the
    convolution's kept rows start from zero in a slot that is used again): every request's result
    is what it gives alone."""
    entry = bc.layer("attention_2", bc.second(3, 1, 8, 8, 0.3, conv=4, rot=(10000.0, 8)), None)
    config = _model(32, [entry])
    (mixer,), _, wd = _build(config, torch.float32)
    h = PartHarness([mixer], [mixer.cache_spec()], torch.float32, page_size=8, num_pages=9,
                    max_seqs=3)
    g = _gen(2)
    for turn in range(5):
        xs = {f"r{turn}a": torch.randn(31 + turn, 32, generator=g),
              f"r{turn}b": torch.randn(20 - turn, 32, generator=g)}
        a, b = sorted(xs)
        got = _run_in_portions([mixer], h, xs, [[(a, 9), (b, 20 - turn)], [(a, 21 + turn)],
                                               [(a, 1)]])[0]
        for rid, x in xs.items():
            assert_close(got[rid], _plain_mixers(config, wd, x.double())[0], torch.float32,
                         f"turn {turn} {rid}")
            h.cache.release(rid)
        h.cache.check_invariants()


# ----------------------------------------------------------------------------- row kernels
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,width", [(1, 42), (37, 320), (5, 2050)])
def test_row_kernels_of_the_block(dtype, n, width):
    """The stream's norm in place, gate * result -> norm -> sum, the mix over the depth, each with
    its rounded copy; the eps inside the root shows on a row that is nearly zero."""
    from distengine_b200.kernels import ops
    g = _gen(n + width)
    x = torch.randn(n, width, generator=g) * 3.0
    x[0] *= 1e-3
    weight = (torch.rand(width, generator=g) + 0.5).to(torch.bfloat16).float()
    eps = 1e-5
    resid, rows = x.to(DEV), torch.empty(n, width, dtype=dtype, device=DEV)
    ops.norm_stream(resid, weight.to(DEV), eps, rows)
    want = pb.rms_norm(x.double(), weight.double(), eps)
    assert_close(resid, want, torch.float32, "norm_stream")
    assert torch.equal(rows.float().cpu(), resid.cpu().to(dtype).float())

    y = torch.randn(n, width, generator=g).to(dtype)
    z = torch.randn(n, width + 8, generator=g).to(dtype)[:, :width]      # rows with a stride
    bias = torch.randn(width, generator=g)
    base = torch.randn(n, width, generator=g)
    want = base.double() + pb.rms_norm(y.double() * pb.sigmoid(z.double() + bias.double()),
                                       weight.double(), eps)
    for y_dtype in {dtype, torch.float32}:
        out = torch.empty(n, width, device=DEV)
        ops.gated_normed_add(y.to(DEV, y_dtype), z.to(DEV), bias.to(DEV), weight.to(DEV), eps,
                             base.to(DEV), out, rows)
        assert_close(out, want, torch.float32, "gated_normed_add")
        assert torch.equal(rows.float().cpu(), out.cpu().to(dtype).float())
    in_place = base.to(DEV)
    ops.gated_normed_add(y.to(DEV), z.to(DEV), bias.to(DEV), weight.to(DEV), eps, in_place,
                         in_place, None)
    assert_close(in_place, want, torch.float32, "gated_normed_add in place")

    history = torch.randn(4, n, width, generator=g)
    coef = torch.randn(3, generator=g)
    out = torch.empty(n, width, device=DEV)
    ops.depth_mix(history.to(DEV)[:3], coef.to(DEV), out, rows)
    want = sum(coef[j].double() * history[j].double() for j in range(3))
    assert_close(out, want, torch.float32, "depth_mix")
    assert torch.equal(rows.float().cpu(), out.cpu().to(dtype).float())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,inner,n", [(42, 30, 19), (64, 96, 1), (48, 130, 70)])
def test_the_cubic_activation(dtype, width, inner, n):
    """down(a N(z) + b N(z^2) + c N(z^3) + e) with z = up x: every power normed by its own root
    mean square over the inner values, the constant added after."""
    config = _model(width, [bc.layer("attention", bc.first(1, 1, 4, 4, 0.5), bc.dense(inner))])
    _, (feed,), wd = _build(config, dtype)
    x = torch.randn(n, width, generator=_gen(inner)).to(dtype)
    want = pb.dense_feed_forward(x.double(), wd, "l0.mlp.", 1e-5, _act(dtype))
    h = PartHarness([feed], [None], dtype)
    got = h.run([("a", n)], lambda ctx, b: feed.forward(x.to(DEV), ctx).clone())
    assert_close(got, want, dtype, "cubic activation")
    # each term matters: without the constant, or with plain powers, the result differs
    z = pb.lin(x.double(), wd["l0.mlp.up"])
    a, b, c, e = wd["l0.mlp.act"]
    plain_powers = pb.lin(a * z + b * z ** 2 + c * z ** 3 + e, wd["l0.mlp.down"])
    assert (plain_powers - want).abs().max() > 1e-2 * want.abs().max()


# ----------------------------------------------------------------------------- routed experts
def _routed(dtype, width, experts, top, inner, identity, seed=5):
    config = _model(width, [bc.layer("attention", bc.first(1, 1, 4, 4, 0.5),
                                     bc.moe(experts, top, inner, identity))])
    _, (feed,), wd = _build(config, dtype)
    return config, feed, wd


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,experts,top,inner,identity,n", [
    (42, 5, 2, 11, 2, 33),        # odd sizes: the CUDA-core tiles
    (64, 4, 6, 16, 2, 150),       # every router output chosen, more than 128 pairs an expert
    (48, 1, 2, 32, 3, 70),        # one expert beside three outputs that hand the input on
    (40, 9, 3, 24, 0, 1),         # no such outputs, a single token
    (32, 16, 1, 8, 1, 20),        # experts that nobody chooses
])
def test_gated_experts_with_outputs_that_hand_on(dtype, width, experts, top, inner, identity, n):
    config, feed, wd = _routed(dtype, width, experts, top, inner, identity)
    x = torch.randn(n, width, generator=_gen(experts + n)).to(dtype)
    h = PartHarness([feed], [None], dtype)
    seen = {}

    def run(ctx, b):
        out = feed.forward(x.to(DEV), ctx).clone()
        seen["chosen"] = ctx.buffer("experts.chosen", (n, top), torch.int32).clone()
        return out

    got = h.run([("a", n)], run)
    chosen = seen["chosen"].cpu().long()
    router = config["layers"][0]["mlp"]["router"]
    if dtype == torch.float32:
        picked, _ = pb.route(x.double(), wd, "l0.mlp.", top)
        assert torch.equal(picked.sort(dim=1).values, chosen.sort(dim=1).values)
    want = pb.routed_feed_forward(x.double(), wd, "l0.mlp.", router, _act(dtype), chosen)
    assert_close(got, want, dtype, "routed experts")
    if identity:
        assert (chosen >= experts).any(), "no token chose an output that hands its input on"


def test_the_correction_moves_the_choice_but_not_the_weights():
    """A large correction on one output makes every token choose it, with the weight of its plain
    score; the scores are the softmax over all outputs and are not renormalised."""
    config, feed, wd = _routed(torch.float32, 32, 6, 2, 8, 2)
    feed.bias.zero_()
    feed.bias[3] = 5.0
    wd["l0.mlp.correction"] = feed.bias.double().cpu()
    n = 40
    x = torch.randn(n, 32, generator=_gen(11))
    h = PartHarness([feed], [None], torch.float32)
    seen = {}

    def run(ctx, b):
        out = feed.forward(x.to(DEV), ctx).clone()
        seen["chosen"] = ctx.buffer("experts.chosen", (n, 2), torch.int32).clone()
        seen["weight"] = ctx.buffer("experts.weight", (n, 2), torch.float32).clone()
        return out

    got = h.run([("a", n)], run)
    chosen, weight = seen["chosen"].cpu().long(), seen["weight"].cpu()
    assert (chosen[:, 0] == 3).all()
    scores = torch.softmax(x.double() @ wd["l0.mlp.router"].t(), dim=-1)
    assert_close(weight, torch.gather(scores, 1, chosen), torch.float32, "weights")
    assert (weight.sum(dim=1) < 0.999).all()
    router = config["layers"][0]["mlp"]["router"]
    assert_close(got, pb.routed_feed_forward(x.double(), wd, "l0.mlp.", router), torch.float32,
                 "corrected choice")


def test_stretched_frequencies_and_adjacent_pairs():
    """The engine's frequency table against the plain one, and the turn of adjacent pairs with the
    grown cosine and sine against a rotation written with complex numbers."""
    from distengine_b200.parts.sink_attention import stretched_frequencies
    for base, dims, stretch in ((40000.0, 48, (6.0, 1024, 16.0, 2.0)), (100.0, 6, (4.0, 16, 8.0, 1.0)),
                                (10000.0, 8, None), (20.0, 2, (40.0, 100, 2.0, 0.5))):
        scaling = None if stretch is None else dict(zip(("factor", "original", "fast", "slow"),
                                                        stretch))
        want, magnitude = pb.stretched_frequencies(base, dims, scaling)
        got, grown = stretched_frequencies(base, dims, stretch)
        assert torch.allclose(got.double(), want, rtol=1e-6, atol=0) and grown == magnitude
        x = torch.randn(5, 2, dims + 3, generator=_gen(dims), dtype=torch.float64)
        pos = torch.tensor([0, 1, 7, 300, 4000])
        turned = pb.rotate_adjacent(x, pos, want, magnitude)
        z = torch.view_as_complex(x[..., :dims].reshape(5, 2, dims // 2, 2).contiguous())
        z = z * torch.polar(torch.full((5, 1, dims // 2), magnitude, dtype=torch.float64),
                            (pos[:, None].double() * want[None, :])[:, None, :])
        assert torch.allclose(turned[..., :dims], torch.view_as_real(z).reshape(5, 2, dims))
        assert torch.equal(turned[..., dims:], x[..., dims:])
    assert math.isclose(pb.stretched_frequencies(10000.0, 8, None)[1], 1.0)
