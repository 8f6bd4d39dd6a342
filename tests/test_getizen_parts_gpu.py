"""The mechanisms of the Getizen design one by one, built through the part registry with sizes of their own, against
the plain functions of ``plain_getizen``: the group norm of the stream with its branches, the clamped gated
feed-forward, retention, gated chunked attention, the gated linear recurrence and the mixers side by side.  Mixers
run a sequence whole, in portions down to one token, and several requests in one batch, from state slots and pages
that other requests used before."""
import pytest
import torch

import plain_getizen as pg
from helpers import close

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = [torch.float32, torch.bfloat16]
PAGE = 16


def rt_for(dt):
    from mini_inference_engine_b200.parts import Runtime
    return Runtime(DEV, dt)


def build(category, kind, **params):
    from mini_inference_engine_b200.config import PartSpec
    from mini_inference_engine_b200.parts import build_part
    return build_part(category, PartSpec(kind, params))


def bind_random(part, rt, seed, overrides=None):
    """Random tensors by the part's own init rules, stored as bfloat16 values (so both modes read the same numbers)."""
    from mini_inference_engine_b200.weights.random_init import random_tensor
    tensors = {n: random_tensor(seed, n, s, torch.bfloat16) for n, s in part.tensor_specs().items()}
    tensors.update({k: v.to(torch.bfloat16) for k, v in (overrides or {}).items()})
    part.bind(tensors, rt)
    return {"p." + k: v.float() for k, v in tensors.items()}


class Harness:
    """Runs one mixer over requests step by step: its own pages and state slots, a batch builder, no model."""

    def __init__(self, mixer, rt, pages=64, slots=4):
        from mini_inference_engine_b200.cache.manager import CacheManager
        from mini_inference_engine_b200.cache.storage import CacheLayout, CacheStorage
        from mini_inference_engine_b200.engine.batch import BatchBuilder
        self.mixer, self.rt = mixer, rt
        layout = CacheLayout.from_needs({0: mixer.cache_need()})
        self.manager = CacheManager(layout.groups, pages, PAGE, slots)
        self.storage = CacheStorage(layout, pages, PAGE, slots, rt.dtype, DEV)
        self.cache = self.storage.layer_cache(0)
        self.builder = BatchBuilder(len(layout.groups), PAGE, DEV)

    def new(self):
        from mini_inference_engine_b200.cache.manager import RequestCache
        return RequestCache()

    def step(self, entries):
        """entries: [(request cache, x rows [n, hidden] float32)] -> list of outputs [n, hidden] float32 (CPU)."""
        from mini_inference_engine_b200.engine.batch import BatchRow
        rows = []
        for rc, x in entries:
            assert self.manager.take_state_slot(rc) and self.manager.reserve(rc, x.shape[0])
            if rc.num_computed == 0 and rc.state_slot:
                self.storage.clear_state_slot(rc.state_slot)
            rows.append(BatchRow([0] * x.shape[0], rc.num_computed, rc.table_arrays(), rc.state_slot, []))
        ctx = self.builder.build(rows)
        x_all = torch.cat([x for _, x in entries], 0).to(self.rt.dtype).to(DEV)
        out = self.mixer.forward(x_all, ctx, self.cache)
        from mini_inference_engine_b200.parts import Branches
        if isinstance(out, Branches):
            out = torch.stack([d.float() for d in out.deltas])        # [branches, T, hidden]
            out = out.permute(1, 0, 2)
        out = out.float().cpu()
        res, at = [], 0
        for rc, x in entries:
            self.manager.advance(rc, x.shape[0])
            res.append(out[at:at + x.shape[0]])
            at += x.shape[0]
        return res

    def free(self, rc):
        self.manager.free(rc)


def run_in_portions(h, x, portions):
    rc, outs, at = h.new(), [], 0
    for n in portions:
        outs.append(h.step([(rc, x[at:at + n])])[0])
        at += n
    assert at == x.shape[0]
    h.free(rc)
    return torch.cat(outs, 0)


def inputs(T, hidden, seed, dt):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(T, hidden, generator=g).to(dt).float()       # values both modes can hold


# ----------------------------------------------------------------------------------------------- norm

@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("groups", [1, 3, 8])
def test_group_norm_of_the_stream_with_branches(dt, groups):
    rt = rt_for(dt)
    n, T, eps = 48, 7, 2e-4
    norm = build("norm", "group_rmsnorm", size=n, eps=eps, groups=groups)
    W = bind_random(norm, rt, 3, {"weight": torch.randn(n)})
    res = torch.randn(T, n)
    d0, d1 = torch.randn(T, n) * 3, torch.randn(T, n) * 0.2
    w0, w1 = torch.randn(n).to(torch.bfloat16).float(), torch.randn(n).to(torch.bfloat16).float()
    # two branches, each normed over its row first, their mean added to 1.5 x the stream
    want = pg.group_norm(1.5 * res + 0.5 * (pg.rms_scale(d0, eps) * w0 + pg.rms_scale(d1, eps) * w1), W["p.weight"], groups, eps)
    r = res.clone().to(DEV)
    out = norm.apply(r, (d0.to(DEV), d1.to(DEV)), (w0.to(DEV), w1.to(DEV)), alpha=1.5, coef=0.5)
    close(r, want, torch.float32, "stream after the norm")
    close(out, want, dt, "the stream in the activation type")
    # one plain branch
    want1 = pg.group_norm(2.0 * res + d0, W["p.weight"], groups, eps)
    r = res.clone().to(DEV)
    norm.apply(r, (d0.to(DEV),), alpha=2.0)
    close(r, want1, torch.float32, "one branch")
    # rows gathered in front of the head: the stream is not written
    r = res.clone().to(DEV)
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
    close(norm(None, r, rows), pg.group_norm(res, W["p.weight"], groups, eps)[[5, 0, 5]], dt, "gathered rows")
    assert torch.equal(r.cpu(), res)


@pytest.mark.parametrize("dt", DTYPES)
def test_clamped_feed_forward(dt):
    rt = rt_for(dt)
    ff = build("feed_forward", "clamped_glu", hidden_size=40, intermediate_size=72, limit=0.75)
    W = bind_random(ff, rt, 4)
    x = inputs(9, 40, 1, dt) * 2                      # large enough that both clamps bite
    want = pg.feed_forward(x, W, "p.", 0.75)
    g = x @ W["p.gate"].T
    assert (g > 0.75).any() and ((x @ W["p.up"].T).abs() > 0.75).any()
    close(ff.forward(x.to(dt).to(DEV), None), want, dt, "clamped feed-forward")


# ----------------------------------------------------------------------------------------------- retention

RETENTIONS = [dict(num_heads=3, dim=16, vdim=32, decay=(0.5, 0.9, 0.999), rot_dims=8),          # key and value sizes differ, part of a head turns
              dict(num_heads=1, dim=48, vdim=16, decay=(0.97,), rot_dims=48),                    # one head, three threads a column
              dict(num_heads=2, dim=80, vdim=40, decay=(1.0, 0.75), rot_dims=0),                 # no decay at all, no rotation
              dict(num_heads=1, dim=64, vdim=136, decay=(0.9,), rot_dims=32)]                    # two value columns a thread, a ragged last slice


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("params", RETENTIONS)
def test_retention_whole_in_portions_and_token_by_token(dt, params):
    rt = rt_for(dt)
    hidden, T = 24, 150                      # portions longer than a chunk of the recurrence's kernel run as several side by side
    mixer = build("mixer", "retention", hidden_size=hidden, rot_base=100.0, eps=1e-5, **params)
    W = bind_random(mixer, rt, 5)
    m = dict(heads=params["num_heads"], dim=params["dim"], vdim=params["vdim"], decay=list(params["decay"]),
             rot=dict(base=100.0, dims=params["rot_dims"]))
    x = inputs(T, hidden, 2, dt)
    want = pg.retention(x, W, "p.", m, 1e-5)
    h = Harness(mixer, rt)
    tol = dt
    close(run_in_portions(h, x, [T]), want, tol, "whole")
    close(run_in_portions(h, x, [9, 2, 70, 1, 1, 64, 2, 1]), want, tol, "portions")         # the slot was used before
    close(run_in_portions(h, x, [129, 21]), want, tol, "a portion of two chunks and one token")
    close(run_in_portions(h, x, [1] * T), want, tol, "token by token")


@pytest.mark.parametrize("dt", DTYPES)
def test_retention_batch_of_unequal_requests_and_a_far_token(dt):
    rt = rt_for(dt)
    hidden = 32
    params = dict(num_heads=2, dim=32, vdim=32, decay=(0.999, 0.9995), rot_dims=16)
    mixer = build("mixer", "retention", hidden_size=hidden, rot_base=1e4, eps=1e-5, **params)
    W = bind_random(mixer, rt, 6)
    m = dict(heads=2, dim=32, vdim=32, decay=[0.999, 0.9995], rot=dict(base=1e4, dims=16))
    xs = [inputs(n, hidden, 10 + i, dt) for i, n in enumerate((300, 7, 64))]
    xs[0][3] *= 8.0                                   # one early token that the state must still hold 296 tokens on
    wants = [pg.retention(x, W, "p.", m, 1e-5) for x in xs]
    quiet = xs[0].clone()
    quiet[3] /= 8.0
    assert (pg.retention(quiet, W, "p.", m, 1e-5)[-1] - wants[0][-1]).abs().max() > 0.05 * wants[0][-1].abs().max()
    h = Harness(mixer, rt, pages=32, slots=3)
    rcs = [h.new() for _ in xs]
    # step 1: portions of all three; step 2: the rest of the first beside single tokens of the others
    a = h.step([(rcs[0], xs[0][:250]), (rcs[1], xs[1][:6]), (rcs[2], xs[2][:63])])
    b = h.step([(rcs[1], xs[1][6:]), (rcs[0], xs[0][250:]), (rcs[2], xs[2][63:])])
    close(torch.cat([a[0], b[1]]), wants[0], dt, "long request")
    close(torch.cat([a[1], b[0]]), wants[1], dt, "short request")
    close(torch.cat([a[2], b[2]]), wants[2], dt, "third request")


# ----------------------------------------------------------------------------------------------- gated attention

def attention_cfg(p):
    return dict(heads=p["num_heads"], kv_heads=p["num_kv_heads"], dim=p["dim"], vdim=p["vdim"], scale=p["scale"],
                mask=dict(size=p["chunk"]), rot=dict(base=p["rot_base"], dims=p["rot_dims"], scaling=p.get("rot_scaling")))


ATTENTIONS = [
    dict(num_heads=4, num_kv_heads=2, dim=32, vdim=32, scale=0.2, rot_dims=32, rot_base=50.0, chunk=24,       # a block of positions that is no multiple of a page
         rot_scaling=dict(factor=8.0, low=1.0, high=4.0, original=64)),
    dict(num_heads=3, num_kv_heads=3, dim=16, vdim=48, scale=0.3, rot_dims=8, rot_base=1e4, chunk=16),        # values wider than keys, a block = a page
    dict(num_heads=6, num_kv_heads=1, dim=64, vdim=32, scale=0.11, rot_dims=64, rot_base=1e6, chunk=40),      # one key head for all, keys wider than values
]


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("params", ATTENTIONS)
def test_gated_attention_whole_in_portions_and_token_by_token(dt, params):
    rt = rt_for(dt)
    hidden, T = 40, 100
    mixer = build("mixer", "gated_attention", hidden_size=hidden, eps=1e-5, **params)
    W = bind_random(mixer, rt, 7)
    x = inputs(T, hidden, 3, dt)
    want = pg.chunked_attention(x, W, "p.", attention_cfg(params), 1e-5)
    h = Harness(mixer, rt, pages=10)
    close(run_in_portions(h, x, [T]), want, dt, "whole")
    close(run_in_portions(h, x, [23, 2, 30, 1, 1, 20, 2, 21]), want, dt, "portions")        # pages were used before
    close(run_in_portions(h, x, [1] * T), want, dt, "token by token")
    assert h.manager.num_free(0) == 9


def test_frequencies_are_rescaled_by_wavelength():
    from mini_inference_engine_b200.parts.rope import rotary_frequencies
    rot = dict(base=50.0, dims=32, scaling=dict(factor=8.0, low=1.0, high=4.0, original=64))
    got, plain = rotary_frequencies(32, 50.0, rot["scaling"]), rotary_frequencies(32, 50.0)
    assert torch.allclose(got, pg.frequencies(rot), rtol=1e-6)
    ratio = (got / plain).tolist()
    assert ratio[0] == 1.0 and abs(ratio[-1] - 1 / 8) < 1e-6 and any(1 / 8 + 1e-3 < r < 1 - 1e-3 for r in ratio)
    pytest.mark.gpu  # (needs no device)


def standout_case(hidden, params, query, planted, dt):
    """Inputs and weights for which the key at ``planted`` scores far above all others for the query at ``query``:
    W_k = -W_q and the planted input is minus the query's, so its key equals the query (and the query's own key
    is its opposite), while its value is minus the query's own."""
    wq = torch.randn(params["num_heads"] * params["dim"], hidden, generator=torch.Generator().manual_seed(1)) * hidden ** -0.5
    x = inputs(query + 1, hidden, 100 + query, dt)
    x[planted] = -x[query]
    return x, {"q": wq, "k": -wq, "q.norm": torch.ones(wq.shape[0]), "k.norm": torch.ones(wq.shape[0])}


STANDOUT = dict(num_heads=2, num_kv_heads=2, dim=16, vdim=16, scale=1.5, rot_dims=0, rot_base=1e4, chunk=24)
STANDOUT_PAIRS = ((70, 48), (70, 47), (71, 48), (95, 72), (95, 71), (48, 47), (200, 192), (200, 191), (200, 3), (23, 0), (24, 0))


def standout_plain(W, query, planted, dt):
    x, _ = standout_case(32, STANDOUT, query, planted, dt)
    Wt = dict(W)
    Wt["p.temp"] = torch.ones(2)
    cfg = attention_cfg(STANDOUT)
    want = pg.chunked_attention(x, Wt, "p.", cfg, 1e-5)
    moved = x.clone()
    moved[planted] = inputs(1, 32, 999, dt)[0]
    seen = (want[query] - pg.chunked_attention(moved, Wt, "p.", cfg, 1e-5)[query]).abs().max() > 0.2 * want[query].abs().max()
    return x, want, bool(seen)


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("decode", [False, True])
def test_a_key_that_stands_out_just_inside_and_just_outside_the_block(dt, decode):
    """Where the mask lets the query see the planted key the output is that key's value, where not it is something
    else -- an edge that is one position off shows in every entry of the output."""
    rt = rt_for(dt)
    mixer = build("mixer", "gated_attention", hidden_size=32, eps=1e-5, head_temp=False, **STANDOUT)
    W = bind_random(mixer, rt, 8, standout_case(32, STANDOUT, 1, 0, dt)[1])
    for query, planted in STANDOUT_PAIRS:
        x, want, seen = standout_plain(W, query, planted, dt)
        assert seen == (planted // 24 == query // 24), "the plain implementation disagrees with the mask's rule"
        h = Harness(mixer, rt, pages=16)
        got = run_in_portions(h, x, [query, 1] if decode else ([5, query - 4] if query > 5 else [query + 1]))
        close(got[query], want[query], dt, f"query {query}, planted key {planted}")


# ----------------------------------------------------------------------------------------------- gated linear recurrence

RECURRENCES = [dict(width=48, blocks=3, taps=4), dict(width=40, blocks=1, taps=2), dict(width=64, blocks=8, taps=5),
               dict(width=33, blocks=1, taps=1)]


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("params", RECURRENCES)
def test_gated_recurrence_whole_in_portions_and_token_by_token(dt, params):
    rt = rt_for(dt)
    hidden, T = 24, 150
    mixer = build("mixer", "gated_linear_recurrence", hidden_size=hidden, **params)
    W = bind_random(mixer, rt, 9)
    m = dict(width=params["width"], blocks=params["blocks"], conv=params["taps"])
    x = inputs(T, hidden, 4, dt)
    want = pg.gated_recurrence(x, W, "p.", m)
    h = Harness(mixer, rt)
    close(run_in_portions(h, x, [T]), want, dt, "whole (scanned in segments)")
    close(run_in_portions(h, x, [2, 1, 1, 2, 70, 3, 1, 64, 2, 4]), want, dt, "portions shorter than the convolution")
    close(run_in_portions(h, x, [1] * T), want, dt, "token by token")


@pytest.mark.parametrize("dt", DTYPES)
def test_gated_recurrence_keeps_a_slowly_decaying_state_and_batches(dt):
    rt = rt_for(dt)
    hidden = 16
    mixer = build("mixer", "gated_linear_recurrence", hidden_size=hidden, width=32, blocks=2, taps=3)
    W = bind_random(mixer, rt, 10, {"lam": torch.full((32,), -7.0)})          # a close to 1: the state forgets slowly
    m = dict(width=32, blocks=2, conv=3)
    xs = [inputs(n, hidden, 20 + i, dt) for i, n in enumerate((260, 3, 90))]
    xs[0][1] *= 20.0
    wants = [pg.gated_recurrence(x, W, "p.", m) for x in xs]
    quiet = xs[0].clone()
    quiet[1] /= 20.0
    assert (pg.gated_recurrence(quiet, W, "p.", m)[-1] - wants[0][-1]).abs().max() > 0.02 * wants[0][-1].abs().max()
    h = Harness(mixer, rt, slots=3)
    rcs = [h.new() for _ in xs]
    a = h.step([(rcs[0], xs[0][:200]), (rcs[1], xs[1][:2]), (rcs[2], xs[2][:89])])
    b = h.step([(rcs[2], xs[2][89:]), (rcs[1], xs[1][2:]), (rcs[0], xs[0][200:])])
    close(torch.cat([a[0], b[2]]), wants[0], dt, "long request")
    close(torch.cat([a[1], b[1]]), wants[1], dt, "short request")
    close(torch.cat([a[2], b[0]]), wants[2], dt, "third request")


# ----------------------------------------------------------------------------------------------- side by side

@pytest.mark.parametrize("dt", DTYPES)
def test_mixers_side_by_side_under_the_post_norm(dt):
    """The parallel mixer hands its branches to the block's norm: together they must give
    norm(alpha x + mean of the normed branches)."""
    from mini_inference_engine_b200.config import PartSpec
    rt = rt_for(dt)
    hidden, T, eps = 32, 50, 1e-5
    att = dict(num_heads=2, num_kv_heads=1, dim=16, vdim=32, scale=0.25, rot_dims=16, rot_base=1e4, chunk=20)
    rec = dict(width=24, blocks=2, taps=4)
    mixer = build("mixer", "parallel", hidden_size=hidden, branches={
        "left": PartSpec("gated_attention", dict(hidden_size=hidden, eps=eps, **att)),
        "right": PartSpec("gated_linear_recurrence", dict(hidden_size=hidden, **rec))})
    W = bind_random(mixer, rt, 11)
    norm = build("norm", "group_rmsnorm", size=hidden, eps=eps, groups=4)
    Wn = bind_random(norm, rt, 12, {"weight": torch.randn(hidden)})
    x = pg.group_norm(inputs(T, hidden, 5, dt), torch.ones(hidden), 4, eps).to(dt).float()
    m = dict(left=attention_cfg(att), right=dict(width=24, blocks=2, conv=4))
    want = pg.group_norm(3.0 * x + pg.parallel_mixer(x, W, "p.", m, eps), Wn["p.weight"], 4, eps)
    h = Harness(mixer, rt)
    for portions in ([T], [7, 1, 40, 2]):
        branches = run_in_portions(h, x, portions)                   # [T, 2, hidden]
        res = x.clone().to(DEV)
        norm.apply(res, tuple(branches[:, i].contiguous().to(DEV) for i in range(2)), tuple(mixer.out_weights), alpha=3.0, coef=0.5)
        close(res, want, dt, f"portions {portions}")
