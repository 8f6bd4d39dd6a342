"""The mechanisms of the Kebudra design one by one, built through the part registry with sizes of their own, against
the plain functions of ``plain_kebudra``: Dynamic Tanh over a stream in several copies with its connections, the scaled
embedding, differential attention, latent attention, the gated delta rule and the routed experts.  Mixers run a
sequence whole, in portions down to one token, and several requests in one batch, from state slots and pages that other
requests used before; where random weights would hide a lost key or a lost state, weights and inputs are made so that
it shows."""
import math

import pytest
import torch

import plain_kebudra as pk
import test_getizen_parts_gpu as harness
import helpers

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = [torch.float32, torch.bfloat16]
rt_for, build, bind_random, Harness, run_in_portions, inputs = (harness.rt_for, harness.build, harness.bind_random, harness.Harness,
                                                                harness.run_in_portions, harness.inputs)


def close(got, want, dtype, what=""):
    """The framework's bound in float32.  In bfloat16 twice its bound for a single kernel: a mixer here rounds its
    activations at up to four places in a row (and differential attention subtracts two rounded outputs), while the plain
    implementation rounds nothing."""
    if dtype == torch.bfloat16:
        got, want = got.float().cpu(), want.float().cpu()
        assert got.shape == want.shape and torch.isfinite(got).all(), what
        scale = max(want.abs().max().item(), 1e-6)
        err = (got - want).abs().max().item()
        assert err <= 4e-2 * scale, f"{what}: max abs error {err:.3e} > 0.04 x {scale:.3e}"
        return err / scale
    return helpers.close(got, want, dtype, what)


def weights_of(W):
    return {k[2:]: v for k, v in W.items()}


# ----------------------------------------------------------------------------------------------- stream, norm, embedding

@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("streams,width", [(1, 48), (2, 50), (4, 64), (8, 12)])
def test_dynamic_tanh_reads_and_writes_a_stream_in_copies(dt, streams, width):
    rt = rt_for(dt)
    T, S = 9, streams
    norm = build("norm", "dynamic_tanh", size=width, streams=S)
    Wn = weights_of(bind_random(norm, rt, 1, {"alpha": torch.tensor(0.7)}))
    before, after = build("connection", "hyper", streams=S), build("connection", "hyper", streams=S)
    Wb, Wa = weights_of(bind_random(before, rt, 2)), weights_of(bind_random(after, rt, 3))
    from mini_inference_engine_b200.parts.block import PendingUpdate
    g = torch.Generator().manual_seed(5)
    x = torch.randn(T, S, width, generator=g)
    y = torch.randn(T, width, generator=g).to(dt).float()
    # the write of the sublayer before, then the read of the next one through the norm
    x_new = torch.einsum("sr,tsw->trw", Wb["mix"], x) + Wb["out"][None, :, None] * y[:, None, :]
    want = pk.dyt(torch.einsum("r,trw->tw", Wa["in"], x_new), Wn["alpha"], Wn["weight"], Wn["b"])
    res = x.reshape(T, S * width).clone().to(DEV)
    out = norm.read(res, PendingUpdate(y.to(dt).to(DEV), before), after)
    close(res.view(T, S, width), x_new, torch.float32, "the copies after the write")
    close(out, want, dt, "what the next sublayer reads")
    # nothing pending: the copies stay as they are
    res = x.reshape(T, S * width).clone().to(DEV)
    out = norm.read(res, None, after)
    assert torch.equal(res.cpu(), x.reshape(T, S * width))
    close(out, pk.dyt(torch.einsum("r,trw->tw", Wa["in"], x), Wn["alpha"], Wn["weight"], Wn["b"]), dt, "a read without a write")
    # in front of the output head: some rows only, the plain sum of the copies, the stream untouched
    rows = torch.tensor([7, 0, 7, 3], dtype=torch.int32, device=DEV)
    res = x.reshape(T, S * width).clone().to(DEV)
    out = norm(PendingUpdate(y.to(dt).to(DEV), before), res, rows=rows)
    assert torch.equal(res.cpu(), x.reshape(T, S * width))
    close(out, pk.dyt(x_new.sum(1), Wn["alpha"], Wn["weight"], Wn["b"])[rows.cpu().long()], dt, "gathered rows")


@pytest.mark.parametrize("dt", DTYPES)
def test_dynamic_tanh_over_one_copy_is_a_fused_sum_and_norm(dt):
    rt = rt_for(dt)
    norm = build("norm", "dynamic_tanh", size=40)
    Wn = weights_of(bind_random(norm, rt, 4))
    res, y = torch.randn(5, 40), torch.randn(5, 40).to(dt).float()
    r = res.clone().to(DEV)
    out = norm(y.to(dt).to(DEV), r)
    close(r, res + y, torch.float32, "res += delta")
    close(out, pk.dyt(res + y, Wn["alpha"], Wn["weight"], Wn["b"]), dt, "norm(res)")


@pytest.mark.parametrize("dt", DTYPES)
def test_scaled_embedding_opens_every_copy(dt):
    from mini_inference_engine_b200.engine.batch import BatchBuilder, BatchRow
    rt = rt_for(dt)
    emb = build("embedding", "scaled_embedding", vocab_size=50, hidden_size=24, scale=3.25, copies=3)
    W = weights_of(bind_random(emb, rt, 6))
    toks = [4, 49, 0, 17]
    ctx = BatchBuilder(1, 16, DEV).build([BatchRow(toks, 0, [[1]], 0, [])])
    res = emb.forward(ctx)
    assert res.dtype == torch.float32 and res.shape == (4, 72)
    want = (W["weight"][toks] * 3.25)[:, None, :].expand(4, 3, 24).reshape(4, 72)
    assert torch.equal(res.cpu(), want)                        # a float32 product of a bfloat16 value and the scale: exact either way


# ----------------------------------------------------------------------------------------------- attention mixers

def diff_params(**kw):
    p = dict(hidden_size=40, num_heads=4, num_kv_heads=2, dim=16, vdim=32, scale=0.3, diff=0.2, eps=1e-5)
    p.update(kw)
    return p


def latent_params(**kw):
    p = dict(hidden_size=40, num_heads=3, dim=16, rot_dim=8, vdim=24, q_rank=20, kv_rank=28, scale=0.25, rot_dims=8, rot_base=100.0,
             eps=1e-5)
    p.update(kw)
    return p


def plain_mixer(kind, params, W, x):
    T = x.shape[0]
    if kind != "channel_delta" and not params.get("gate", True):
        # the plain functions always gate; a gate of zero logits halves the heads, and the output projection is linear
        rows = params["num_heads"] * (1 if kind == "differential_attention" else params["vdim"])
        return 2.0 * plain_mixer(kind, dict(params, gate=True), dict(W, g=torch.zeros(rows, params["hidden_size"])), x)
    if kind == "differential_attention":
        m = dict(heads=params["num_heads"], kv_heads=params["num_kv_heads"], dim=params["dim"], vdim=params["vdim"],
                 scale=params["scale"], diff=params["diff"])
        return pk.differential_attention(x, W, m, params["eps"])[0]
    if kind == "latent_attention":
        m = dict(heads=params["num_heads"], dim=params["dim"], rot_dim=params["rot_dim"], vdim=params["vdim"], kv_rank=params["kv_rank"],
                 scale=params["scale"], rot=dict(dims=params["rot_dims"], base=params["rot_base"]))
        return pk.latent_attention(x, W, m, params["eps"], torch.arange(T))
    m = dict(heads=params["num_heads"], kv_heads=params["num_kv_heads"], dim=params["dim"], vdim=params["vdim"])
    return pk.channel_delta(x, W, m, params["eps"])


ATTENTION_CASES = [
    ("differential_attention", diff_params()),
    ("differential_attention", diff_params(num_heads=3, num_kv_heads=3, dim=32, vdim=16, diff=0.5)),       # keys wider than values, no grouping
    ("differential_attention", diff_params(num_heads=2, num_kv_heads=1, dim=64, vdim=64, scale=0.125)),    # heads of 64: the tensor-core kernels
    ("differential_attention", diff_params(num_heads=1, num_kv_heads=1, dim=48, vdim=128, gate=False)),    # one head, heads of 128, no gate
    ("differential_attention", diff_params(num_heads=2, num_kv_heads=1, dim=24, vdim=160)),                # heads beyond 128: the CUDA-core kernel in both modes
    ("latent_attention", latent_params()),
    ("latent_attention", latent_params(num_heads=1, dim=32, rot_dim=32, vdim=64, rot_dims=16)),            # rotation over half the rotated part
    ("latent_attention", latent_params(num_heads=2, dim=96, rot_dim=32, vdim=48, kv_rank=16, q_rank=8)),   # heads of 128, ranks below the head size
    ("latent_attention", latent_params(num_heads=2, dim=8, rot_dim=0, vdim=40, rot_dims=0, gate=False)),   # nothing rotated, values wider than keys
]


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("kind,params", ATTENTION_CASES)
def test_attention_whole_in_portions_and_in_batches(dt, kind, params):
    rt = rt_for(dt)
    mixer = build("mixer", kind, **params)
    W = weights_of(bind_random(mixer, rt, 11))
    h = Harness(mixer, rt, pages=24, slots=3)
    hid = params["hidden_size"]
    x = inputs(75, hid, 1, dt)
    want = plain_mixer(kind, params, W, x)
    close(run_in_portions(h, x, [75]), want, dt, "whole")
    close(run_in_portions(h, x, [33, 1, 1, 14, 2, 17, 1, 1, 1, 1, 1, 1, 1]), want, dt, "portions and single tokens")
    # three unequal requests in one batch, each continued, on pages that the runs above gave back
    xs = [inputs(n, hid, 20 + i, dt) for i, n in enumerate((40, 9, 61))]
    wants = [plain_mixer(kind, params, W, xi) for xi in xs]
    rcs = [h.new() for _ in xs]
    cuts = [(17, 23), (8, 1), (60, 1)]
    first = h.step([(rc, xi[:a]) for rc, xi, (a, _) in zip(rcs, xs, cuts)])
    second = h.step([(rc, xi[a:]) for rc, xi, (a, _) in zip(rcs, xs, cuts)])
    for i, (f, s) in enumerate(zip(first, second)):
        close(torch.cat([f, s], 0), wants[i], dt, f"request {i} of a batch")
    for rc in rcs:
        h.free(rc)
    h.manager.check()


def planted_overrides(mixer, kind, params):
    """Differential attention: both maps' keys are made by the matrix of the group's first query head, so that equal
    inputs score |W_q x|^2, far above everything else.  (Latent attention needs no help: its planted score stands out.)"""
    if kind != "differential_attention":
        return {}
    from mini_inference_engine_b200.weights.random_init import random_tensor
    H, G, D, hid = params["num_heads"], params["num_kv_heads"], params["dim"], params["hidden_size"]
    q = random_tensor(12, "q", mixer.tensor_specs()["q"], torch.bfloat16).float().view(G, H // G, 2, D, hid)
    return {"k": q[:, 0].reshape(G * 2 * D, hid)}


def planted_inputs(kind, params, W, dt, far, T):
    """Inputs whose token ``far`` is three times the last three tokens' input plus something of its own, the rest small;
    the plain output with it, and with a small token in its place."""
    hid = params["hidden_size"]
    x = inputs(T, hid, 2, dt) * 0.1
    g = torch.Generator().manual_seed(9)
    mark = torch.randn(hid, generator=g).to(dt).float() * 1.2
    small = x[far].clone()
    x[far] = (3.0 * mark + torch.randn(hid, generator=g) * 1.2).to(dt).float()
    x[T - 3:] = mark
    without = x.clone()
    without[far] = small
    return x, plain_mixer(kind, params, W, x), plain_mixer(kind, params, W, without)


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("kind", ["differential_attention", "latent_attention"])
@pytest.mark.parametrize("far", [0, 15, 16, 250])
def test_a_planted_key_far_back_decides_the_output(dt, kind, far):
    """One key among 300 answers the last queries with a score far above all others (its input is three times theirs plus
    something of its own, so its value is unlike the rest).  A key that is lost at a page border, or by a decoding step,
    changes the output altogether."""
    rt = rt_for(dt)
    params = diff_params(num_heads=2, num_kv_heads=1, scale=1.0) if kind == "differential_attention" else latent_params(num_heads=2, scale=1.0)
    mixer = build("mixer", kind, **params)
    W = weights_of(bind_random(mixer, rt, 12, planted_overrides(mixer, kind, params)))
    hid, T = params["hidden_size"], 300
    x, want, lost = planted_inputs(kind, params, W, dt, far, T)
    assert (want[-3:] - lost[-3:]).abs().max() > 0.05 * want[-3:].abs().max(), "the planted key must matter"
    h = Harness(mixer, rt, pages=24, slots=1)
    close(run_in_portions(h, x, [T]), want, dt, "whole")
    close(run_in_portions(h, x, [T - 5, 2, 1, 1, 1]), want, dt, "the last queries decoded alone")


# ----------------------------------------------------------------------------------------------- gated delta rule

def delta_params(**kw):
    p = dict(hidden_size=40, num_heads=4, num_kv_heads=2, dim=16, vdim=24, taps=4, eps=1e-5, decay_rank=8, gate_rank=12)
    p.update(kw)
    return p


DELTA_CASES = [delta_params(), delta_params(num_heads=1, num_kv_heads=1, dim=48, vdim=8, taps=1),
               delta_params(num_heads=2, num_kv_heads=2, dim=128, vdim=40, taps=2), delta_params(num_heads=3, num_kv_heads=1, dim=200, vdim=16, taps=6),
               delta_params(num_heads=2, num_kv_heads=1, dim=8, vdim=130, taps=3)]


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("params", DELTA_CASES)
def test_delta_rule_whole_in_portions_and_in_batches(dt, params):
    rt = rt_for(dt)
    mixer = build("mixer", "channel_delta", **params)
    W = weights_of(bind_random(mixer, rt, 13))
    h = Harness(mixer, rt, pages=8, slots=3)
    hid = params["hidden_size"]
    x = inputs(70, hid, 3, dt)
    want = plain_mixer("channel_delta", params, W, x)
    close(run_in_portions(h, x, [70]), want, dt, "whole")
    close(run_in_portions(h, x, [1, 1, 2, 30, 1, 1, 1, 3, 2, 28]), want, dt, "portions shorter than the convolution")
    xs = [inputs(n, hid, 30 + i, dt) for i, n in enumerate((25, 3, 44))]
    wants = [plain_mixer("channel_delta", params, W, xi) for xi in xs]
    rcs = [h.new() for _ in xs]                        # slots that the runs above used and gave back
    cuts = [(24, 1), (1, 2), (2, 42)]
    first = h.step([(rc, xi[:a]) for rc, xi, (a, _) in zip(rcs, xs, cuts)])
    second = h.step(list(reversed([(rc, xi[a:]) for rc, xi, (a, _) in zip(rcs, xs, cuts)])))
    for i, (f, s) in enumerate(zip(first, reversed(second))):
        close(torch.cat([f, s], 0), wants[i], dt, f"request {i} of a batch")


@pytest.mark.parametrize("dt", DTYPES)
def test_delta_rule_state_holds_a_far_token_and_long_decoding(dt):
    """Decays of almost 1 (A_log far below zero): what the first token wrote is still read 260 tokens later, most of
    them decoded one by one.  A state that is lost, or cleared between steps, shows at once."""
    rt = rt_for(dt)
    params = delta_params(num_heads=2, num_kv_heads=2)
    mixer = build("mixer", "channel_delta", **params)
    W = weights_of(bind_random(mixer, rt, 14, {"A_log": torch.full((2,), -9.0)}))
    x = inputs(260, params["hidden_size"], 4, dt)
    x[0] *= 4.0
    want = plain_mixer("channel_delta", params, W, x)
    gone = plain_mixer("channel_delta", params, W, x[1:])
    assert (want[-1] - gone[-1]).abs().max() > 0.02 * want[-1].abs().max(), "the first token must still matter at the end"
    h = Harness(mixer, rt, pages=24, slots=1)
    close(run_in_portions(h, x, [10] + [1] * 250), want, dt, "long decoding")


# ----------------------------------------------------------------------------------------------- routed experts

@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("experts,top,ff", [(6, 2, 24), (5, 1, 10), (3, 3, 16), (1, 1, 8), (17, 4, 33), (40, 2, 16)])
def test_routed_experts(dt, experts, top, ff):
    from mini_inference_engine_b200.parts import StepContext  # noqa: F401  (the part takes the step's context and ignores it)
    rt = rt_for(dt)
    hid = 40
    ffw = build("feed_forward", "routed_experts", hidden_size=hid, num_experts=experts, top=top, expert_size=ff)
    W = weights_of(bind_random(ffw, rt, 15, {"router": torch.randn(experts, hid)}))       # logits well apart: no close calls
    for T in (1, 3, 50, 200):
        x = inputs(T, hid, 40 + T, dt)
        want = pk.routed_experts(x, W, dict(router=dict(top=top)))
        got = ffw.forward(x.to(dt).to(DEV), None)
        assert got.dtype == torch.float32
        close(got, want, dt, f"{T} tokens")


def test_router_takes_the_largest_logits_and_weighs_by_their_softmax():
    from mini_inference_engine_b200.kernels import ops
    z = torch.tensor([[0.5, 3.0, -1.0, 3.0, 2.0], [-5.0, -7.0, -6.0, -5.5, -9.0]], device=DEV)
    ids, w = ops.moe_route(z, 3)
    assert ids.cpu().tolist() == [[1, 3, 4], [0, 3, 2]]              # equal logits: the lower index first
    for r in range(2):
        want = torch.softmax(z[r].cpu()[ids[r].cpu().long()], 0)
        assert torch.allclose(w[r].cpu(), want, atol=1e-6)
    assert math.isclose(float(w.sum()), 2.0, rel_tol=1e-6)
    # the same choice with the logits computed in the kernel, from float32 and from bfloat16 inputs
    g = torch.Generator().manual_seed(3)
    wr = torch.randn(11, 70, generator=g).to(DEV)
    for dt in DTYPES:
        x = torch.randn(9, 70, generator=g).to(dt).to(DEV)
        logits = torch.empty(9, 11, device=DEV)
        ids2, w2 = ops.moe_router(x, wr, 4, logits)
        want = x.float() @ wr.t()
        assert torch.allclose(logits, want, atol=1e-4, rtol=1e-5)
        ids3, w3 = ops.moe_route(want.contiguous(), 4)
        assert torch.equal(ids2, ids3) and torch.allclose(w2, w3, atol=1e-5)


@pytest.mark.parametrize("dim,vdim", [(16, 32), (64, 64), (48, 128), (24, 160)])
def test_attention_kernels_leave_their_output_in_float32(dim, vdim, monkeypatch):
    """The option that differential attention uses in bfloat16 mode: every paged attention kernel (decoding, portions on
    mma.sync and on tcgen05, the CUDA-core kernel for wide heads) writes float32 when handed a float32 output; rounded to
    bfloat16 it is what the kernel writes otherwise."""
    from mini_inference_engine_b200.parts import attention as part
    rt = rt_for(torch.bfloat16)
    params = diff_params(num_heads=2, num_kv_heads=1, dim=dim, vdim=vdim)
    mixer = build("mixer", "differential_attention", **params)
    bind_random(mixer, rt, 16)
    h = Harness(mixer, rt, pages=12, slots=1)
    seen = []
    plain = part.attn_kernels.attention

    def both(q, ctx, cache, out, *a, **k):
        plain(q, ctx, cache, out, *a, **k)
        rounded = torch.empty_like(out, dtype=torch.bfloat16)
        plain(q, ctx, cache, rounded, *a, **k)
        seen.append((out.clone(), rounded))
        return out

    monkeypatch.setattr(part.attn_kernels, "attention", both)
    x = inputs(70, params["hidden_size"], 5, torch.bfloat16)
    run_in_portions(h, x, [40, 1, 1, 27, 1])             # portions and single tokens: both kinds of kernel
    assert len(seen) == 5
    for f32, b16 in seen:
        assert f32.dtype == torch.float32 and torch.isfinite(f32).all()
        err = (f32 - b16.float()).abs().max().item()
        assert err <= 2 ** -7 * max(f32.abs().max().item(), 1e-6), f"float32 and bfloat16 outputs differ by {err:.3e}"
        assert (f32 != f32.bfloat16().float()).any(), "the float32 output carries more than bfloat16 holds"
