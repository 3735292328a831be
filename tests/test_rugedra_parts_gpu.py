"""Each mechanism of the Rugedra design alone on the GPU, against the plain implementation's
function for it (`tests/plain_rugedra.py`) or against the plain stand-in of a kernel
(`tests/ref_ops.py`): layer norm with scaled residual add, learned positions, the squared-relu
and the routed feed-forward (routing with groups, experts nobody chooses, several tiles per
expert), the latent attention over its paged rows (far keys, page borders, the first tokens),
the gated delta rule (portions, single tokens, slots used again), in both precisions."""

from __future__ import annotations

import pytest
import torch

from inference_engine_b200.config.spec import PartSpec
from inference_engine_b200.parts import BuildEnv, CacheBinding, build_part
from tests import plain_rugedra as P
from tests import rugedra_configs as R

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


def _tol(dtype, scale=1.0):
    return dict(atol=4e-5 * scale, rtol=1e-4) if dtype == "float32" else dict(atol=5e-2 * scale, rtol=5e-2)


def _total(t):
    return t.float().sum(0) if t.dim() == 3 else t.float()


def _ops():
    from inference_engine_b200.kernels import get_ops

    return get_ops("cuda")


class _Ctx:
    def __init__(self, n):
        from inference_engine_b200.engine.workspace import Workspace

        self.ops, self.ws, self.num_tokens = _ops(), Workspace("cuda"), n


def _env(width, dtype, positions=None, max_positions=512):
    return BuildEnv(width, dtype, max_positions, positions or {}, "cuda")


def _bf(t):
    return t.to(torch.bfloat16)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [72, 1000, 5000])
def test_layer_norm_adds_the_scaled_delta(dtype, width):
    env = _env(width, dtype)
    norm = build_part("norm", PartSpec("layer", {"weight": "w", "eps": 2e-5}), env)
    w = _bf(1 + 0.1 * torch.randn(width))
    norm.bind({"w": w.cuda()}, env)
    h = torch.randn(7, width, device="cuda") * 3 + 1.5
    parts = torch.randn(3, 7, width, device="cuda")
    h0 = h.clone()
    out = norm.add_norm(h, parts, _Ctx(7), delta_scale=0.7)
    x = h0 + 0.7 * parts.sum(0)
    torch.testing.assert_close(h, x, atol=2e-6, rtol=1e-6)
    torch.testing.assert_close(out.float().cpu(), P.layer_norm(x.cpu().double(), w.double(), 2e-5).float(), **_tol(dtype))
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device="cuda")
    kept = h.clone()
    picked = norm.add_norm(h, parts[0], _Ctx(3), rows=rows, delta_scale=0.5)
    assert torch.equal(h, kept)  # picking rows leaves the residual stream alone
    y = (kept + 0.5 * parts[0])[rows.long()]
    torch.testing.assert_close(picked.float().cpu(), P.layer_norm(y.cpu().double(), w.double(), 2e-5).float(), **_tol(dtype))


def test_rms_norm_takes_a_delta_scale_too():
    env = _env(80, "float32")
    norm = build_part("norm", PartSpec("rms", {"weight": "w", "eps": 1e-6}), env)
    w = _bf(1 + 0.1 * torch.randn(80))
    norm.bind({"w": w.cuda()}, env)
    h, d = torch.randn(5, 80, device="cuda"), torch.randn(5, 80, device="cuda")
    x = (h + 0.25 * d).cpu()
    out = norm.add_norm(h, d, _Ctx(5), delta_scale=0.25)
    torch.testing.assert_close(out.cpu(), x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float(), atol=3e-6, rtol=1e-5)


@pytest.mark.parametrize("dtype", DTYPES)
def test_learned_positions_and_scaled_head(dtype):
    env = _env(40, dtype)
    pos = build_part("position", PartSpec("learned", {"weight": "pos", "positions": 33}), env)
    table = _bf(torch.randn(33, 40))
    pos.bind({"pos": table.cuda()}, env)
    ctx = _Ctx(4)
    ctx.positions = torch.tensor([32, 0, 7, 7], dtype=torch.int32, device="cuda")
    h = torch.randn(4, 40, device="cuda")
    h0 = h.clone()
    pos.apply_to_embedding(h, ctx)
    torch.testing.assert_close(h.cpu(), h0.cpu() + table.float()[ctx.positions.cpu().long()])
    ctx.positions = torch.tensor([33, 0, 7, 7], dtype=torch.int32, device="cuda")
    pos.apply_to_embedding(h, ctx)
    with pytest.raises(Exception, match="position"):
        ctx.ops.check_errors()
    head = build_part("head", PartSpec("linear", {"weight": "head", "vocab_size": 50, "logit_scale": 0.3}), env)
    wh = _bf(torch.randn(50, 40))
    head.bind({"head": wh.cuda()}, env)
    x = torch.randn(4, 40).to(env.torch_dtype)
    torch.testing.assert_close(head.forward(x.cuda(), ctx).cpu(), x.float() @ wh.float().t() * 0.3, **_tol(dtype, 8))


@pytest.mark.parametrize("dtype", DTYPES)
def test_squared_relu_feed_forward(dtype):
    env = _env(72, dtype)
    ffn = build_part("feed_forward", PartSpec("relu2", {"up_proj": "up", "down_proj": "down", "intermediate_size": 100}), env)
    w = {"up": _bf(torch.randn(100, 72) * 0.2), "down": _bf(torch.randn(72, 100) * 0.2)}
    ffn.bind({k: v.cuda() for k, v in w.items()}, env)
    x = torch.randn(19, 72).to(env.torch_dtype)
    want = P.dense_ff(x.double(), {k: v.double() for k, v in w.items()}).float()
    torch.testing.assert_close(_total(ffn.forward(x.cuda(), _Ctx(19))).cpu(), want, **_tol(dtype, 8))


def _moe_part(env, mlp, hidden, seed):
    r = mlp["router"]
    ffn = build_part("feed_forward", PartSpec("routed_experts", {
        "router": "router", "expert_prefix": "e", "experts": r["experts"], "top": r["top"],
        "groups": r["groups"]["count"], "keep_groups": r["groups"]["keep"],
        "intermediate_size": mlp["expert"]["ff"], "limit": mlp["expert"]["limit"]}), env)
    g = torch.Generator().manual_seed(seed)
    w = {n: _bf(torch.randn(d.shape, generator=g) * (0.5 if n == "router" else 0.25)) for n, d in ffn.weights().items()}
    return ffn, w


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens,mlp,hidden", [
    (9, R.moe(40, 6, 3, 3, 2), 72),      # few tokens, groups of two of which two are kept
    (700, R.moe(96, 8, 2, 1, 1), 64),    # several tiles per expert
    (150, R.moe(20, 5, 1, 5, 1), 52),    # one expert per token, rows that are not multiples of 8
])
def test_routed_feed_forward(dtype, tokens, mlp, hidden):
    env = _env(hidden, dtype)
    ffn, w = _moe_part(env, mlp, hidden, seed=tokens)
    w["router"][1] = -2.0 * w["router"][0]  # an expert that few choose beside a favourite
    ffn.bind({k: v.cuda() for k, v in w.items()}, env)
    x = torch.randn(tokens, hidden, generator=torch.Generator().manual_seed(1)).to(env.torch_dtype)
    ctx = _Ctx(tokens)
    out = ffn.forward(x.cuda(), ctx)
    assert out.shape == (mlp["router"]["top"], tokens, hidden)
    wd = {k: v.double() for k, v in w.items()}
    chosen, weights = P.route(x.double(), wd["router"], mlp)
    ids = ctx.ws.buffer("moe.ids", tokens, mlp["router"]["top"], torch.int32).cpu().long()
    got_w = ctx.ws.buffer("moe.weights", tokens, mlp["router"]["top"], torch.float32).cpu()
    assert torch.equal(ids, chosen), "the routing differs"
    torch.testing.assert_close(got_w, weights.float(), atol=2e-6, rtol=1e-5)
    want = P.moe_ff(x.double(), wd, mlp).float()
    torch.testing.assert_close(_total(out).cpu(), want, **_tol(dtype, 4))
    ctx.ops.check_errors()


class _OneMixer:
    def __init__(self, mixer):
        from inference_engine_b200.cache import PagedGroupSpec, StateGroupSpec
        from inference_engine_b200.parts import PagedKVRequest

        req = mixer.cache_request()
        self.paged_groups, self.state_groups = [], []
        if isinstance(req, PagedKVRequest):
            self.paged_groups = [PagedGroupSpec(1, req.num_kv_heads, req.head_dim, req.window, req.value_dim)]
        else:
            self.state_groups = [StateGroupSpec(1, tuple(req.shape))]


def _runner(mixer, env, pages=64, page_size=8, requests=2):
    from inference_engine_b200.cache import CacheManager, CacheStorage
    from inference_engine_b200.engine.runner import ModelRunner

    model = _OneMixer(mixer)
    cache = CacheManager(model.paged_groups, model.state_groups, pages, page_size, requests)
    storage = CacheStorage(cache, env.torch_dtype, "cuda")
    return ModelRunner(model, cache, storage, _ops(), "cuda", 64, requests), cache


def _feed(runner, cache, mixer, x, portions, env, rid="a"):
    """`x` through the mixer in portions, as one request; returns the outputs in order."""
    from inference_engine_b200.engine.batch import StepEntry

    cache.add_request(rid)
    outs, pos = [], 0
    for n in portions:
        cache.grow(rid, pos, pos + n)
        ctx, _ = runner.build_context([StepEntry(rid, [0] * n, pos, [])])
        runner.reset_fresh_state(ctx)
        out = mixer.forward(x[pos:pos + n].cuda().to(env.torch_dtype), ctx, CacheBinding(0, 0))
        outs.append(_total(out).cpu().clone())
        pos += n
    cache.free(rid)
    return torch.cat(outs)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes", [R.latent(3, 12, 8, 20, 20, rot_dims=4), R.latent(5, 8, 16, 8, 24, base=500.0),
                                   R.latent(1, 64, 32, 48, 96), R.latent(2, 16, 8, 16, 32, rot_dims=0),
                                   R.latent(16, 32, 16, 24, 128), R.latent(20, 16, 8, 16, 40)])
def test_latent_attention_mixer(dtype, sizes):
    width = 72
    env = _env(width, dtype)
    if sizes["rot"]["dims"]:
        rot = build_part("position", PartSpec("rotary", {"rotary_dim": sizes["rot"]["dims"], "theta": sizes["rot"]["base"],
                                                         "layout": "interleaved"}), env)
        rot.bind({}, env)
        env.positions = {"rot": rot}
    names = {"q": "q", "dkv": "dkv", "latent_norm": "dkv.norm", "uk": "uk", "uv": "uv", "gate": "g", "o": "o"}
    mixer = build_part("mixer", PartSpec("latent_attention", {
        "names": names, "heads": sizes["heads"], "dim": sizes["dim"], "rot_dim": sizes["rot_dim"], "vdim": sizes["vdim"],
        "kv_rank": sizes["kv_rank"], "scale": sizes["scale"], "eps": 1e-5,
        "position": "rot" if sizes["rot"]["dims"] else None}), env)
    g = torch.Generator().manual_seed(3)
    w = {}
    for n, d in mixer.weights().items():
        t = torch.randn(d.shape, generator=g) * 0.1
        w[n] = _bf(t * 4 if n in ("q", "dkv", "uk") else t + 1 if n == "dkv.norm" else t)
    mixer.bind({n: w[n].cuda() for n in w}, env)
    req = mixer.cache_request()
    assert (req.num_kv_heads, req.head_dim, req.value_dim) == (1, sizes["kv_rank"] + sizes["rot_dim"], 0)
    t = 77
    x = torch.randn(t, width, generator=g) * 0.8
    xq = x.to(env.torch_dtype).double()
    want = P.latent_attention(xq, {k: v.double() for k, v in w.items()}, "", sizes, 1e-5).float()
    runner, cache = _runner(mixer, env)
    # whole; portions that end on, just before and just after page borders (pages of 8); single tokens
    for portions in ([t], [8, 7, 2, 16, 1, 1, 23, 9, 2, 8]):
        got = _feed(runner, cache, mixer, x, portions, env)
        torch.testing.assert_close(got, want, **_tol(dtype, 2))
    _ops().check_errors()


@pytest.mark.parametrize("dtype", DTYPES)
def test_latent_rows_far_away_and_at_page_borders(dtype):
    """One key's score stands out among hundreds: the value that comes back is that key's latent
    part.  The key sits far back, on a page's last and first place, on the first position, and
    on the query's own place; the query is a prompt portion's or a decoded token's."""
    from inference_engine_b200.engine.batch import StepEntry
    from tests.ref_ops import RefOps

    tdt = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    heads, rank, rot, page = 3, 24, 8, 16
    row = rank + rot

    class M:
        from inference_engine_b200.cache import PagedGroupSpec
        paged_groups, state_groups = [PagedGroupSpec(1, 1, row, None, 0)], []

    from inference_engine_b200.cache import CacheManager, CacheStorage
    from inference_engine_b200.engine.runner import ModelRunner

    cache = CacheManager(M.paged_groups, [], 40, page, 2)
    storage = CacheStorage(cache, tdt, "cuda")
    runner = ModelRunner(M, cache, storage, _ops(), "cuda", 64, 2)
    total = 600
    g = torch.Generator().manual_seed(0)
    rows = torch.randn(total, row, generator=g)
    rows = rows / rows.norm(dim=-1, keepdim=True)
    cache.add_request("a")
    cache.grow("a", 0, total)
    table = cache.table(0, "a")
    k = storage.paged[0].k[0]
    for p in range(total):
        k[table[p // page], 0, p % page] = rows[p].to(tdt).cuda()
    for q_len, last in ((1, 599), (5, 599), (40, 300), (1, 16), (2, 1)):
        start = last + 1 - q_len
        ctx, _ = runner.build_context([StepEntry("a", [0] * q_len, start, [])])
        for target in (0, 15, 16, 17, last - 1, last, 255, 256):
            if target > start:  # visible to every query of the portion only if it is not ahead of the first
                continue
            q = torch.randn(q_len, heads, row, generator=g) * 0.1
            q[:, 1] += 40.0 * rows[target]  # head 1 asks for the target with a score nothing else reaches
            qd = q.reshape(q_len, heads * row).to(tdt).cuda()
            out = torch.empty(q_len, heads * rank, dtype=tdt, device="cuda")
            _ops().paged_attention(qd, k, k, ctx.groups[0].block_tables, ctx, heads, 1, row, page, 1.0, 0, out,
                                   value_dim=rank)
            ref = torch.empty(q_len, heads * rank, dtype=tdt)
            cpu_ctx = type("C", (), {"positions": ctx.positions.cpu(), "seq_of_token": ctx.seq_of_token.cpu(),
                                     "num_tokens": q_len})
            RefOps().paged_attention(qd.cpu(), k.cpu(), k.cpu(), ctx.groups[0].block_tables.cpu(), cpu_ctx, heads, 1,
                                     row, page, 1.0, 0, ref, value_dim=rank)
            torch.testing.assert_close(out.cpu().float(), ref.float(), **_tol(dtype))
            got = out.view(q_len, heads, rank)[:, 1].float().cpu()
            torch.testing.assert_close(got, rows[target, :rank].to(tdt).float().expand(q_len, rank), atol=2e-2, rtol=0)
    _ops().check_errors()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes", [R.delta(6, 2, 12, 20, 4), R.delta(2, 2, 40, 8, 2), R.delta(1, 1, 24, 24, 1),
                                   R.delta(4, 1, 64, 100, 3), R.delta(2, 1, 200, 16, 3), R.delta(1, 1, 300, 8, 2)])
def test_delta_rule_mixer(dtype, sizes):
    width = 56
    env = _env(width, dtype)
    names = {k: k for k in ("q", "k", "v", "A_log", "dt_bias", "a1", "a2", "g1", "g2", "o")}
    names.update(q_conv="q.conv", k_conv="k.conv", v_conv="v.conv", beta="b", out_norm="norm")
    mixer = build_part("mixer", PartSpec("channel_delta", {
        "names": names, "heads": sizes["heads"], "kv_heads": sizes["kv_heads"], "dim": sizes["dim"], "vdim": sizes["vdim"],
        "taps": sizes["conv"], "decay_rank": 6, "gate_rank": 10, "eps": 1e-5}), env)
    g = torch.Generator().manual_seed(5)
    w = {}
    for n, d in mixer.weights().items():
        t = torch.randn(d.shape, generator=g) * 0.15
        w[n] = _bf(t - 2.5 if n == "A_log" else t * 3 + 0.4 if n.endswith(".conv") else t + 1 if n == "norm" else t)
    mixer.bind({n: w[n].cuda() for n in w}, env)
    t = 61
    x = torch.randn(t, width, generator=g)
    xq = x.to(env.torch_dtype).double()
    want = P.channel_delta(xq, {k: v.double() for k, v in w.items()}, sizes, 1e-5).float()
    runner, cache = _runner(mixer, env)
    # whole; then portions shorter than the convolution, single tokens and a long one, in the slot the first
    # request used (it must start from zero again); then once more beside a request that holds the other slot
    for portions in ([t], [1, 1, 2, 1, 3, 30, 1, 1, 2, 19]):
        got = _feed(runner, cache, mixer, x, portions, env)
        torch.testing.assert_close(got, want, **_tol(dtype, 3))
    cache.add_request("other")
    got = _feed(runner, cache, mixer, x, [9, 2, 50], env, rid="b")
    torch.testing.assert_close(got, want, **_tol(dtype, 3))
    _ops().check_errors()


def test_delta_rule_batches_unequal_requests():
    """Three requests in one step (a portion, a single token, a longer portion) give what each
    gives alone; the kernels against their plain stand-ins on the same inputs."""
    from tests.ref_ops import RefOps

    heads, kvh, dim, vdim, taps = 4, 2, 24, 36, 3
    channels = 2 * kvh * dim + heads * vdim
    floats = heads * dim * vdim + (taps - 1) * channels
    g = torch.Generator().manual_seed(2)
    q_lens, slots = [5, 1, 17], [2, 0, 3]
    n = sum(q_lens)
    qkvb, a = torch.randn(n, channels + heads, generator=g), torch.randn(n, heads * dim, generator=g)
    conv, A_log, dt = torch.randn(channels, taps, generator=g), torch.randn(heads, generator=g) - 2, torch.randn(heads * dim, generator=g)
    state = torch.randn(5, floats, generator=g) * 0.3

    cpu = type("C", (), {"q_starts": [0, 5, 6], "q_lens": q_lens})
    outs = {}
    for dev in ("cpu", "cuda"):
        ops = RefOps() if dev == "cpu" else _ops()
        st = state.clone().to(dev)
        bufs = [torch.zeros(n, w, device=dev) for w in (kvh * dim, kvh * dim, heads * vdim, heads, heads * dim, heads * vdim)]
        ctx = cpu if dev == "cpu" else type("G", (), {
            "seq_of_token": torch.tensor([0] * 5 + [1] + [2] * 17, dtype=torch.int32, device=dev),
            "cu_q": torch.tensor([0, 5, 6, 23], dtype=torch.int32, device=dev), "num_seqs": 3})
        sl = torch.tensor(slots, dtype=torch.int32, device=dev)
        ops.delta_prep(qkvb.to(dev), a.to(dev), conv.to(dev), A_log.to(dev), dt.to(dev), st, sl, ctx, *bufs[:5],
                       heads, kvh, dim, vdim, taps)
        ops.delta_rule(*bufs[:5], st, sl, ctx, bufs[5], heads, kvh, dim, vdim)
        outs[dev] = [b.cpu() for b in bufs] + [st.cpu()]
    for got, want, what in zip(outs["cuda"], outs["cpu"], ("q", "k", "v", "beta", "decay", "out", "state")):
        torch.testing.assert_close(got, want, atol=3e-5, rtol=1e-4, msg=lambda m, what=what: f"{what}: {m}")
    assert torch.equal(outs["cuda"][6][1], state[1]) and torch.equal(outs["cuda"][6][4], state[4])  # other slots untouched


@pytest.mark.parametrize("dtype", DTYPES)
def test_headwise_linear_on_strided_views(dtype):
    tdt = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    n, heads, k, o = 37, 3, 20, 45
    g = torch.Generator().manual_seed(1)
    x_all = torch.randn(n, heads, k + 6, generator=g).to(tdt).cuda()
    out_all = torch.zeros(n, heads, o + 5, dtype=tdt, device="cuda")
    w = torch.randn(heads, o, k, generator=g).to(tdt).cuda()
    scale = torch.rand(n, heads, generator=g).cuda()
    _ops().headwise_linear(x_all[:, :, 3: 3 + k], w, out_all[:, :, 5:], row_scale=scale)
    want = torch.einsum("nhk,hok->nho", x_all[:, :, 3: 3 + k].float(), w.float()) * scale[..., None]
    torch.testing.assert_close(out_all[:, :, 5:].float(), want, **_tol(dtype, 4))
    assert float(out_all[:, :, :5].abs().max()) == 0.0
