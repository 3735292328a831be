"""The Ravapel design in the engine against the plain whole-sequence implementation
(`tests/plain_ravapel.py`): whole prompts, token-by-token decoding, portions down to two tokens,
mixed batches with pages and state slots used again, four configurations of odd sizes; every
mechanism alone against its plain function, with inputs made so that a key just inside or just
outside a chunk, a lost state or a wrong previous token shows; on the CPU through the plain
stand-ins of the kernels, on the GPU through the kernels in both precisions; long decoding; greedy
generation through the engine's own entry point and scheduler."""

from __future__ import annotations

from types import SimpleNamespace

import pytest
import torch

from tests import helpers as H
from tests import plain_ravapel as P
from tests import ravapel_configs as R

LENGTHS = [50, 21, 37, 64, 9, 1]
BF16_TOL = dict(atol=0.35, rtol=0.0, pos_rel_rms=0.08, rel_rms=0.04)
# (under these names the run's summary lists this file's comparisons: their bounds are measured)
LABEL = {"float32": "float32, Ravapel", "bfloat16": "bfloat16, Ravapel"}


def _requests(cfg, lengths=LENGTHS, seed=700):
    return {f"r{i}": torch.randint(0, cfg["vocab"], (n,), generator=torch.Generator().manual_seed(seed + i)).tolist()
            for i, n in enumerate(lengths)}


def _want(cfg, weights, requests):
    return {rid: P.forward(cfg, weights, toks, torch.float64).float() for rid, toks in requests.items()}


def _float32_bound(cfg, weights, requests, want) -> dict:
    """The 32-bit bound of a configuration: three times what rounding alone does to the plain
    implementation when it runs in 32-bit instead of 64-bit (a model of several passes over
    recurrent layers that forget slowly adds up more rounding than the engine's fixed bound for
    tiny models allows), and never below that fixed bound.  A lost state, a wrong key or a wrong
    previous token moves logits by 1e-2 and more."""
    worst = max(float((P.forward(cfg, weights, toks, torch.float32) - want[rid]).abs().max())
                for rid, toks in requests.items())
    return dict(atol=max(3 * worst, H.TOL["float32"]["atol"]), rtol=H.TOL["float32"]["rtol"])


def _bfloat16_bound(tmp_path, cfg, weights, requests, want) -> dict:
    """The bfloat16 bound of a configuration: three times what rounding does to the same requests
    on the plain stand-ins of the kernels run in bfloat16 (activations rounded between the parts,
    as the kernels round them), and never below the fixed bounds.  Peaked sigmoid weights and
    several passes over the same layers make a few positions move by a tenth under rounding
    alone; a lost or wrongly seen key moves them by several tenths."""
    from tests.ref_ops import RefOps

    room = sum(H.round64(len(t)) for t in requests.values())
    got = H.collect(_session(tmp_path / "bound", cfg, weights, "bfloat16", "cpu", RefOps(), room, 16),
                    H.trace_whole(requests))
    tol = dict(BF16_TOL)
    for rid in requests:
        diff = (got[rid].double() - want[rid].double()).abs()
        pos_rel = diff.pow(2).mean(-1).sqrt() / want[rid].double().pow(2).mean(-1).sqrt().clamp_min(1e-12)
        rel = float(diff.pow(2).mean().sqrt() / want[rid].double().pow(2).mean().sqrt())
        tol["atol"] = max(tol["atol"], 3 * float(diff.max()))
        tol["pos_rel_rms"] = max(tol["pos_rel_rms"], 3 * float(pos_rel.max()))
        tol["rel_rms"] = max(tol["rel_rms"], 3 * rel)
    return tol


def _session(tmp_path, cfg, weights, dtype, device, ops, max_tokens, page_size):
    from inference_engine_b200.engine.replay import ReplaySession

    folder = H.write_model_dir(tmp_path / f"m{abs(hash(str(cfg))) % 10**8}", cfg, weights)
    return ReplaySession(folder, dtype, max_tokens, device=device, ops=ops, page_size=page_size)


def _run_all_modes(tmp_path, name, dtype, device, ops, page_size=4, lengths=LENGTHS):
    cfg = R.CONFIGS[name]
    weights = R.make_weights(cfg, seed=11)
    requests = _requests(cfg, lengths)
    want = _want(cfg, weights, requests)
    tol = (_float32_bound(cfg, weights, requests, want) if dtype == "float32"
           else _bfloat16_bound(tmp_path, cfg, weights, requests, want))
    mixed, peak = H.trace_mixed(requests, seed=5, tail=7, max_portion=15)
    whole_room = sum(H.round64(len(t)) for t in requests.values())
    results = {}
    for mode, (trace, room) in {"whole": (H.trace_whole(requests), whole_room),
                                "tail": (H.trace_decode_tail(requests, 14), whole_room),
                                "portions": (H.trace_portions(requests, (5, 2, 13, 3, 2, 8)), whole_room),
                                "mixed": (mixed, peak)}.items():
        session = _session(tmp_path, cfg, weights, dtype, device, ops, room, page_size)
        got = H.collect(session, trace)
        for rid in requests:
            H.assert_close(got[rid], want[rid], LABEL[dtype], f"ravapel {name} {mode} {rid}", tol)
        # everything went back to the pools
        assert session.cache.num_free_pages == [p.num_pages for p in session.cache.pools]
        assert session.cache.slots.num_free == session.cache.slots.num_slots
        results[mode] = got
    return results


@pytest.mark.parametrize("name", list(R.CONFIGS))
def test_every_way_of_cutting_on_the_plain_kernels(tmp_path, name):
    from tests.ref_ops import RefOps

    _run_all_modes(tmp_path, name, "float32", "cpu", RefOps(), lengths=[30, 13, 21, 9, 1])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(R.CONFIGS))
def test_every_way_of_cutting_on_the_gpu(tmp_path, name, dtype):
    from inference_engine_b200.kernels import get_ops

    results = _run_all_modes(tmp_path, name, dtype, "cuda", get_ops("cuda"), lengths=[150, 21, 67, 64, 9, 1, 33])
    if dtype == "float32":  # a row's arithmetic does not depend on the cutting or the batch at all
        for mode in ("tail", "portions", "mixed"):
            for rid, rows in results["whole"].items():
                assert torch.equal(rows, results[mode][rid]), f"{name} {mode} {rid}: 32-bit logits differ by cutting"
    get_ops("cuda").check_errors()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_wider_model_with_long_prompts(tmp_path, dtype):
    """Prompts of hundreds of tokens over several chunks and many pages of 16, sizes that reach the
    tensor-core attention in bfloat16 and the wider instances of the recurrence."""
    from inference_engine_b200.kernels import get_ops

    cfg = R.WIDE
    weights = R.make_weights(cfg, seed=21)
    requests = _requests(cfg, [420, 130, 257, 64], seed=900)
    want = _want(cfg, weights, requests)
    tol = (_float32_bound(cfg, weights, requests, want) if dtype == "float32"
           else _bfloat16_bound(tmp_path, cfg, weights, requests, want))
    mixed, peak = H.trace_mixed(requests, seed=8, tail=20, max_portion=90)
    room = sum(H.round64(len(t)) for t in requests.values())
    before = dict(get_ops("cuda").launch_counts)
    results = {}
    for mode, (trace, space) in {"whole": (H.trace_whole(requests), room),
                                 "tail": (H.trace_decode_tail(requests, 40), room),
                                 "portions": (H.trace_portions(requests, (70, 2, 129, 3, 64, 33)), room),
                                 "mixed": (mixed, peak)}.items():
        session = _session(tmp_path / mode, cfg, weights, dtype, "cuda", get_ops("cuda"), space, 16)
        results[mode] = H.collect(session, trace)
        for rid in requests:
            H.assert_close(results[mode][rid], want[rid], LABEL[dtype], f"wide {mode} {rid}", tol)
        assert session.cache.num_free_pages == [p.num_pages for p in session.cache.pools]
    ran = get_ops("cuda").launch_counts.get("sigmoid_attention_mma", 0) - before.get("sigmoid_attention_mma", 0)
    if dtype == "float32":
        assert ran == 0
        for mode in ("tail", "portions", "mixed"):
            for rid in requests:
                assert torch.equal(results["whole"][rid], results[mode][rid]), (mode, rid)
    else:
        assert ran > 0  # (the tensor-core kernel did serve these sizes)
    get_ops("cuda").check_errors()


def test_layout_of_the_model_and_its_caches():
    from inference_engine_b200.config import build_model_spec, config_from_dict
    from inference_engine_b200.engine.model import Model

    model = Model(build_model_spec(config_from_dict(R.MIXED)), "float32", 64)
    assert [e.layer for e in model.spec.schedule] == [0, 1, 2, 1, 2, 1, 2, 3, 4]
    assert [e.before for e in model.spec.schedule] == [None, "loop_in", None, "loop_in", None, "loop_in", None,
                                                      None, None]
    kinds = [type(b.mixer.inner).__name__ for b in model.blocks]
    assert kinds == ["HGRN2", "ParallelSum", "HGRN2", "ParallelSum", "HGRN2"]
    # every pass of the loop has a cache of its own: layer 1's attention three times in its group
    assert [(g.num_layers, g.num_kv_heads, g.head_dim, g.value_dim, g.chunk) for g in model.paged_groups] == [
        (3, 2, 16, 24, 10), (1, 3, 8, 8, 7)]
    shapes = {g.shape: g.num_layers for g in model.state_groups}
    assert shapes[(2 * 72,)] == 9  # the convolution's last two inputs, for every run of a layer
    assert shapes[(1,)] == 1  # the previous token
    assert shapes[(3 * (12 + 1) * 8 + 3,)] == 3  # matrix memory, normaliser column, maxima; three passes
    assert shapes[(2 * 8 * 20,)] == 3 and shapes[(3 * 20 * 12,)] == 1
    assert model.keeps_embedding and model.captures
    plain = Model(build_model_spec(config_from_dict(R.PLAIN)), "float32", 64)
    assert not plain.keeps_embedding and plain.embedding_binding is None
    assert [(g.chunk, g.value_dim) for g in plain.paged_groups] == [(None, 8)]


@pytest.mark.parametrize("name", list(R.CONFIGS))
def test_footprint_formula_counts_what_the_model_declares(name):
    from inference_engine_b200.architectures.ravapel import ravapel_footprint
    from inference_engine_b200.config import build_model_spec, config_from_dict
    from inference_engine_b200.engine.model import Model

    cfg = config_from_dict(R.CONFIGS[name])
    assert ravapel_footprint(cfg) == Model(build_model_spec(cfg), "float32", 64).footprint()


def test_configuration_errors():
    from inference_engine_b200.config import ConfigError, config_from_dict

    with pytest.raises(ConfigError, match="type"):
        config_from_dict(dict(R.MIXED, layers=[dict(R.MIXED["layers"][0], type="other")]))
    with pytest.raises(ConfigError, match="loop"):
        config_from_dict(dict(R.MIXED, loop={"start": 3, "stop": 2, "times": 1}))
    with pytest.raises(ConfigError, match="kv_heads"):
        bad = R.config(16, 11, [(R.parallel(R.left(3, 2, 4, 4), R.right(1, 4, 4)), None)])
        config_from_dict(bad)


def test_pages_before_the_current_chunk_go_back():
    from inference_engine_b200.cache.manager import CacheManager, PagedGroupSpec

    cache = CacheManager([PagedGroupSpec(1, 1, 8, chunk=10, value_dim=8), PagedGroupSpec(1, 1, 8)], [], 16, 4, 2)
    cache.add_request("a")
    cache.grow("a", 0, 23)
    assert cache.pages_held("a") == [6, 6]
    cache.release_behind_window("a", 23)  # the next query sits in the chunk 20..29: pages before 20 go
    assert cache.table(0, "a")[:5] == [-1] * 5 and cache.table(0, "a")[5] >= 0
    assert cache.pages_held("a") == [1, 6]
    cache.grow("a", 23, 31)  # into the chunk 30..39: page 7 holds 28..31
    cache.release_behind_window("a", 31)
    assert [p >= 0 for p in cache.table(0, "a")] == [False] * 7 + [True]
    cache.check_invariants()
    cache.free("a")
    assert cache.num_free_pages == [16, 16]


# --- every mechanism alone, against its plain function -------------------------------------------


def _ops(device):
    if device == "cpu":
        from tests.ref_ops import RefOps

        return RefOps()
    from inference_engine_b200.kernels import get_ops

    return get_ops("cuda")


def _ctx(lens, starts, device, slots=None):
    """The parts of a step's context the kernels read, for requests with `lens` new tokens that
    start at positions `starts`."""
    b = len(lens)
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    seq = [i for i, n in enumerate(lens) for _ in range(n)]
    pos = [s + t for s, n in zip(starts, lens) for t in range(n)]
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=device)  # noqa: E731
    return SimpleNamespace(num_tokens=cu[-1], num_seqs=b, seq_of_token=i32(seq), positions=i32(pos), cu_q=i32(cu),
                           q_starts=cu[:-1], q_lens=list(lens), start_positions=list(starts), max_q_len=max(lens),
                           ctx_lens=i32([s + n for s, n in zip(starts, lens)]), bounds=None, padded=False,
                           slots=i32(slots if slots is not None else list(range(b))))


DEVICES = ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)]


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("heads,dim,vdim", [(3, 12, 20), (1, 5, 3), (2, 48, 16), (2, 100, 40), (1, 130, 8), (1, 260, 33)])
def test_gated_write_recurrence_in_pieces(device, heads, dim, vdim):
    """HGRN2's recurrence over 61 tokens cut into pieces of 1 to 17 tokens, from and to a state slot,
    against the whole-sequence function; a second request beside it must not disturb it."""
    ops, g = _ops(device), torch.Generator().manual_seed(dim)
    T = 61
    q = torch.randn(T, heads, dim, generator=g)
    f = torch.sigmoid(torch.randn(T, heads, dim, generator=g) * 2 + 3)  # slow forgetting: early tokens matter
    v = torch.randn(T, heads, vdim, generator=g)
    want = P.hgrn2_recurrence(q.double(), f.double(), v.double()).float()
    state = torch.zeros(3, heads * vdim * dim, device=device)
    state[1] = 7.0  # another request's slot: left alone
    got, at = [], 0
    for n in [1, 17, 2, 8, 1, 1, 16, 9, 6]:
        # the request (slot 2) beside a stranger (slot 0) that brings 3 tokens of noise
        ctx = _ctx([3, n], [0, at], device, slots=[0, 2])
        rows = lambda x, w: torch.cat([torch.randn(3, heads * w, generator=g), x[at: at + n].reshape(n, -1)]).to(device)  # noqa: E731
        qq, ff, vv = rows(q, dim), rows(f, dim).abs().clamp(max=1.0), rows(v, vdim)
        out = torch.zeros(3 + n, heads * vdim, device=device)
        ops.gated_recurrence(qq, ff, (1 - ff).contiguous(), None, vv, state, ctx.slots, ctx, out, heads, dim, vdim,
                             vdim, 1.0)
        got.append(out[3:].cpu().view(n, heads, vdim))
        at += n
    torch.testing.assert_close(torch.cat(got), want, atol=2e-4, rtol=2e-4)
    assert torch.all(state[1] == 7.0)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("heads,dim,vdim", [(3, 8, 12), (1, 6, 10), (2, 32, 48), (1, 72, 5)])
def test_matrix_memory_in_pieces(device, heads, dim, vdim):
    """mLSTM gates (running maximum from 0), recurrence with the normaliser's column, and read-out
    over 53 tokens cut into pieces, against the whole-sequence function.  Input gates far above and
    far below the forget gates: the maximum moves, and exp(-m) decides the denominator at times."""
    ops, g = _ops(device), torch.Generator().manual_seed(dim + 1)
    T, cap, eps = 53, 7.0, 1e-5
    q = torch.randn(T, heads, dim, generator=g)
    k = torch.randn(T, heads, dim, generator=g)
    v = torch.randn(T, heads, vdim, generator=g)
    pre_i = torch.randn(T, heads, generator=g) * 6
    pre_f = torch.randn(T, heads, generator=g) * 4 + 2
    bi, bf = torch.randn(heads, generator=g), torch.randn(heads, generator=g)
    weight = torch.randn(heads * vdim, generator=g) + 1
    gate = torch.randn(T, heads * vdim, generator=g)
    D = torch.float64
    logi = cap * torch.tanh((pre_i.to(D) + bi.to(D)) / cap)
    logf = torch.nn.functional.logsigmoid(cap * torch.tanh((pre_f.to(D) + bf.to(D)) / cap))
    o = P.mlstm_recurrence(q.to(D) * dim ** -0.5, k.to(D), v.to(D), logi, logf)
    want = (P.rms(o, eps).reshape(T, -1) * weight.to(D) * torch.sigmoid(gate.to(D))).float()
    cols, matrix = vdim + 1, heads * (vdim + 1) * dim
    state = torch.zeros(2, matrix + heads, device=device)
    got, at = [], 0
    for n in [2, 1, 19, 1, 3, 27]:
        ctx = _ctx([n], [at], device, slots=[1])
        sl = slice(at, at + n)
        proj = torch.cat([q[sl].reshape(n, -1), k[sl].reshape(n, -1), v[sl].reshape(n, -1), gate[sl],
                          pre_i[sl], pre_f[sl]], dim=1).to(device)
        qk, vs = heads * dim, heads * vdim
        gates = torch.zeros(n, heads * 3, device=device)
        ops.mlstm_gates(proj[:, 2 * qk + 2 * vs: 2 * qk + 2 * vs + heads], proj[:, 2 * qk + 2 * vs + heads:],
                        bi.to(device), bf.to(device), cap, state, matrix, ctx.slots, ctx, gates, heads)
        out = torch.zeros(n, heads * cols, device=device)
        ops.gated_recurrence(proj[:, :qk], None, proj[:, qk: 2 * qk], gates, proj[:, 2 * qk: 2 * qk + vs], state,
                             ctx.slots, ctx, out, heads, dim, vdim, cols, dim ** -0.5)
        y = torch.zeros(n, vs, device=device)
        ops.recurrence_readout(out, gates, weight.to(device), eps, proj[:, 2 * qk + vs: 2 * qk + 2 * vs], y, heads,
                               vdim, cols)
        got.append(y.cpu())
        at += n
    torch.testing.assert_close(torch.cat(got), want, atol=3e-4, rtol=3e-4)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("taps,channels", [(4, 20), (1, 7), (2, 33), (6, 8)])
def test_input_convolution_in_pieces(device, taps, channels):
    ops, g = _ops(device), torch.Generator().manual_seed(taps)
    T = 40
    x = torch.randn(T, channels, generator=g)
    w = torch.randn(channels, taps, generator=g)
    want = (x.double() + P.causal_conv(x.double(), w.double())).float()
    state = torch.zeros(2, max((taps - 1) * channels, 1), device=device)
    got, at = [], 0
    for n in [1, 1, 2, 9, 1, 3, 23]:  # pieces shorter than the taps too
        ctx = _ctx([n], [at], device, slots=[1])
        out = torch.zeros(n, channels, device=device)
        ops.short_conv_residual(x[at: at + n].to(device).contiguous(), w.to(device), state, ctx.slots, ctx, out)
        got.append(out.cpu())
        at += n
    torch.testing.assert_close(torch.cat(got), want, atol=1e-5, rtol=1e-5)


def _paged(x, page_size, pages_total, order, device):
    """Rows [T, G, d] into a cache [pages, G, page_size, d] at the pages `order` names."""
    T, G, d = x.shape
    cache = torch.full((pages_total + 1, G, page_size, d), 9.0, device=device)  # (unused rows hold nonsense)
    for t in range(T):
        cache[order[t // page_size], :, t % page_size] = x[t].to(device)
    return cache


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("chunk", [None, 1, 5, 12, 150])
def test_sigmoid_attention_sees_exactly_its_chunk(device, chunk):
    """One key per query stands out (score +30 against a bias of -15, every other score near -15,
    so weights of 1 and of 1e-7): the key just inside the query's chunk, or the one just before the
    chunk's first position, which must not be seen.  Prompt portions and single tokens, scattered
    pages, grouped heads, value rows of another size than key rows."""
    ops = _ops(device)
    g = torch.Generator().manual_seed(3)
    T, H, G, d, dv, ps = 45, 4, 2, 48, 6, 4  # (a dimension of its own for every query)
    k = torch.randn(T, G, d, generator=g) * 0.01
    v = torch.randn(T, G, dv, generator=g)
    q = torch.randn(T, H, d, generator=g) * 0.01
    for t in range(T):  # the query of position t looks for the key at the position named below
        first = (t // chunk) * chunk if chunk else 0
        target = first if t % 2 == 0 else first - 1  # just inside / just outside (or before the start)
        if 0 <= target < T:
            k[target, :, t] += 1.0
            q[t, :, t] += 30.0
    bias = torch.full((H,), -15.0)
    want = P.sigmoid_chunk_attention(q.double(), k.double(), v.double(), 1.0, bias.double(), chunk).float()
    order = [7, 2, 11, 0, 5, 9, 3, 10, 1, 8, 6, 4]
    kc, vc = _paged(k, ps, 12, order, device), _paged(v, ps, 12, order, device)
    tables = torch.tensor([order], dtype=torch.int32, device=device)
    got, at = [], 0
    for n in [13, 1, 1, 2, 20, 1, 7]:
        ctx = _ctx([n], [at], device)
        out = torch.zeros(n, H * dv, device=device)
        ops.sigmoid_attention(q[at: at + n].reshape(n, -1).to(device).contiguous(), kc, vc, tables, ctx, H, G, d, dv,
                              ps, 1.0, chunk, bias.to(device), out)
        got.append(out.cpu().view(n, H, dv))
        at += n
    torch.testing.assert_close(torch.cat(got), want, atol=1e-4, rtol=1e-4)
    if chunk and chunk > 1 and 2 * chunk + 1 < T:  # the made-up inputs do tell inside from outside
        seen = want.abs().amax((1, 2))
        inside, outside = 2 * chunk, 2 * chunk + 1  # an even position (looks just inside) and an odd one
        assert seen[inside] > 0.1 and seen[outside] < 1e-3


@pytest.mark.gpu
@pytest.mark.parametrize("d,dv,chunk", [(16, 32, 50), (64, 64, None), (128, 128, 160), (48, 16, 64), (128, 64, 1)])
def test_sigmoid_attention_on_the_tensor_cores(d, dv, chunk):
    """The bfloat16 kernel for prompt portions against the plain function: portions that start and end
    inside chunks and tiles, two requests of unequal length in one step (one of them a single token),
    scattered pages, a key per query that stands out just inside or just outside the chunk."""
    from inference_engine_b200.kernels import get_ops

    ops, g = get_ops("cuda"), torch.Generator().manual_seed(d + dv)
    T, H, G, ps = 333, 6, 2, 16
    bf = lambda x: x.to(torch.bfloat16).float()  # noqa: E731
    k = bf(torch.randn(T, G, d, generator=g) * 0.3)
    v = bf(torch.randn(T, G, dv, generator=g))
    q = bf(torch.randn(T, H, d, generator=g) * 0.3)
    for t in range(0, T, 3):
        first = (t // chunk) * chunk if chunk else 0
        target = first if t % 2 == 0 else first - 1
        if 0 <= target < T:
            k[target, :, t % d] += 2.0
            q[t, :, t % d] += 8.0
    q, k = bf(q), bf(k)
    bias = torch.linspace(-6.0, -2.0, H)
    scale = 0.7
    want = P.sigmoid_chunk_attention(q.double(), k.double(), v.double(), scale, bias.double(), chunk).float()
    pages = -(-T // ps)
    order = torch.randperm(pages + 3, generator=g).tolist()[:pages]
    kc = _paged(k, ps, pages + 3, order, "cuda").to(torch.bfloat16)
    vc = _paged(v, ps, pages + 3, order, "cuda").to(torch.bfloat16)
    other = [pages + 3] * pages  # the second request: one token on the scratch page
    tables = torch.tensor([order, other], dtype=torch.int32, device="cuda")
    kc[pages + 3], vc[pages + 3] = 0.5, 0.25
    before = ops.launch_counts.get("sigmoid_attention_mma", 0)
    got, at = [], 0
    for n in [70, 33, 130, 100]:
        ctx = _ctx([n, 1], [at, 0], "cuda")
        qq = torch.cat([q[at: at + n].reshape(n, -1), torch.ones(1, H * d)]).to("cuda", torch.bfloat16)
        out = torch.zeros(n + 1, H * dv, device="cuda", dtype=torch.bfloat16)
        ops.sigmoid_attention(qq, kc, vc, tables, ctx, H, G, d, dv, ps, scale, chunk, bias.cuda(), out)
        got.append(out[:n].float().cpu().view(n, H, dv))
        lone = torch.sigmoid(torch.tensor(d * 0.5 * scale) + bias)[:, None] * 0.25  # its one key and value
        torch.testing.assert_close(out[n].float().cpu().view(H, dv), lone.expand(H, dv), atol=2e-2, rtol=2e-2)
        at += n
    ops.check_errors()
    assert ops.launch_counts.get("sigmoid_attention_mma", 0) == before + 4  # (the kernel under test did run)
    # (weights keep 16 bits of mantissa in the second product; outputs are rounded to bfloat16)
    torch.testing.assert_close(torch.cat(got), want, atol=0.015, rtol=0.01)


@pytest.mark.parametrize("device", DEVICES)
def test_query_key_norm_rotation_and_cache_rows(device):
    ops, g = _ops(device), torch.Generator().manual_seed(8)
    n, H, G, d, dv, ps, rot, base, eps = 9, 3, 1, 10, 14, 4, 6, 50.0, 1e-5
    proj = torch.randn(n, (H + G) * d + G * dv, generator=g)
    wq, wk = torch.randn(d, generator=g) + 1, torch.randn(d, generator=g) + 1
    pos = torch.tensor([0, 1, 2, 3, 17, 18, 19, 5, 6])
    D = torch.float64
    q = P.rotate_halves(P.rms(proj[:, : H * d].view(n, H, d).to(D), eps) * wq.to(D), pos, rot, base)
    k = P.rotate_halves(P.rms(proj[:, H * d: (H + G) * d].view(n, G, d).to(D), eps) * wk.to(D), pos, rot, base)
    half = rot // 2
    freq = torch.tensor([base ** (-2 * i / rot) for i in range(half)], dtype=D)
    angles = torch.arange(32, dtype=D)[:, None] * freq
    table = torch.stack([angles.cos(), angles.sin()], dim=1).float().to(device)
    q_out = torch.zeros(n, H * d, device=device)
    kc, vc = torch.zeros(9, G, ps, d, device=device), torch.zeros(9, G, ps, dv, device=device)
    slots = torch.tensor([p + 8 for p in pos.tolist()], dtype=torch.int32, device=device)  # pages 2..6
    ops.qk_norm_rope_write(proj.to(device), pos.to(torch.int32).to(device), table, rot, wq.to(device), wk.to(device),
                           eps, q_out, kc, vc, slots, H, G, d, dv, ps)
    torch.testing.assert_close(q_out.cpu().view(n, H, d), q.float(), atol=1e-5, rtol=1e-5)
    for i, s in enumerate(slots.tolist()):
        torch.testing.assert_close(kc[s // ps, :, s % ps].cpu(), k[i].float(), atol=1e-5, rtol=1e-5)
        torch.testing.assert_close(vc[s // ps, :, s % ps].cpu(), proj[i, (H + G) * d:].view(G, dv))


@pytest.mark.parametrize("device", DEVICES)
def test_bigram_rows_and_the_previous_token(device):
    """Buckets, multipliers, the first token's own row, and the previous token carried in the slot
    from one step to the next, also for single tokens and beside another request."""
    ops, g = _ops(device), torch.Generator().manual_seed(4)
    vocab, hidden, buckets, mp, mc = 50, 12, 7, 13, 5
    emb, big = torch.randn(vocab, hidden, generator=g), torch.randn(buckets + 1, hidden, generator=g) * 3
    toks = {0: torch.randint(0, vocab, (12,), generator=g).tolist(), 1: torch.randint(0, vocab, (9,), generator=g).tolist()}
    cfg = {"embedding": {"bigram": {"buckets": buckets, "mul_prev": mp, "mul_cur": mc}}}
    W = {"embed": emb.double(), "bigram": big.double(), "pos": torch.zeros(16, hidden, dtype=torch.float64)}
    want = {r: P.embed(t, W, cfg).float() for r, t in toks.items()}
    state = torch.zeros(3, 1, device=device)
    got, at = {0: [], 1: []}, {0: 0, 1: 0}
    for step in [{0: 5, 1: 1}, {1: 1}, {0: 1, 1: 4}, {0: 1}, {1: 3, 0: 5}]:
        reqs = list(step)
        ctx = _ctx([step[r] for r in reqs], [at[r] for r in reqs], device, slots=[2 - r for r in reqs])
        ids = torch.tensor([t for r in reqs for t in toks[r][at[r]: at[r] + step[r]]], dtype=torch.int32, device=device)
        out = torch.zeros(ids.shape[0], hidden, device=device)
        ops.bigram_embedding(emb.to(device), big.to(device), ids, ctx, state, ctx.slots, out, buckets, mp, mc)
        row = 0
        for r in reqs:
            got[r].append(out[row: row + step[r]].cpu())
            row, at[r] = row + step[r], at[r] + step[r]
    for r in toks:
        torch.testing.assert_close(torch.cat(got[r]), want[r], atol=1e-6, rtol=1e-6)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("hidden", [50, 72, 1100])
def test_norm_add_norm_in_one_kernel(device, hidden):
    ops, g = _ops(device), torch.Generator().manual_seed(hidden)
    n, eps = 7, 1e-5
    h, delta = torch.randn(n, hidden, generator=g), torch.randn(2, n, hidden, generator=g) * 3
    bias, wb, w = torch.randn(hidden, generator=g), torch.randn(hidden, generator=g) * 0.1, torch.randn(hidden, generator=g) * 0.1
    D = torch.float64
    h_want = h.to(D) + P.norm_one_plus(delta.to(D).sum(0) + bias.to(D), wb.to(D), eps)
    out_want = P.norm_one_plus(h_want, w.to(D), eps)
    hd, out = h.clone().to(device), torch.zeros(n, hidden, device=device)
    ops.sandwich_norm(hd, delta.to(device), bias.to(device), (1 + wb).to(device), eps, (1 + w).to(device), eps, out)
    torch.testing.assert_close(hd.cpu(), h_want.float(), atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(out.cpu(), out_want.float(), atol=1e-5, rtol=1e-5)
    rows = torch.tensor([5, 0], dtype=torch.int32, device=device)  # selected rows: h stays as it is
    hd2, out2 = h.clone().to(device), torch.zeros(2, hidden, device=device)
    ops.sandwich_norm(hd2, delta.to(device), bias.to(device), (1 + wb).to(device), eps, (1 + w).to(device), eps, out2, rows)
    torch.testing.assert_close(out2.cpu(), out_want.float()[[5, 0]], atol=1e-5, rtol=1e-5)
    assert torch.equal(hd2.cpu(), h)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("inter", [24, 30, 1096])
def test_gated_activation_with_biases(device, inter):
    ops, g = _ops(device), torch.Generator().manual_seed(inter)
    n = 5
    gate_up, bias = torch.randn(n, 2 * inter, generator=g) * 3, torch.randn(2 * inter, generator=g)
    want = torch.nn.functional.silu(gate_up[:, :inter].double() + bias[:inter].double()) * (
        gate_up[:, inter:].double() + bias[inter:].double())
    out = torch.zeros(n, inter, device=device)
    ops.silu_mul_bias(gate_up.to(device), bias.to(device), out)
    torch.testing.assert_close(out.cpu(), want.float(), atol=1e-5, rtol=1e-5)
    # the product rounded to bfloat16 first (what the bfloat16 path hands over), biases added in 32-bit
    rounded = gate_up.to(torch.bfloat16)
    want16 = torch.nn.functional.silu(rounded[:, :inter].double() + bias[:inter].double()) * (
        rounded[:, inter:].double() + bias[inter:].double())
    out16 = torch.zeros(n, inter, device=device, dtype=torch.bfloat16)
    ops.silu_mul_bias(rounded.to(device), bias.to(device), out16)
    torch.testing.assert_close(out16.float().cpu(), want16.float(), atol=1e-2, rtol=1e-2)


# --- long decoding and generation through the engine ------------------------------------------------


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_state_and_pages(tmp_path, dtype):
    """400 tokens decoded one by one after a short prompt, across many chunks: the recurrent states,
    the convolutions' kept inputs, the previous token and the cached rows carry every earlier token."""
    from inference_engine_b200.kernels import get_ops

    cfg = dict(R.MIXED, max_positions=512)
    weights = R.make_weights(cfg, seed=3)
    toks = _requests(cfg, [410], seed=5)["r0"]
    want = P.forward(cfg, weights, toks, torch.float64).float()
    session = _session(tmp_path, cfg, weights, dtype, "cuda", get_ops("cuda"), 448, 16)
    got = H.collect(session, H.trace_decode_tail({"a": toks}, 400))["a"]
    H.assert_close(got, want, LABEL[dtype], "long decoding",
                   _float32_bound(cfg, weights, {"a": toks}, {"a": want}) if dtype == "float32"
                   else _bfloat16_bound(tmp_path, cfg, weights, {"a": toks}, {"a": want}))


def _greedy_plain(cfg, weights, prompt, count):
    ids = list(prompt)
    for _ in range(count):
        ids.append(int(P.forward(cfg, weights, ids, torch.float64)[-1].argmax()))
    return ids[len(prompt):]


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["mixed", "odd"])
def test_greedy_generation_through_the_engine(name):
    """`LLMEngine` with the scheduler cutting prompts into portions and batching requests, decode
    steps captured and launched ahead: the tokens are the plain implementation's greedy choices."""
    from inference_engine_b200 import SamplingParams
    from inference_engine_b200.engine.llm_engine import LLMEngine
    from inference_engine_b200.engine.loading import model_from_tensors

    cfg = R.CONFIGS[name]
    weights = R.make_weights(cfg, seed=4)
    model, _ = model_from_tensors(cfg, weights, "float32", "cuda", cfg["max_positions"])
    engine = LLMEngine(model, None, (), num_blocks=48, block_size=8, max_num_seqs=3,
                       max_num_batched_tokens=16, debug_checks=True)
    assert engine.graphs is not None  # decode steps are captured, with per-request state too
    prompts = {f"p{i}": _requests(cfg, [n], seed=90 + i)["r0"] for i, n in enumerate([5, 40, 23, 1, 31])}
    for rid, prompt in prompts.items():
        engine.add_request(rid, prompt, SamplingParams(max_tokens=10, temperature=0.0))
    got: dict[str, list[int]] = {rid: [] for rid in prompts}
    while engine.has_unfinished():
        for out in engine.step():
            got[out.request_id].append(out.token_id)
    for rid, prompt in prompts.items():
        assert got[rid] == _greedy_plain(cfg, weights, prompt, 10), rid
    engine.cache.check_invariants()
    assert engine.cache.slots.num_free == engine.cache.slots.num_slots


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_captured_short_steps_with_portions(tmp_path, dtype):
    """Portions and mixed batches replayed through captured launch sequences (launched for bounds, padded
    with tokens that belong to no request): key and value sizes the tensor-core attention takes, so in
    bfloat16 that kernel runs sized by the token bound.  Against the plain implementation; in 32-bit
    equal bit for bit to the eagerly launched steps."""
    from inference_engine_b200.engine.graphs import DecodeGraphs, MixedGraphs
    from inference_engine_b200.kernels import get_ops

    cfg = R.config(64, 89, [
        (R.hgrn2(2, 16, 24), R.dense(48)),
        (R.parallel(R.left(4, 2, 16, 32, chunk=24, rot_dims=8), R.right(2, 8, 16)), R.dense(64)),
        (R.parallel(R.left(2, 1, 32, 16, chunk=9), R.right(3, 4, 8)), None),
    ], taps=2, loop=(1, 3, 2))
    weights = R.make_weights(cfg, seed=6)
    requests = _requests(cfg, [70, 45, 33, 90, 20, 60], seed=300)
    want = _want(cfg, weights, requests)
    tol = (_float32_bound(cfg, weights, requests, want) if dtype == "float32"
           else _bfloat16_bound(tmp_path, cfg, weights, requests, want))
    mixed, peak = H.trace_mixed(requests, seed=2, tail=6, max_portion=20)
    results = {}
    for captured in (True, False):
        for mode, (trace, room) in {"portions": (H.trace_portions(requests), 128), "mixed": (mixed, peak)}.items():
            session = _session(tmp_path / f"{mode}{captured}", cfg, weights, dtype, "cuda", get_ops("cuda"), room, 8)
            if captured:
                graphs = MixedGraphs(DecodeGraphs(session.runner, 256, max(64, -(-room // 8))))
                eager = session.runner.step
                session.runner.step = lambda entries, g=graphs, e=eager: g.run(entries) if g.can_run(entries) else e(entries)
            got = H.collect(session, trace)
            for rid in requests:
                H.assert_close(got[rid], want[rid], LABEL[dtype], f"captured={captured} {mode} {rid}", tol)
            if captured:
                assert graphs.replays > len(requests)
            results[(captured, mode)] = got
    if dtype == "float32":
        for mode in ("portions", "mixed"):
            for rid in requests:
                assert torch.equal(results[(True, mode)][rid], results[(False, mode)][rid]), (mode, rid)
    get_ops("cuda").check_errors()
