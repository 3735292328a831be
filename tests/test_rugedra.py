"""The Rugedra design in the engine against the plain whole-sequence implementation
(`tests/plain_rugedra.py`): whole prompts, token-by-token decoding, portions down to two
tokens, mixed batches with pages and state slots used again, three configurations of odd
sizes; on the CPU through the plain stand-ins of the kernels, on the GPU through the kernels
in both precisions, and greedy generation through the engine's own entry point."""

from __future__ import annotations

import pytest
import torch

from tests import helpers as H
from tests import plain_rugedra as P
from tests import rugedra_configs as R

LENGTHS = [50, 21, 37, 64, 9, 1]


def _requests(cfg, lengths=LENGTHS, seed=700):
    return {f"r{i}": torch.randint(0, cfg["vocab"], (n,), generator=torch.Generator().manual_seed(seed + i)).tolist()
            for i, n in enumerate(lengths)}


def _want(cfg, weights, requests):
    return {rid: P.forward(cfg, weights, toks, torch.float64).float() for rid, toks in requests.items()}


def _session(tmp_path, cfg, weights, dtype, device, ops, max_tokens, page_size):
    from inference_engine_b200.engine.replay import ReplaySession

    folder = H.write_model_dir(tmp_path / f"m{abs(hash(str(cfg))) % 10**8}", cfg, weights)
    return ReplaySession(folder, dtype, max_tokens, device=device, ops=ops, page_size=page_size)


BF16_TOL = dict(atol=0.35, rtol=0.0, pos_rel_rms=0.08, rel_rms=0.04)


def _run_all_modes(tmp_path, name, dtype, device, ops, page_size=4, lengths=LENGTHS):
    cfg = R.CONFIGS[name]
    weights = R.make_weights(cfg, seed=11)
    requests = _requests(cfg, lengths)
    want = _want(cfg, weights, requests)
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
            H.assert_close(got[rid], want[rid], dtype, f"rugedra {name} {mode} {rid}",
                           H.TOL["float32"] if dtype == "float32" else BF16_TOL)
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


def test_layout_of_the_model_and_its_caches():
    from inference_engine_b200.config import build_model_spec, config_from_dict
    from inference_engine_b200.engine.model import Model

    model = Model(build_model_spec(config_from_dict(R.with_ranks(R.MIXED))), "float32", 64)
    kinds = [(type(b.mixer).__name__, type(b.feed_forward).__name__) for b in model.blocks]
    assert kinds == [("ChannelDeltaRule", "RoutedExperts"), ("LatentAttention", "NoneType"),
                     ("LatentAttention", "SquaredReluFF"), ("ChannelDeltaRule", "SquaredReluFF")]
    # a cached row is the latent and the rotated key part; no value rows beside it
    assert [(g.num_layers, g.num_kv_heads, g.head_dim, g.value_dim) for g in model.paged_groups] == [
        (1, 1, 28, 0), (1, 1, 40, 0)]
    # a state slot: the heads' matrices and the last taps - 1 inputs of the convolutions
    assert [g.shape for g in model.state_groups] == [(6 * 12 * 20 + 3 * (2 * 2 * 12 + 6 * 20),),
                                                     (2 * 40 * 8 + 1 * (2 * 2 * 40 + 2 * 8),)]
    assert all(b.residual_mult == 0.8 for b in model.blocks)
    fp = model.footprint()
    assert fp.cache_values_per_token == 28 + 40


def test_ranks_come_from_the_tensor_shapes(tmp_path):
    from inference_engine_b200.config import ConfigError, build_model_spec, config_from_dict, load_config

    weights = R.make_weights(R.DELTA_ONLY, seed=1)
    folder = H.write_model_dir(tmp_path / "d", R.DELTA_ONLY, weights)
    cfg = load_config(folder)
    assert cfg.layers[0].mixer["decay_rank"] == R.RANKS["decay_rank"]
    assert cfg.layers[1].mixer["gate_rank"] == R.RANKS["gate_rank"]
    with pytest.raises(ConfigError, match="decay_rank"):
        build_model_spec(config_from_dict(R.DELTA_ONLY))  # neither tensors nor keys say
    bad = dict(R.MIXED, layers=[dict(R.MIXED["layers"][0], type="other")])
    with pytest.raises(ConfigError, match="type"):
        config_from_dict(bad)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_state_and_pages(tmp_path, dtype):
    """420 tokens decoded one by one after a short prompt: the recurrent state, the convolution's
    kept inputs and the cached rows carry every earlier token."""
    from inference_engine_b200.kernels import get_ops

    cfg = R.MIXED
    weights = R.make_weights(cfg, seed=3)
    cfg = dict(cfg, max_positions=512)
    weights["pos"] = (torch.randn(512, cfg["width"], generator=torch.Generator().manual_seed(9)) * 0.5).bfloat16()
    toks = _requests(cfg, [430], seed=5)["r0"]
    want = P.forward(cfg, weights, toks, torch.float64).float()
    session = _session(tmp_path, cfg, weights, dtype, "cuda", get_ops("cuda"), 448, 16)
    got = H.collect(session, H.trace_decode_tail({"a": toks}, 420))["a"]
    H.assert_close(got, want, dtype, "long decoding", H.TOL["float32"] if dtype == "float32" else BF16_TOL)


def _greedy_plain(cfg, weights, prompt, count):
    ids = list(prompt)
    for _ in range(count):
        ids.append(int(P.forward(cfg, weights, ids, torch.float64)[-1].argmax()))
    return ids[len(prompt):]


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["mixed", "latent_only"])
def test_greedy_generation_through_the_engine(name):
    """`generate` with the scheduler cutting prompts into portions and batching requests: the
    tokens are the plain implementation's greedy choices (32-bit)."""
    from inference_engine_b200 import SamplingParams
    from inference_engine_b200.engine.llm_engine import LLMEngine
    from inference_engine_b200.engine.loading import model_from_tensors

    cfg = R.with_ranks(R.CONFIGS[name])
    weights = R.make_weights(R.CONFIGS[name], seed=4)
    model, _ = model_from_tensors(cfg, weights, "float32", "cuda", cfg["max_positions"])
    engine = LLMEngine(model, None, (), num_blocks=48, block_size=8, max_num_seqs=3,
                       max_num_batched_tokens=16, debug_checks=True)
    assert engine.graphs is not None  # decode steps are captured, with per-request state too
    prompts = {f"p{i}": _requests(R.CONFIGS[name], [n], seed=90 + i)["r0"] for i, n in enumerate([5, 40, 23, 1, 31])}
    for rid, prompt in prompts.items():
        engine.add_request(rid, prompt, SamplingParams(max_tokens=10, temperature=0.0))
    got: dict[str, list[int]] = {rid: [] for rid in prompts}
    while engine.has_unfinished():
        for out in engine.step():
            got[out.request_id].append(out.token_id)
    for rid, prompt in prompts.items():
        assert got[rid] == _greedy_plain(R.CONFIGS[name], weights, prompt, 10), rid
    engine.cache.check_invariants()
    assert engine.cache.slots.num_free == engine.cache.slots.num_slots
