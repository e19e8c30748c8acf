"""Murilorn on the CPU: the plain model's mechanisms one by one, and the engine
(configuration, loader, run order, cache and state, step function, scheduler) over the
kernels' plain references against the plain model."""
import json
import os

import numpy as np
import pytest
import torch

from garuda_b200 import Engine, SamplingParams, StepEntry, ConfigError, WeightError
from garuda_b200.config.registry import build_model, read_model_config
from garuda_b200.parts.base import FixedState, PagedKV
from tests import helpers
from tests.murilorn_cases import CASES, MA, MB, MC, ME, model_dir, plain_logits, random_tokens, weights
from tests.plain import murilorn_plain as mp
from tests.plain.cpu_ops import CpuOps


def assert_close(got, want, dtype, what):
    """Against the 64-bit plain model, as a fraction of the largest logit: 32-bit sums in another
    order through up to six layer runs with sharpened weights differ by up to 1.8e-5 (seen), so
    the limit here is three times that."""
    scale = max(float(np.abs(want).max()), 1e-6)
    err = float(np.abs(np.asarray(got) - want).max())
    assert got.shape == want.shape and np.isfinite(got).all(), what
    helpers.OBSERVED[f"murilorn/{dtype}"] = max(helpers.OBSERVED.get(f"murilorn/{dtype}", 0.0), err / scale)
    assert err <= 6e-5 * scale, f"{what}: max difference {err:.3e} (limit {6e-5 * scale:.3e})"


def engine(name, **kw):
    kw.setdefault("page_size", 8)
    kw.setdefault("kv_tokens", 512)
    kw.setdefault("context", 256)
    return Engine(model_dir(name), dtype="float32", ops=CpuOps(), cuda_graphs=False, **kw)


# ------------------------------------------------------------------ the plain model's mechanisms
def test_norm_weight_lies_about_zero():
    x = np.array([[3.0, 4.0]])
    assert np.allclose(mp.rms_norm(x, np.zeros(2), 0.0), x / np.sqrt(12.5))
    assert np.allclose(mp.rms_norm(x, np.array([1.0, -0.5]), 0.0), x / np.sqrt(12.5) * [2.0, 0.5])
    assert np.allclose(mp.rms_plain(x, np.array([1.0, -0.5]), 0.0), x / np.sqrt(12.5) * [1.0, -0.5])
    # eps sits inside the root, beside the mean
    assert np.allclose(mp.rms_norm(np.array([[0.0, 0.0]]), np.zeros(2), 4.0), 0.0)
    assert np.allclose(mp.rms_norm(np.array([[2.0, 2.0]]), np.zeros(2), 5.0), 2.0 / 3.0)


def test_mask_is_a_window_plus_the_first_positions():
    seen = [[j for j in range(12) if mp.visible(i, j, 4, 2)] for i in range(12)]
    assert seen[0] == [0] and seen[3] == [0, 1, 2, 3]
    assert seen[4] == [0, 1, 2, 3, 4]                 # 0 is outside the window of 4 but kept
    assert seen[6] == [0, 1, 3, 4, 5, 6]              # 2 is neither in the window nor kept
    assert seen[11] == [0, 1, 8, 9, 10, 11]
    assert [j for j in range(8) if mp.visible(7, j, 1, 0)] == [7]


def test_sink_adds_one_to_the_denominator():
    s = np.array([[0.0, np.log(3.0)]])
    p = mp.attention_weights(s, np.array([[True, True]]))
    assert np.allclose(p, [[1 / 5, 3 / 5]])           # 1 + 1 + 3 in the denominator
    p = mp.attention_weights(s, np.array([[True, False]]))
    assert np.allclose(p, [[0.5, 0.0]])
    big = mp.attention_weights(np.array([[800.0, 799.0]]), np.array([[True, True]]))
    assert np.isfinite(big).all() and np.isclose(big.sum(), 1.0)
    small = mp.attention_weights(np.array([[-800.0]]), np.array([[True]]))
    assert np.allclose(small, 0.0)                    # everything goes to the sink


def test_short_convolution_is_causal_and_starts_from_zeros():
    x = np.arange(1.0, 6.0)[:, None] * np.array([[1.0, 10.0]])
    taps = np.array([[0.5, 0.0, 2.0], [0.0, 1.0, 0.0]])        # the last column weighs the current token
    y = mp.short_conv(x, taps)
    assert np.allclose(y[:, 0], [2.0, 4.0, 6.5, 9.0, 11.5])     # 2 x_t + 0.5 x_{t-2}
    assert np.allclose(y[:, 1], [0.0, 10.0, 20.0, 30.0, 40.0])  # x_{t-1}


def test_delta_rule_by_hand():
    # one head, dim 2, vdim 1; the projections pick channels of h
    w = {"p.q": np.array([[1.0, 0, 0, 0], [0, 1.0, 0, 0]]), "p.k": np.array([[1.0, 0, 0, 0], [0, 1.0, 0, 0]]),
         "p.v": np.array([[0, 0, 1.0, 0]]), "p.q.conv": np.array([[1.0], [1.0]]), "p.k.conv": np.array([[1.0], [1.0]]),
         "p.v.conv": np.array([[1.0]]), "p.b": np.array([[0, 0, 0, 1.0]]), "p.A_log": np.array([0.0]),
         "p.a1": np.zeros((1, 4)), "p.a2": np.zeros((2, 1)), "p.dt_bias": np.array([0.0, 50.0]),
         "p.g1": np.zeros((1, 4)), "p.g2": np.zeros((1, 1)), "p.norm": np.array([1.0]), "p.o": np.array([[1.0]])}
    m = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 1}
    big = 40.0          # silu(40) = 40, sigmoid(40) = 1
    h = np.array([[big, 0.0, big, big], [0.0, big, big, big]])
    out = mp.channel_delta(h, w, "p.", m, 0.0)
    # both tokens write a unit key; the read-out is normed to +-1 and gated by sigmoid(0) = 1/2
    assert np.allclose(np.abs(out), 0.5)
    # the decay: channel 0 by exp(-softplus(0)) = 1/2, channel 1 by exp(-softplus(50)) = 0
    T = 3
    h = np.array([[big, 0.0, big, big]] * T)
    S, v = 0.0, mp.silu(big)
    for _ in range(T):
        S = 0.5 * S
        S = S + 1.0 * (v - S)              # k = (1, 0), beta = 1: the state's row 0 becomes v
    assert np.isclose(S, v)


def test_router_weighs_by_its_own_sigmoid_and_scales_the_input():
    w = {"p.router": np.eye(3), "p.e0.gate": np.array([[1.0, 0, 0]]), "p.e0.up": np.array([[1.0, 0, 0]]),
         "p.e0.down": np.array([[1.0], [0], [0]])}
    for e in (1, 2):
        for t in ("gate", "up", "down"):
            w[f"p.e{e}.{t}"] = w[f"p.e0.{t}"] * (e + 1)
    h = np.array([[2.0, 0.5, 1.0]])
    idx, score = mp.route(h, w, "p.", 2)
    assert idx.tolist() == [[0, 2]] and np.allclose(score, mp.sigmoid(np.array([2.0, 1.0])))
    out = mp.routed_experts(h, w, "p.", {"router": {"top": 2}})
    s0, s2 = mp.sigmoid(2.0), mp.sigmoid(1.0)
    want = mp.silu(s0 * 2.0) * (s0 * 2.0) + 3 * (mp.silu(3 * s2 * 2.0) * (3 * s2 * 2.0))
    assert np.isclose(out[0, 0], want) and not np.isclose(out[0, 0], s0 * mp.silu(2.0) * 2.0 + s2 * 3 * mp.silu(6.0) * 6.0)


def test_streams_mix_from_the_old_values():
    w = {"c.in": np.array([1.0, 2.0]), "c.out": np.array([10.0, 100.0]), "c.mix": np.array([[1.0, 3.0], [5.0, 7.0]])}
    X = np.stack([np.full((1, 2), 1.0), np.full((1, 2), 2.0)])
    got = mp.sublayer(X, lambda h: np.ones_like(h), np.zeros(2), 0.0, w, "c.")
    # to stream 0: 1 * x0 + 5 * x1 + 10 y; to stream 1: 3 * x0 + 7 * x1 + 100 y (mix is [from, to])
    assert np.allclose(got[0], 1 + 10 + 10) and np.allclose(got[1], 3 + 14 + 100)


def test_run_order_of_the_loop():
    assert mp.run_order(MA) == [0, 1, 2, 1, 2, 3]
    assert mp.run_order(MB) == [0, 1]
    assert mp.run_order(MC) == [0, 1, 0, 1, 0, 1]
    _, model = build_model(MA)
    assert [c.layer for c in model.spec.order] == [0, 1, 2, 1, 2, 3]
    # every pass has a cache or a state of its own
    assert len(model.state_calls) == 3 and sum(len(g.calls) for g in model.cache_groups) == 3


def test_attention_alone_reads_exactly_its_mask():
    cfg, w = ME, weights("ME")
    size, keep = 9, 2
    toks = random_tokens("ME", 40, 1)
    base = mp.forward(cfg, w, toks)
    i = 30

    def changed(j):
        t = list(toks)
        t[j] = (t[j] + 7) % cfg["vocab"]
        return np.abs(mp.forward(cfg, w, t)[i] - base[i]).max()

    assert changed(i - size) == 0.0 and changed(i - size + 1) > 1e-6      # just outside, just inside the window
    assert changed(keep) == 0.0 and changed(keep - 1) > 1e-6              # the first not kept, the last kept
    assert changed(i + 1) == 0.0


# ------------------------------------------------------------------ configuration and loader
def test_configuration_errors_name_the_key():
    for drop, text in (("vocab", "'vocab'"), ("norm", "'norm.eps'"), ("embedding", "'embedding.scale'")):
        bad = {k: v for k, v in MA.items() if k != drop}
        with pytest.raises(ConfigError, match=text):
            read_model_config(bad)
    bad = json.loads(json.dumps(MA))
    del bad["layers"][1]["mixer"]["scale"]
    with pytest.raises(ConfigError, match=r"layers\[1\]\.mixer\.scale"):
        read_model_config(bad)
    bad = json.loads(json.dumps(MA))
    bad["layers"][0]["type"] = "something"
    with pytest.raises(ConfigError, match="not a mixer of this design"):
        read_model_config(bad)
    bad = json.loads(json.dumps(MA))
    bad["layers"][0]["mlp"]["router"]["top"] = 9
    with pytest.raises(ConfigError, match="exceeds"):
        read_model_config(bad)


def test_cache_needs_come_from_the_configuration():
    _, model = build_model(MA)
    needs = {g.need for g in model.cache_groups}
    assert PagedKV(2, 16, 6, value_dim=24, keep_first=3) in needs and PagedKV(1, 8, 21, value_dim=12, keep_first=10) in needs
    states = [model.call_need[i] for i in model.state_calls]
    assert FixedState((4 * 12 * 20 + 2 * (2 * 2 * 12 + 4 * 20),)) in states
    assert FixedState((2 * 20 * 8 + 1 * (2 * 2 * 20 + 2 * 8),)) in states
    _, model = build_model(MB)
    assert [g.need for g in model.cache_groups] == [PagedKV(3, 8, None, value_dim=8, keep_first=0)]


def test_low_rank_sizes_come_from_the_file(tmp_path):
    # the same configuration without the rank hints loads the folder all the same
    cfg = json.loads(json.dumps(MB))
    for layer in cfg["layers"]:
        layer["mixer"].pop("decay_rank", None)
        layer["mixer"].pop("gate_rank", None)
    import shutil
    d = tmp_path / "m"
    shutil.copytree(model_dir("MB"), d)
    (d / "config.json").write_text(json.dumps(cfg))
    e = Engine(str(d), dtype="float32", ops=CpuOps(), cuda_graphs=False, page_size=8, kv_tokens=64, context=64)
    toks = random_tokens("MB", 9, 5)
    assert_close(e.step([StepEntry(1, toks, range(9))]).numpy(), plain_logits("MB", torch.float32, toks), "float32", "ranks from the file")


def test_a_missing_tensor_is_reported(tmp_path):
    from garuda_b200.weights import SafetensorsFolder, write_safetensors
    f = SafetensorsFolder(model_dir("MC"))
    tensors = {n: f.tensor(n) for n in f.names() if n != "l0.hc1.mix"}
    os.makedirs(tmp_path / "m")
    write_safetensors(str(tmp_path / "m" / "model.safetensors"), tensors)
    (tmp_path / "m" / "config.json").write_text(json.dumps(MC))
    with pytest.raises(WeightError, match="l0.hc1.mix"):
        Engine(str(tmp_path / "m"), dtype="float32", ops=CpuOps(), cuda_graphs=False)


# ------------------------------------------------------------------ the engine against the plain model
@pytest.mark.parametrize("name", ["MA", "MB", "MC", "ME"])
def test_whole_prompt(name):
    toks = random_tokens(name, 45, 2)
    e = engine(name)
    got = e.step([StepEntry(1, toks, range(len(toks)))]).numpy()
    assert_close(got, plain_logits(name, torch.float32, toks), "float32", f"{name} whole")


@pytest.mark.parametrize("name", ["MA", "MC"])
def test_token_by_token_from_the_first_token(name):
    toks = random_tokens(name, 40, 3)
    e = engine(name)
    got = np.stack([e.step([StepEntry(1, [t], [0])]).numpy()[0].copy() for t in toks])
    assert_close(got, plain_logits(name, torch.float32, toks), "float32", f"{name} token by token")


@pytest.mark.parametrize("name,cuts", [("MA", [2, 4, 5, 12, 13, 16, 24, 33, 35, 50]), ("MB", [1, 3, 8, 9, 17, 40, 50]),
                                       ("MC", [7, 9, 11, 26, 28, 50])])
def test_portions_cut_anywhere(name, cuts):
    toks = random_tokens(name, 50, 4)
    e = engine(name)
    rows, a = [], 0
    for b in cuts:
        rows.append(e.step([StepEntry(1, toks[a:b], range(b - a))]).numpy().copy())
        a = b
    assert_close(np.concatenate(rows), plain_logits(name, torch.float32, toks), "float32", f"{name} in portions")


def test_unequal_requests_in_one_batch_with_pages_and_slots_used_again():
    name = "MA"
    e = engine(name, kv_tokens=136, max_concurrent=3)          # 17 pages of 8 for requests of up to 60 tokens
    prompts = {i: random_tokens(name, n, 10 + i) for i, n in enumerate([60, 23, 41, 9, 37, 52])}
    at = {i: 0 for i in prompts}
    got = {i: [] for i in prompts}
    live, waiting = [], list(prompts)
    rng = np.random.default_rng(0)
    steps = 0
    while live or waiting:
        while waiting and len(live) < 3:
            live.append(waiting.pop(0))
        entries = []
        for i in live:
            n = int(rng.choice([1, 1, 2, 3, 7, 16]))
            n = min(n, len(prompts[i]) - at[i])
            entries.append(StepEntry(100 + i, prompts[i][at[i]:at[i] + n], range(n)))
        out = e.step(entries).numpy()
        row = 0
        for i, en in zip(list(live), entries):
            n = len(en.tokens)
            got[i].append(out[row:row + n].copy())
            row += n
            at[i] += n
            if at[i] == len(prompts[i]):
                e.runner.end(100 + i)
                live.remove(i)
        e.cache.manager.check_invariants()
        steps += 1
    assert e.cache.manager.pages_reused > 0
    for i, toks in prompts.items():
        assert_close(np.concatenate(got[i]), plain_logits(name, torch.float32, toks), "float32", f"request {i} in a mixed batch")


def test_windowed_pages_go_back_but_the_kept_ones_stay():
    e = engine("ME", kv_tokens=48, context=200)       # 6 pages of 8; the request runs to 150 tokens
    toks = random_tokens("ME", 150, 6)
    rows = [e.step([StepEntry(1, toks[a:a + 5], range(5))]).numpy().copy() for a in range(0, 150, 5)]
    assert_close(np.concatenate(rows), plain_logits("ME", torch.float32, toks), "float32", "a long request in a small pool")
    held = [p for p in range(e.cache.table_width) if _page(e, 1, p) >= 0]
    assert held[0] == 0 and held[1] >= (150 - 9) // 8 and len(held) <= 3      # the kept first page and the window's


def _page(e, request, index):
    return int(e.cache.manager.block_table_row(request, 0)[index])


def test_long_decoding_after_a_prompt():
    name = "MA"
    toks = random_tokens(name, 120, 7)
    e = engine(name)
    rows = [e.step([StepEntry(1, toks[:20], range(20))]).numpy().copy()]
    rows += [e.step([StepEntry(1, [t], [0])]).numpy().copy() for t in toks[20:]]
    assert_close(np.concatenate(rows), plain_logits(name, torch.float32, toks), "float32", "100 decoded tokens")


def test_greedy_generation_through_the_scheduler():
    name = "MA"
    e = engine(name, max_batch_tokens=16, prefill_chunk=8)
    prompts = [random_tokens(name, n, 20 + n) for n in (19, 5, 30)]
    results = e.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12))
    for p, r in zip(prompts, results):
        seq = list(p)
        for _ in range(12):
            seq.append(int(np.argmax(mp.forward(MA, weights(name), seq)[-1])))
        assert r.tokens == seq[len(p):]
