"""Kavenex on the CPU: the plain model's mechanisms one by one, and the engine
(configuration, loader, run order, cache, step function, scheduler) over the
kernels' plain references against the plain model."""
import json
import os

import numpy as np
import pytest
import torch

from garuda_b200 import Engine, SamplingParams, StepEntry, ConfigError, WeightError
from garuda_b200.config.registry import build_model, read_model_config
from garuda_b200.parts.base import PagedLatent
from tests.helpers import assert_close
from tests.kavenex_cases import CASES, KA, KB, KC, model_dir, plain_logits, random_tokens, weights
from tests.plain import kavenex_plain as kp
from tests.plain.cpu_ops import CpuOps


def engine(name, **kw):
    kw.setdefault("page_size", 8)
    kw.setdefault("kv_tokens", 512)
    kw.setdefault("context", 256)
    return Engine(model_dir(name), dtype="float32", ops=CpuOps(), cuda_graphs=False, **kw)


# ------------------------------------------------------------------ the plain model's mechanisms
def test_rotation_turns_pairs_and_depends_on_distance_only():
    rng = np.random.default_rng(0)
    q, k = rng.standard_normal((1, 12)), rng.standard_normal((1, 12))
    # dims 8 of 12: the last four channels pass unchanged, lengths are kept
    r = kp.rotate_pairs(q, [5], 100.0, 8)
    assert np.allclose(r[0, 8:], q[0, 8:]) and np.isclose(np.linalg.norm(r), np.linalg.norm(q))
    assert np.allclose(kp.rotate_pairs(q, [0], 100.0, 8), q)
    # pair 0 at position 1 turns by one radian: (u, v) -> (u cos 1 - v sin 1, v cos 1 + u sin 1)
    one = kp.rotate_pairs(np.array([[1.0, 0.0] + [0.0] * 10]), [1], 100.0, 8)
    assert np.allclose(one[0, :2], [np.cos(1.0), np.sin(1.0)])
    dots = [float(kp.rotate_pairs(q, [p + 7], 100.0, 8)[0] @ kp.rotate_pairs(k, [p], 100.0, 8)[0]) for p in (0, 3, 40)]
    assert np.allclose(dots, dots[0])


def test_norms_and_activations():
    x = np.array([[1.0, 2.0, 3.0, 6.0]])
    assert np.allclose(kp.layer_norm(x, 1.0, 0.0, 0.0).mean(), 0) and np.allclose(kp.layer_norm(x, 1.0, 0.0, 0.0).var(), 1)
    assert np.allclose(kp.layer_norm(x, 2.0, 0.5, 0.0), 2 * (x - 3.0) / np.sqrt(3.5) + 0.5)
    assert np.allclose(kp.rms(x, 0.0), x / np.sqrt(12.5))
    assert np.isclose(kp.gelu_tanh(np.array(1.0)), 0.8411919906082768)
    w = {"p.gate": np.array([[3.0]]), "p.up": np.array([[-5.0]]), "p.down": np.array([[1.0]])}
    # gate clamped from above only, up from both sides: min(3, 2) * sigmoid(1.702 * 2) * (max(-5, -2) + 1)
    assert np.allclose(kp.expert(np.array([[1.0]]), w, "p.", 2.0), 2.0 / (1 + np.exp(-3.404)) * (-1.0))
    w = {"p.gate": np.array([[-7.0]]), "p.up": np.array([[0.5]]), "p.down": np.array([[1.0]])}
    assert np.allclose(kp.expert(np.array([[1.0]]), w, "p.", 2.0), -7.0 / (1 + np.exp(7 * 1.702)) * 1.5)


def test_router_takes_the_largest_logits_and_weighs_them_alone():
    w = {"p.router": np.eye(4), "p.router.b": np.array([0.0, 0.0, 0.0, 2.5])}
    idx, wt = kp.route(np.array([[1.0, 3.0, 2.0, 0.0]]), w, "p.", 2)
    assert idx.tolist() == [[1, 3]]          # logits 1, 3, 2, 2.5
    assert np.allclose(wt, np.exp([3.0, 2.5]) / np.exp([3.0, 2.5]).sum())


def test_latent_attention_is_causal_and_reads_far_keys():
    cfg, w = KB, weights("KB")
    toks = random_tokens("KB", 60, 3)
    a = kp.forward(cfg, w, toks)
    b = kp.forward(cfg, w, toks[:30] + [(toks[30] + 1) % cfg["vocab"]] + toks[31:])
    assert np.array_equal(a[:30], b[:30]) and np.abs(a[30:] - b[30:]).max() > 1e-3
    c = kp.forward(cfg, w, [(toks[0] + 5) % cfg["vocab"]] + toks[1:])
    assert np.abs(a[-1] - c[-1]).max() > 1e-4 * np.abs(a[-1]).max()      # the first token still matters at the end


def test_run_order_of_the_loop():
    assert kp.run_order(KA) == [(0, 0), (1, None), (0, 1), (1, None), (0, 2), (1, None), (2, None)]
    assert kp.run_order(KB) == [(0, None), (1, None)]
    assert kp.run_order(KC) == [(0, None), (1, 0)]
    _, model = build_model(KA)
    order = model.spec.order
    assert [c.layer for c in order] == [0, 1, 0, 1, 0, 1, 2]
    assert [c.add_embedding for c in order] == [False, False, True, False, True, False, False]
    assert [c.add_row and c.add_row[1] for c in order] == [0, None, 1, None, 2, None, None]
    # every pass has a cache of its own: seven calls, one group of latent rows 40 + 8 wide
    assert len(model.cache_groups) == 1 and model.cache_groups[0].need == PagedLatent(48, None)
    assert model.cache_groups[0].calls == tuple(range(7))
    _, model = build_model(KC)
    assert sorted(g.need.width for g in model.cache_groups) == [20, 64]


# ------------------------------------------------------------------ configuration and weights
def test_configuration_errors_name_the_key():
    for path, text in ((("vocab",), "vocab"), (("norm", "eps"), "norm.eps"), (("layers", 0, "mixer", "kv_rank"), "kv_rank"),
                       (("layers", 0, "mlp", "router"), "router"), (("embedding",), "embedding.scale")):
        cfg = json.loads(json.dumps(KA))
        d = cfg
        for k in path[:-1]:
            d = d[k]
        del d[path[-1]]
        with pytest.raises(ConfigError, match=text):
            read_model_config(cfg)
    bad = json.loads(json.dumps(KA))
    bad["layers"][1]["type"] = "something_else"
    with pytest.raises(ConfigError, match="something_else"):
        read_model_config(bad)
    bad = json.loads(json.dumps(KA))
    bad["loop"]["stop"] = 9
    with pytest.raises(ConfigError, match="loop"):
        read_model_config(bad)
    bad = json.loads(json.dumps(KB))
    bad["layers"][0]["mixer"]["rot"]["dims"] = 14
    with pytest.raises(ConfigError, match="rot.dims"):
        read_model_config(bad)


def test_the_loader_names_what_does_not_fit(tmp_path):
    from garuda_b200.weights import write_random_model
    from garuda_b200.weights.safetensors_io import SafetensorsFolder, write_safetensors
    d = write_random_model(str(tmp_path / "m"), KC, 1)
    f = SafetensorsFolder(d)
    t = {n: f.tensor(n) for n in f.names()}
    del t["l0.mlp.e3.up"]
    t["l1.mix.uk"] = t["l1.mix.uk"][:, :-1].contiguous()
    t["stray"] = torch.zeros(3)
    write_safetensors(os.path.join(d, "model.safetensors"), t)
    with pytest.raises(WeightError) as e:
        Engine(d, dtype="float32", ops=CpuOps(), cuda_graphs=False, context=64)
    assert e.value.missing == ["l0.mlp.e3.up"] and e.value.unexpected == ["stray"]
    assert [w[0] for w in e.value.wrong_shape] == ["l1.mix.uk"]


# ------------------------------------------------------------------ the engine against the plain model
@pytest.mark.parametrize("name", ["KA", "KB", "KC"])
def test_whole_decode_and_portions_agree_with_the_plain_model(name):
    e = engine(name)
    toks = random_tokens(name, 75, 5)
    ref = plain_logits(name, torch.float32, toks)
    whole = e.step([StepEntry(1, toks, range(len(toks)))]).numpy().copy()
    assert_close(whole, ref, "float32", "whole")
    assert_close(whole[:3], ref[:3], "float32", "the first tokens")
    e.runner.end(1)
    outs = [e.step([StepEntry(2, toks[:1], [0])]).numpy().copy()]           # from the very first token on
    for t in toks[1:]:
        outs.append(e.step([StepEntry(2, [t], [0])]).numpy().copy())
    assert_close(np.concatenate(outs), ref, "float32", "token by token")
    e.runner.end(2)
    pos, outs = 0, []
    for c in [7, 2, 9, 3, 2, 8, 2, 17, 1, 15, 2, 7]:       # cuts inside, at and just after page borders (pages of 8)
        outs.append(e.step([StepEntry(3, toks[pos:pos + c], range(c))]).numpy().copy())
        pos += c
    assert pos == 75
    assert_close(np.concatenate(outs), ref, "float32", "portions")
    e.runner.end(3)
    e.cache.manager.check_invariants()
    assert e.cache.manager.pages_reused > 0


def test_mixed_batches_with_few_pages_and_slots_used_again():
    name = "KA"
    e = engine(name, kv_tokens=136, max_concurrent=3)
    lens = [50, 23, 41, 9, 30, 2]
    toks = [random_tokens(name, n, 30 + i) for i, n in enumerate(lens)]
    refs = [plain_logits(name, torch.float32, t) for t in toks]
    fed, got = [0] * len(lens), [[] for _ in lens]
    live, waiting = [], list(range(len(lens)))
    rng = np.random.default_rng(2)
    held = lambda i: (lens[i] + 7) // 8 * 8
    most = 0
    while live or waiting:
        while waiting and len(live) < 3 and sum(held(i) for i in live) + held(waiting[0]) <= 136:
            live.append(waiting.pop(0))
        most = max(most, len(live))
        entries = []
        for i in list(live):
            left = lens[i] - fed[i]
            entries.append((i, 1 if left <= 6 else int(min(left - 6, rng.integers(2, 10)))))
        out = e.step([StepEntry(100 + i, toks[i][fed[i]:fed[i] + n], range(n)) for i, n in entries]).numpy().copy()
        row = 0
        for i, n in entries:
            got[i].append(out[row:row + n])
            row += n
            fed[i] += n
            if fed[i] == lens[i]:
                live.remove(i)
                e.runner.end(100 + i)
    assert most == 3 and e.cache.manager.pages_reused > 0
    for i in range(len(lens)):
        assert_close(np.concatenate(got[i]), refs[i], "float32", f"request {i}")
    e.cache.manager.check_invariants()


def test_greedy_generation_through_the_scheduler():
    for name in ("KA", "KC"):
        e = engine(name, max_concurrent=2, max_batch_tokens=16, prefill_chunk=8)
        cfg, w = CASES[name][0], weights(name)
        prompts = [random_tokens(name, n, 50 + n) for n in (11, 3, 19)]
        res = e.generate(prompts, SamplingParams.greedy(max_tokens=6))
        for p, r in zip(prompts, res):
            seq = list(p)
            for _ in range(6):
                seq.append(int(np.argmax(kp.forward(cfg, w, seq)[-1])))
            assert r.tokens == seq[len(p):] and r.finish_reason == "length"
