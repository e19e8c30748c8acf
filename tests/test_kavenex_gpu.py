"""Kavenex on the GPU: every new kernel against its plain reference, then
bin/trace_run replaying requests whole, decoded token by token, in portions and
mixed with page reuse, in 32-bit and bfloat16, against the plain model; greedy
generation through ``Engine.generate`` (graphs, steps launched ahead)."""
import numpy as np
import pytest
import torch

from tests.helpers import TraceRunner, assert_close
from tests.kavenex_cases import CASES, model_dir, plain_logits, random_tokens, weights

pytestmark = pytest.mark.gpu

STORE = {"float32": torch.float32, "bfloat16": torch.bfloat16}
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def up64(n):
    return (n + 63) // 64 * 64


# ---------------------------------------------------------------------------- kernels
class _Ctx:
    def __init__(self):
        from garuda_b200.engine.batch import Workspace
        self.ws = Workspace(torch.device("cuda:0"))


@pytest.fixture(scope="module", params=["float32", "bfloat16"])
def both(request):
    from garuda_b200.kernels.ops import CudaOps
    from tests.plain.cpu_ops import CpuOps
    dt = DTYPES[request.param]
    return CudaOps("cuda:0", tensor_cores=dt == torch.bfloat16), CpuOps(), dt


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator().manual_seed(hash((shape, seed)) % (1 << 31))
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def close(got, want, dt, what):
    got, want = got.float().cpu(), want.float()
    tol = 2e-2 if dt == torch.bfloat16 else 2e-5
    err = (got - want).abs().max().item() / max(want.abs().max().item(), 1e-6)
    assert torch.isfinite(got).all() and err <= tol, f"{what}: {err:.2e}"


@pytest.mark.parametrize("T,d", [(1, 40), (37, 200), (5, 1030), (3, 4096), (2, 6000), (4, 2052)])
def test_layer_norm_rms_add_and_residual_forms(both, T, d):
    ops, cpu, dt = both
    x, y, w, b = rnd(T, d), rnd(T, d, seed=1), rnd(d, dtype=dt, seed=2), rnd(d, dtype=dt, seed=3)
    out, ref = torch.empty(T, d, dtype=dt, device="cuda"), torch.empty(T, d, dtype=dt)
    ops.layernorm(x.cuda() + 3.0, w.cuda(), b.cuda(), 1e-5, out)
    cpu.layernorm(x + 3.0, w, b, 1e-5, ref)
    close(out, ref, dt, "layernorm")
    rows = torch.tensor([T - 1, 0], dtype=torch.int32)
    out, ref = torch.empty(2, d, dtype=dt, device="cuda"), torch.empty(2, d, dtype=dt)
    ops.layernorm(x.cuda(), w.cuda(), None, 1e-5, out, rows.cuda())
    cpu.layernorm(x, w, None, 1e-5, ref, rows)
    close(out, ref, dt, "layernorm of some rows, no bias")
    for alpha, yy, row in ((0.3, y, w), (1.0, None, w), (0.7, y, None)):
        a, c = x.clone().cuda(), x.clone()
        ops.residual_axpy(a, None if yy is None else yy.cuda(), alpha, None if row is None else row.cuda())
        cpu.residual_axpy(c, yy, alpha, row)
        close(a, c, torch.float32, "residual_axpy")
    a, c = x.clone().cuda(), x.clone()
    ops.rms_add(a, y.cuda(), w.cuda(), 1e-5, 0.3)
    cpu.rms_add(c, y, w, 1e-5, 0.3)
    close(a, c, torch.float32, "rms_add")
    table, ids = rnd(50, d, dtype=dt, seed=4), torch.randint(0, 50, (T,), dtype=torch.int32)
    a, c = torch.empty(T, d, device="cuda"), torch.empty(T, d)
    ops.embedding(table.cuda(), ids.cuda(), a, 3.0)
    cpu.embedding(table, ids, c, 3.0)
    close(a, c, torch.float32, "scaled embedding")


@pytest.mark.parametrize("kind,limit", [("silu", 0.0), ("gelu_tanh", 0.0), ("clamped_swish", 1.0), ("clamped_swish", 2.5)])
def test_gated_activations_and_the_token_gate(both, kind, limit):
    ops, cpu, dt = both
    T, F = 29, 83
    gu = rnd(T, 2 * F, scale=2.5)
    out, ref = torch.empty(T, F, dtype=dt, device="cuda"), torch.empty(T, F, dtype=dt)
    ops.gated_act(gu.cuda(), out, kind, limit)
    cpu.gated_act(gu, ref, kind, limit)
    close(out, ref, dt, kind)
    z, table, ids = rnd(T, 12), rnd(40, 36, dtype=dt, seed=1), torch.randint(0, 40, (T,), dtype=torch.int32)
    out, ref = torch.empty(T, 12, dtype=dt, device="cuda"), torch.empty(T, 12, dtype=dt)
    ops.gelu_gather_mul(z.cuda(), table.cuda(), ids.cuda(), 24, out)
    cpu.gelu_gather_mul(z, table, ids, 24, ref)
    close(out, ref, dt, "gelu_gather_mul")


@pytest.mark.parametrize("M,N,K", [(3, 48, 40), (70, 160, 128), (300, 72, 200)])
def test_product_into_the_residual_with_a_multiplier(both, M, N, K):
    ops, cpu, dt = both
    a, w, x = rnd(M, K, dtype=dt), rnd(N, K, dtype=dt, scale=0.1, seed=1), rnd(M, N, seed=2)
    g, c = x.clone().cuda(), x.clone()
    ops.linear(a.cuda(), w.cuda(), g, accumulate=True, alpha=0.3)
    cpu.linear(a, w, c, True, 0.3)
    close(g, c, dt, "linear with a multiplier")


@pytest.mark.parametrize("kind,limit", [("gelu_tanh", 0.0), ("clamped_swish", 1.0), ("silu", 0.0)])
@pytest.mark.parametrize("M,F,K", [(1, 64, 128), (9, 328, 184), (64, 96, 64), (200, 200, 128), (700, 512, 256), (33, 50, 44)])
def test_gate_up_product_with_the_activation_in_its_epilogue(both, kind, limit, M, F, K):
    ops, cpu, dt = both
    h, g, u = rnd(M, K, dtype=dt), rnd(F, K, dtype=dt, scale=0.25, seed=1), rnd(F, K, dtype=dt, scale=0.25, seed=2)
    act, ref = torch.empty(M, F, dtype=dt, device="cuda"), torch.empty(M, F, dtype=dt)
    ops.linear_gated(_Ctx(), h.cuda(), ops.pack_gate_up(g.cuda(), u.cuda()), act, kind, limit)
    cpu.linear_gated(None, h, cpu.pack_gate_up(g, u), ref, kind, limit)
    close(act, ref, dt, f"gate/up with {kind}")


@pytest.mark.parametrize("T,E,top,K,F", [(1, 4, 4, 40, 16), (37, 12, 3, 176, 24), (130, 33, 1, 72, 50), (9, 64, 8, 256, 64),
                                         (300, 5, 2, 136, 72), (700, 12, 4, 160, 72), (8, 32, 4, 512, 200), (1100, 7, 3, 256, 136),
                                         (2048, 16, 4, 512, 320)])
def test_router_and_routed_experts(both, T, E, top, K, F):
    ops, cpu, dt = both
    h, wr, br = rnd(T, K, dtype=dt), rnd(E, K, dtype=dt, scale=0.5, seed=1), rnd(E, seed=2)
    ids, wt = torch.empty(T, top, dtype=torch.int32, device="cuda"), torch.empty(T, top, device="cuda")
    ids_c, wt_c = torch.empty(T, top, dtype=torch.int32), torch.empty(T, top)
    ops.route_topk(h.cuda(), wr.cuda(), br.cuda(), top, ids, wt)
    cpu.route_topk(h, wr, br, top, ids_c, wt_c)
    assert torch.equal(ids.cpu(), ids_c)
    close(wt, wt_c, torch.float32, "router weights")
    assert torch.allclose(wt.sum(-1).cpu(), torch.ones(T), atol=1e-5)
    gates = [rnd(F, K, dtype=dt, scale=0.3, seed=30 + e) for e in range(E)]
    ups = [rnd(F, K, dtype=dt, scale=0.3, seed=300 + e) for e in range(E)]
    wd, x = rnd(E, K, F, dtype=dt, scale=0.3, seed=4), rnd(T, K, seed=5)
    g, c = x.clone().cuda(), x.clone()
    # in the layout the kernels want: packed per expert where the tensor-core products take the sizes
    wgu = ops.pack_expert_gate_up([t.cuda() for t in gates], [t.cuda() for t in ups])
    ops.routed_feed_forward(_Ctx(), h.cuda(), wgu, wd.cuda(), ids, wt, g, "clamped_swish", 1.5, 0.3)
    cpu.routed_feed_forward(None, h, cpu.pack_expert_gate_up(gates, ups), wd, ids_c, wt_c, c, "clamped_swish", 1.5, 0.3)
    close(g, c, dt, "routed experts")


def test_router_ties_go_to_the_lower_index(both):
    ops, cpu, dt = both
    h = torch.ones(2, 8, dtype=dt)
    wr = torch.zeros(6, 8, dtype=dt)
    wr[1], wr[4] = 0.5, 0.5
    ids, wt = torch.empty(2, 3, dtype=torch.int32, device="cuda"), torch.empty(2, 3, device="cuda")
    ops.route_topk(h.cuda(), wr.cuda(), None, 3, ids, wt)
    assert ids.cpu().tolist() == [[1, 4, 0], [1, 4, 0]]


@pytest.mark.parametrize("rank,rot,dims,H,dn,dv", [(24, 8, 6, 3, 10, 12), (80, 16, 16, 4, 24, 40), (200, 40, 40, 2, 24, 56),
                                                   (512, 64, 64, 2, 64, 64)])
def test_latent_cache_rows_head_products_and_attention_over_them(both, rank, rot, dims, H, dn, dv):
    from garuda_b200.parts.rotary import RotaryParams
    ops, cpu, dt = both
    T, ps, start = 45, 16, 19
    src = rnd(T, rank + rot + 5)[:, 5:]                     # a view with a row stride of its own
    nw = rnd(rank, dtype=dt, seed=1)
    rp = RotaryParams(1e4, dims, True, tuple(float(1e4 ** (-2 * i / dims)) for i in range(dims // 2)))
    pos = torch.arange(start, start + T, dtype=torch.int32)
    req = torch.zeros(T, dtype=torch.int32)
    bt = torch.tensor([[4, 2, 7, 1, -1]], dtype=torch.int32)
    pool_c = torch.full((8, 1, ps, rank + rot), float("nan"), dtype=dt)       # an unused cache byte must never matter
    pool_c[4, 0, :] = rnd(ps, rank + rot, dtype=dt, seed=2)
    pool_c[2, 0, :start - ps] = rnd(start - ps, rank + rot, dtype=dt, seed=3)
    pool = pool_c.clone().cuda()
    ops.latent_append(src.cuda(), nw.cuda(), 1e-5, rank, rot, rp, pos.cuda(), req.cuda(), bt.cuda(), pool, ps)
    cpu.latent_append(src, nw, 1e-5, rank, rot, rp, pos, req, bt, pool_c, ps)
    written = ~torch.isnan(pool_c.float())
    assert torch.equal(written, ~torch.isnan(pool.float().cpu()))
    close(torch.nan_to_num(pool), torch.nan_to_num(pool_c), dt, "latent_append")
    qv = rnd(T, H * (dn + rot) + 7, seed=4)[:, :H * (dn + rot)].unflatten(1, (H, dn + rot))
    wuk = rnd(H * dn, rank, dtype=dt, scale=0.3, seed=5)
    q, q_c = torch.zeros(T, H, rank + rot, dtype=dt, device="cuda"), torch.zeros(T, H, rank + rot, dtype=dt)
    ops.head_linear(qv.cuda(), wuk.cuda(), q, rank, dn, True, rot)
    cpu.head_linear(qv, wuk, q_c, rank, dn, True, rot)
    close(q, q_c, dt, "query into the latent's coordinates")
    cu, kvl = torch.tensor([0, T], dtype=torch.int32), torch.tensor([start + T], dtype=torch.int32)
    qs = (q_c.float() * 0.3).to(dt)
    mixed, mixed_c = torch.zeros(T, H * rank, dtype=dt, device="cuda"), torch.zeros(T, H * rank, dtype=dt)
    ops.paged_attention(qs.cuda(), pool, pool, bt.cuda(), cu.cuda(), kvl.cuda(), req.cuda(), mixed, 0.2, 0, ps, 1, T,
                        start + T, value_dim=rank)
    cpu.paged_attention(qs, pool_c, pool_c, bt, cu, kvl, req, mixed_c, 0.2, 0, ps, 1, T, start + T, value_dim=rank)
    close(mixed, mixed_c, dt, "attention over the latent rows")
    wuv = rnd(H * dv, rank, dtype=dt, scale=0.3, seed=6)
    o, o_c = torch.zeros(T, H * dv, dtype=dt, device="cuda"), torch.zeros(T, H * dv, dtype=dt)
    ops.head_linear(mixed_c.cuda().unflatten(1, (H, rank)), wuv.cuda(), o.unflatten(1, (H, dv)), dv, rank, False)
    cpu.head_linear(mixed_c.unflatten(1, (H, rank)), wuv, o_c.unflatten(1, (H, dv)), dv, rank, False)
    close(o, o_c, dt, "values out of the latent")


@pytest.mark.parametrize("T,H,dn,rot,dims,rank", [(5, 3, 10, 8, 6, 24), (300, 4, 24, 16, 16, 80), (70, 16, 64, 64, 64, 512)])
def test_query_rows_prepared_and_mapped_into_the_latent(both, T, H, dn, rot, dims, rank):
    from garuda_b200.parts.rotary import RotaryParams
    ops, cpu, dt = both
    rp = RotaryParams(1e4, dims, True, tuple(float(1e4 ** (-2 * i / dims)) for i in range(dims // 2)))
    src = rnd(T, H * (dn + rot) + 9)[:, :H * (dn + rot)]
    pos = torch.arange(7, 7 + T, dtype=torch.int32)
    qn, ql = torch.zeros(T, H, dn, dtype=dt, device="cuda"), torch.zeros(T, H, rank + rot, dtype=dt, device="cuda")
    qn_c, ql_c = torch.zeros(T, H, dn, dtype=dt), torch.zeros(T, H, rank + rot, dtype=dt)
    ops.latent_query_prepare(src.cuda(), H, dn, rot, rp, pos.cuda(), qn, ql)
    cpu.latent_query_prepare(src, H, dn, rot, rp, pos, qn_c, ql_c)
    close(qn, qn_c, dt, "unrotated query parts")
    close(ql, ql_c, dt, "rotated query parts")
    # the same, with the cache row written by the same kernel
    ps = 16
    full = torch.cat([src, rnd(T, rank + rot, seed=2)], dim=1).contiguous()
    nw = rnd(rank, dtype=dt, seed=3)
    req = torch.zeros(T, dtype=torch.int32)
    pages = (7 + T + ps - 1) // ps
    bt = torch.arange(pages - 1, -1, -1, dtype=torch.int32).view(1, pages)
    pool_c = torch.zeros(pages, 1, ps, rank + rot, dtype=dt)
    pool, qn2, ql2 = pool_c.clone().cuda(), torch.zeros_like(qn), torch.zeros_like(ql)
    qn2_c, ql2_c = torch.zeros_like(qn_c), torch.zeros_like(ql_c)
    ops.latent_rows(full.cuda(), H, dn, rot, rank, rp, pos.cuda(), qn2, ql2, nw.cuda(), 1e-5, req.cuda(), bt.cuda(), pool, ps)
    cpu.latent_rows(full, H, dn, rot, rank, rp, pos, qn2_c, ql2_c, nw, 1e-5, req, bt, pool_c, ps)
    close(qn2, qn2_c, dt, "queries, fused")
    close(ql2, ql2_c, dt, "rotated query parts, fused")
    close(pool, pool_c, dt, "cache rows, fused")
    w = rnd(H * rank, dn, dtype=dt, scale=0.3, seed=1)
    ops.head_linear(qn_c.cuda(), w.cuda(), ql, rank, dn, False)
    cpu.head_linear(qn_c, w, ql_c, rank, dn, False)
    close(ql, ql_c, dt, "query in the latent's coordinates")


@pytest.mark.parametrize("rank,rot,H", [(64, 32, 4), (512, 64, 16), (96, 16, 3), (256, 32, 8)])
@pytest.mark.parametrize("batch", ["mixed", "decode", "one long prompt"])
def test_latent_attention_on_the_tensor_cores(rank, rot, H, batch):
    """Unequal requests in one launch (prompt portions that start inside a page beside single
    tokens with long and with one-token contexts), keys split over CTAs and merged, every unused
    cache byte NaN, pages in a scrambled order."""
    from garuda_b200.kernels.ops import CudaOps
    from tests.plain.cpu_ops import CpuOps
    ops, cpu, dt = CudaOps("cuda:0"), CpuOps(), torch.bfloat16
    ps, row = 16, rank + rot
    reqs = {"mixed": [(1, 700), (130, 130), (37, 300), (1, 1), (64, 95), (2, 33)],
            "decode": [(1, 1500), (1, 17)], "one long prompt": [(400, 1100)]}[batch]
    R, T = len(reqs), sum(q for q, _ in reqs)
    width = max((kv + ps - 1) // ps for _, kv in reqs) + 1
    pages = sum((kv + ps - 1) // ps for _, kv in reqs)
    perm = torch.randperm(pages + 3, generator=torch.Generator().manual_seed(5)).tolist()
    bt = torch.full((R, width), -1, dtype=torch.int32)
    pool_c = torch.full((pages + 3, 1, ps, row), float("nan"), dtype=dt)
    at = 0
    for r, (_, kv) in enumerate(reqs):
        for p in range((kv + ps - 1) // ps):
            bt[r, p] = perm[at]
            n = min(ps, kv - p * ps)
            pool_c[perm[at], 0, :n] = rnd(n, row, dtype=dt, seed=at)
            at += 1
    q = rnd(T, H, row, dtype=dt, scale=0.6)
    cu = torch.tensor([0] + list(np.cumsum([ql for ql, _ in reqs])), dtype=torch.int32)
    kvl = torch.tensor([kv for _, kv in reqs], dtype=torch.int32)
    req = torch.repeat_interleave(torch.arange(R, dtype=torch.int32), torch.tensor([ql for ql, _ in reqs]))
    out, ref = torch.zeros(T, H * rank, dtype=dt, device="cuda"), torch.zeros(T, H * rank, dtype=dt)
    max_q, max_kv = max(ql for ql, _ in reqs), max(kv for _, kv in reqs)
    pool = pool_c.cuda()
    ops.paged_attention(q.cuda(), pool, pool, bt.cuda(), cu.cuda(), kvl.cuda(), req.cuda(), out, 0.11, 0, ps, R,
                        max_q, max_kv, value_dim=rank, min_q_len=min(ql for ql, _ in reqs))
    assert (rank, rot) in ops.tc._latent, "the tensor-core kernel did not take these sizes"
    if batch == "decode":
        assert ops.tc.latent_plan(R, H, max_q, max_kv) > 1
    cpu.paged_attention(q, pool_c, pool_c, bt, cu, kvl, req, ref, 0.11, 0, ps, R, max_q, max_kv, value_dim=rank)
    close(out, ref, dt, f"latent attention, {batch}")


# ---------------------------------------------------------------------------- the engine, replayed
# bfloat16 against the 64-bit plain model, as a fraction of the largest logit: three times what a B200 showed
TOL_BF16 = {"KA": 0.03, "KB": 0.03, "KC": 0.03, "KD": 0.03}


def check(got, ref, dtype, what, name):
    if dtype == "float32":
        return assert_close(got, ref, dtype, what, config=name)
    scale = float(np.abs(ref).max())
    err = float(np.abs(got - ref).max()) / scale
    from tests import helpers
    helpers.OBSERVED[f"{name}/{dtype}"] = max(helpers.OBSERVED.get(f"{name}/{dtype}", 0.0), err)
    assert np.isfinite(got).all() and err <= TOL_BF16[name], f"{what}: {err:.3e} of the largest logit"


@pytest.fixture(scope="module", params=[(n, d) for n in CASES for d in ("float32", "bfloat16")], ids=lambda p: f"{p[0]}-{p[1]}")
def run(request):
    name, dtype = request.param
    tr = TraceRunner(model_dir(name, STORE[dtype]), dtype, max_tokens=4 * up64(130), extra=["--page-size", "16"])
    yield name, dtype, tr
    assert tr.close() == 0


def test_whole(run):
    name, dtype, tr = run
    for n, seed in ((1, 1), (2, 2), (17, 3), (130, 4)):
        toks = random_tokens(name, n, seed)
        out = tr.step([("w", toks, range(n))], end=["w"])
        check(out, plain_logits(name, STORE[dtype], toks), dtype, f"whole, {n} tokens", name)


def test_prompt_then_token_by_token(run):
    name, dtype, tr = run
    toks = random_tokens(name, 120, 7)
    ref = plain_logits(name, STORE[dtype], toks)
    outs = [tr.step([("d", toks[:79], [78])])]
    for i in range(79, 120):
        outs.append(tr.step([("d", [toks[i]], [0])], end=["d"] if i == 119 else []))
    check(np.concatenate(outs), ref[78:], dtype, "decode after a prompt", name)


def test_long_decoding_from_the_first_token(run):
    name, dtype, tr = run
    toks = random_tokens(name, 100, 9)
    ref = plain_logits(name, STORE[dtype], toks)
    outs = [tr.step([("l", [t], [0])], end=["l"] if i == 99 else []) for i, t in enumerate(toks)]
    got = np.concatenate(outs)
    check(got[:4], ref[:4], dtype, "first tokens", name)
    check(got, ref, dtype, "long decoding", name)


def test_portions_down_to_two_tokens(run):
    name, dtype, tr = run
    toks = random_tokens(name, 118, 11)
    ref = plain_logits(name, STORE[dtype], toks)
    cuts = [7, 2, 19, 3, 2, 16, 2, 31, 1, 15, 2, 18]
    pos, outs = 0, []
    for i, c in enumerate(cuts):
        outs.append(tr.step([("p", toks[pos:pos + c], range(c))], end=["p"] if i == len(cuts) - 1 else []))
        pos += c
    assert pos == 118
    check(np.concatenate(outs), ref, dtype, "portions", name)


def test_mixed_requests_reusing_pages_and_slots(run):
    name, dtype, tr = run
    lens = [90, 33, 128, 21, 64, 2, 75]
    toks = [random_tokens(name, n, 20 + i) for i, n in enumerate(lens)]
    refs = [plain_logits(name, STORE[dtype], t) for t in toks]
    pool = 4 * up64(130) - 128
    fed, got = [0] * len(lens), [[] for _ in lens]
    live, waiting = [], list(range(len(lens)))
    rng = np.random.default_rng(1)
    most = 0
    while live or waiting:
        while waiting and len(live) < 4 and sum(up64(lens[i]) for i in live) + up64(lens[waiting[0]]) <= pool:
            live.append(waiting.pop(0))
        most = max(most, len(live))
        entries, ended = [], []
        active = [i for i in live if rng.random() > 0.15] or live[:1]        # now and then a request sits a step out
        for i in active:
            left = lens[i] - fed[i]
            n = 1 if left <= 12 else int(min(left - 12, rng.integers(2, 24)))
            entries.append((f"m{i}", toks[i][fed[i]:fed[i] + n], range(n)))
            if fed[i] + n == lens[i]:
                ended.append(f"m{i}")
        out = tr.step(entries, end=ended)
        row = 0
        for (_, t, _), i in zip(entries, active):
            got[i].append(out[row:row + len(t)])
            row += len(t)
            fed[i] += len(t)
            if fed[i] == lens[i]:
                live.remove(i)
    assert most == 4
    for i in range(len(lens)):
        check(np.concatenate(got[i]), refs[i], dtype, f"mixed, request {i}", name)


def test_every_way_of_cutting_gives_the_same_logits_in_32_bit(run):
    name, dtype, tr = run
    if dtype != "float32":
        pytest.skip("compared against the plain model in bfloat16")
    toks = random_tokens(name, 80, 31)
    whole = tr.step([("x", toks, range(80))], end=["x"])
    parts = [tr.step([("y", toks[:50], range(50))])]
    parts += [tr.step([("y", [t], [0])]) for t in toks[50:79]]
    parts.append(tr.step([("y", [toks[79]], [0])], end=["y"]))
    assert np.abs(np.concatenate(parts) - whole).max() <= 2e-6 * max(1.0, np.abs(whole).max())


def test_a_key_hundreds_of_positions_back(tmp_path):
    """One early key made to stand out: a one-layer model with sharpened query and key weights, a
    token that occurs once, 590 positions back, and a last token chosen (by search in the plain
    model) so that a head puts nearly all its weight on that one key. Run whole, and cut with the end
    decoded: an engine that lost the key would answer from other values altogether."""
    from garuda_b200.weights import write_random_model
    from tests.plain import kavenex_plain as kp
    from tests.helpers import folder_weights
    mixer = {"heads": 2, "dim": 16, "rot_dim": 4, "vdim": 16, "kv_rank": 24, "scale": 1.0, "rot": {"base": 1e6, "dims": 4}}
    cfg = {"architecture": "Kavenex", "vocab": 64, "width": 32, "embedding": {"scale": 4.0}, "norm": {"eps": 1e-5},
           "residual_mult": 1.0, "layers": [{"type": "latent_attention", "mlp": None, "mixer": mixer}]}
    d = write_random_model(str(tmp_path / "far"), cfg, 5, scale={"mix.q": 14.0, "mix.dkv": 30.0, "mix.uk": 12.0,
                                                                  "mix.uv": 10.0, "mix.o": 10.0, "head": 5.0, "embed": 30.0})
    w = {k: np.asarray(v, dtype=np.float64) for k, v in folder_weights(d).items()}
    toks = np.random.default_rng(3).integers(1, 63, 600).tolist()
    toks[9] = 63

    def weight_on_the_far_key(last):
        t = toks[:-1] + [last]
        h = kp.layer_norm(w["embed"][np.asarray(t)] * 4.0, w["l0.norm1"], w["l0.norm1.b"], 1e-5)
        heads = []
        kp.latent_attention(h, w, "l0.mix.", mixer, 1e-5, np.arange(600), heads)
        return max(float(hd[-1, 9]) for hd in heads)

    toks[-1] = max(range(1, 63), key=weight_on_the_far_key)
    assert weight_on_the_far_key(toks[-1]) > 0.9
    ref = kp.forward(cfg, w, toks).astype(np.float32)
    other = kp.forward(cfg, w, toks[:9] + [5] + toks[10:])
    assert np.abs(ref[-1] - other[-1]).max() > 0.1 * np.abs(ref[-1]).max()
    tr = TraceRunner(d, "float32", max_tokens=2 * up64(600), extra=["--page-size", "16"])
    whole = tr.step([("a", toks, range(560, 600))], end=["a"])
    assert_close(whole, ref[560:], "float32", "whole, far keys")
    outs = [tr.step([("b", toks[:300], [])]), tr.step([("b", toks[300:570], range(260, 270))])]
    outs += [tr.step([("b", [t], [0])]) for t in toks[570:]]
    got = np.concatenate([o for o in outs if o is not None])
    assert_close(got, ref[560:], "float32", "cut and decoded, far keys")
    assert tr.close() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(dtype):
    from garuda_b200 import Engine, SamplingParams
    from tests.plain import kavenex_plain as kp
    name = "KD"
    cfg, w = CASES[name][0], weights(name, STORE[dtype])
    e = Engine(model_dir(name, STORE[dtype]), dtype=dtype, context=256, kv_tokens=1024, max_concurrent=4)
    assert e.model.graph_safe
    prompts = [random_tokens(name, n, 70 + n) for n in (5, 40, 1, 23, 64)]
    res = e.generate(prompts, SamplingParams.greedy(max_tokens=12))
    assert e.runner.graphs.replays > 0
    for p, r in zip(prompts, res):
        assert r.finish_reason == "length" and len(r.tokens) == 12
        seq = list(p)
        for tok in r.tokens:
            logits = kp.forward(cfg, w, seq)[-1]
            best = float(logits.max())
            # the engine's token is the plain model's, or in bfloat16 one whose logit is within rounding of it
            slack = (1e-4 if dtype == "float32" else 0.03) * float(np.abs(logits).max())
            assert logits[tok] >= best - slack, f"token {tok} has logit {logits[tok]}, the best is {best}"
            seq.append(tok)


# ---------------------------------------------------------------------------- configurations drawn at random
def _random_config(rng):
    def pick(xs):
        return xs[int(rng.integers(0, len(xs)))]

    def mixer():
        rot_dim = pick([0, 4, 8, 12, 16, 32])
        dims = pick([d for d in (0, 4, 8, 12, 16, 32) if d <= rot_dim])
        return {"heads": pick([1, 2, 3, 5, 8]), "dim": pick([8, 16, 24, 40, 64]), "rot_dim": rot_dim,
                "vdim": pick([8, 16, 24, 48, 64]), "kv_rank": pick([16, 24, 40, 64, 80, 128, 272]), "scale": pick([0.1, 0.2, 0.05]),
                "rot": {"base": pick([100.0, 1e4, 5e5]), "dims": dims}}

    def mlp():
        kind = pick(["dense", "moe", "moe", None])
        if kind is None:
            return None
        if kind == "dense":
            return {"kind": "dense", "ff": pick([24, 64, 100, 136, 328])}
        experts = pick([2, 4, 7, 12, 40])
        return {"kind": "moe", "router": {"experts": experts, "top": pick([t for t in (1, 2, 3, 4, 8) if t <= experts])},
                "expert": {"ff": pick([8, 20, 32, 56, 72]), "limit": pick([1.0, 2.0, 7.0])},
                "shared": pick([None, {"ff": pick([16, 40, 88]), "limit": pick([0.5, 1.0, 3.0])}])}

    n = pick([1, 2, 3, 4])
    shared_mixer = mixer() if pick([True, False]) else None
    cfg = {"architecture": "Kavenex", "vocab": pick([50, 97, 300, 1000]), "width": pick([40, 64, 72, 136, 256]),
           "embedding": {"scale": pick([1.0, 3.0, 0.5])}, "norm": {"eps": pick([1e-5, 1e-6])},
           "residual_mult": pick([1.0, 0.3, 0.7]),
           "layers": [{"type": "latent_attention", "mixer": shared_mixer or mixer(), "mlp": mlp()} for _ in range(n)]}
    if pick([True, False]):
        cfg["token_side"] = {"dim": pick([4, 8, 16, 24])}
    if pick([True, True, False]):
        start = int(rng.integers(0, n))
        cfg["loop"] = {"start": start, "stop": int(rng.integers(start + 1, n + 1)), "times": pick([1, 2, 3])}
    return cfg


@pytest.mark.parametrize("seed", [1, 7, 23])
def test_configurations_drawn_at_random(seed, tmp_path):
    """Sizes nobody chose (no rotated part at all, one head, widths and ranks that no tensor-core kernel
    takes, every expert chosen, loops of one pass): whole, in portions, and decoded two requests side by
    side through graphs; 32-bit against the plain model, bfloat16 finite and near it."""
    from garuda_b200 import Engine, StepEntry
    from garuda_b200.weights import write_random_model
    from tests.helpers import folder_weights
    from tests.kavenex_cases import SHARPEN
    from tests.plain import kavenex_plain as kp
    rng = np.random.default_rng(seed)
    for case in range(4):
        cfg = _random_config(rng)
        toks = rng.integers(0, cfg["vocab"], 120).tolist()
        for dtype in ("float32", "bfloat16"):
            d = write_random_model(str(tmp_path / f"m{case}{dtype}"), cfg, seed + case, norm_init=("normal_about_one", 0.1),
                                   store_dtype=STORE[dtype], scale=SHARPEN)
            ref = kp.forward(cfg, folder_weights(d), toks)
            e = Engine(d, dtype=dtype, context=256, kv_tokens=1024, page_size=16, max_concurrent=4)
            whole = e.step([StepEntry(1, toks, range(120))]).float().cpu().numpy().copy()
            e.runner.end(1)
            outs, pos = [], 0
            for c in [7, 2, 33, 1, 16, 31]:
                outs.append(e.step([StepEntry(2, toks[pos:pos + c], range(c))]).float().cpu().numpy().copy())
                pos += c
            while pos < 120:
                two = e.step([StepEntry(2, [toks[pos]], [0]), StepEntry(3, [toks[pos - 90]], [0])])
                outs.append(two.float().cpu().numpy()[:1].copy())
                pos += 1
            cut = np.concatenate(outs)
            scale = float(np.abs(ref).max())
            for got, what in ((whole, "whole"), (cut, "cut")):
                per_position = np.abs(got - ref).max(-1) / scale
                assert np.isfinite(got).all(), f"{what}, {dtype}: not finite with {cfg}"
                if dtype == "float32":
                    # 32-bit sums against the 64-bit oracle under sharpened weights: up to 4e-5 seen; a wrong
                    # key, page or expert moves the logits by a hundred times that
                    assert per_position.max() <= 1e-4, f"{what}: {per_position.max():.2e} with {cfg}"
                else:
                    # bfloat16 rounding may turn a router's close call (one of two experts, say), which changes
                    # that token and what later tokens read of it: the typical position is what is bounded
                    assert np.median(per_position) <= 0.03, f"{what}: median {np.median(per_position):.2e} with {cfg}"
