"""Dezelorn on the GPU against the plain implementation (``plain_dezelorn``): every new
kernel alone, then whole models replayed whole, token by token, in portions down to two tokens
and in mixed batches with pages and state slots used again, in float32 and bfloat16, and
greedy generation through the engine."""

import math

import numpy as np
import pytest
import torch

import dezelorn_cases as C
import helpers as H
import plain_dezelorn as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64


def _ctx(entries, groups=1):
    from servelab_b200.engine.batch import StepContext
    return StepContext.pack(entries, groups, DEV)


def _entry(tokens, start, table, slot=0):
    from servelab_b200.engine.batch import BatchEntry
    return BatchEntry(tokens=[0] * tokens, start=start, want=(), block_tables=[table], state_slot=slot)


# ------------------------------------------------------------------ norm
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dim", [48, 77, 1024])
def test_dynamic_tanh_kernel(dtype, dim):
    from servelab_b200.ops import kernels as K
    g = torch.Generator().manual_seed(dim)
    T = 9
    resid = torch.randn(T, dim, generator=g) * 2
    delta = (torch.randn(T, dim, generator=g) * 3).to(dtype)
    post = (torch.tensor([0.7]), torch.randn(dim, generator=g), torch.randn(dim, generator=g))
    pre = (torch.tensor([0.4]), torch.randn(dim, generator=g), torch.randn(dim, generator=g))
    dev = lambda ts: tuple(t.to(DEV) for t in ts)
    want_resid = resid.double() + plain.dynamic_tanh(delta.double(), post[1].double(), post[2].double(), 0.7)
    want_out = plain.dynamic_tanh(want_resid, pre[1].double(), pre[2].double(), 0.4)
    r = resid.to(DEV)
    out = torch.empty(T, dim, dtype=dtype, device=DEV)
    K.dyt_add_norm(r, delta.to(DEV), dev(post), dev(pre), out)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert (r.cpu().double() - want_resid).abs().max() < 1e-5          # the stream stays float32
    assert (out.cpu().double() - want_out).abs().max() < tol
    # rows selected: the stream is left alone, the update still counts for the selected rows
    rows = torch.tensor([7, 2], dtype=torch.int32, device=DEV)
    r2 = resid.to(DEV)
    out2 = torch.empty(2, dim, dtype=dtype, device=DEV)
    K.dyt_add_norm(r2, delta.to(DEV), dev(post), dev(pre), out2, rows)
    assert torch.equal(r2.cpu(), resid) and torch.equal(out2, out[[7, 2]])
    # no pending norm on the update, and an update without a following norm
    r3 = resid.to(DEV)
    K.dyt_add_norm(r3, delta.to(DEV), None, None, None)
    assert (r3.cpu().double() - (resid.double() + delta.double())).abs().max() < 1e-6


@pytest.mark.parametrize("M", [1, 8, 16, 40])
def test_product_with_both_norms_in_its_epilogue(M):
    """The product that closes a branch, the Dynamic Tanh of its result, the add and the Dynamic
    Tanh of the next sublayer's input in one kernel, against the oracle; one row of the stream
    a thousand times larger than the others."""
    from servelab_b200.ops import kernels as K
    g = torch.Generator().manual_seed(M)
    N, Kd = 384, 1024
    x = (torch.randn(M, Kd, generator=g) * 0.5).bfloat16()
    w = (torch.randn(N, Kd, generator=g) * 0.05).bfloat16()
    resid = torch.randn(M, N, generator=g)
    resid[M // 2] *= 1000.0
    post = (torch.tensor([0.8]), torch.randn(N, generator=g), torch.randn(N, generator=g))
    pre = (torch.tensor([0.3]), torch.randn(N, generator=g), torch.randn(N, generator=g))
    prod = x.double() @ w.double().T
    want_resid = resid.double() + plain.dynamic_tanh(prod, post[1].double(), post[2].double(), 0.8)
    want_z = plain.dynamic_tanh(want_resid, pre[1].double(), pre[2].double(), 0.3)
    r = resid.to(DEV)
    z = K.gemm_tc_resid_dyt(x.to(DEV), w.to(DEV), r, tuple(t.to(DEV) for t in post),
                            tuple(t.to(DEV) for t in pre))
    assert K.gemm_tc_status() == 0
    assert ((r.cpu().double() - want_resid).abs() / (1 + want_resid.abs())).max() < 2e-3
    assert (z.cpu().double() - want_z).abs().max() < 3e-2


# ----------------------------------------------------- convolution + cache
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("D", [8, 6])
@pytest.mark.parametrize("taps", [1, 2, 4, 7, 20])
def test_conv_kernel_over_portions_and_single_tokens(dtype, taps, D):
    """Two requests fed in unequal portions (one of them of single tokens from the start, so
    the state is shifted on the spot) give the convolution of their whole sequences; keys land
    in the pages the tables name; the extra columns of the projection are not touched."""
    from servelab_b200.ops import kernels as K
    H_, Hkv, ps, pages = 3, 2, 4, 24           # (head size 6: no 16-byte vectors, the scalar instance)
    qs, kv = H_ * D, Hkv * D
    Cw = qs + kv
    g = torch.Generator().manual_seed(taps)
    lens = {"a": 23, "b": 9}
    extra = 8 if D == 8 else 5                 # (rows stay 16-byte aligned for head size 8)
    proj = {r: torch.randn(n, Cw + extra, generator=g).to(dtype) for r, n in lens.items()}
    w = torch.randn(Cw, taps, generator=g)
    state = torch.zeros(4, max(taps - 1, 1), Cw, device=DEV) if taps > 1 else None
    kc = torch.zeros(pages, Hkv, ps, D, dtype=dtype, device=DEV)
    order = torch.randperm(pages, generator=g).tolist()
    tables = {"a": order[:6], "b": order[6:9]}
    slots = {"a": 2, "b": 0}
    got_q = {r: [] for r in lens}
    done = {r: 0 for r in lens}
    plan = [{"a": 5, "b": 1}, {"a": 1, "b": 1}, {"a": 2, "b": 1}, {"b": 1}, {"a": 1, "b": 1},
            {"a": 9, "b": 1}, {"a": 1, "b": 1}, {"a": 1, "b": 1}, {"a": 1}, {"a": 1, "b": 1}, {"a": 1}]
    coef, every = 0.5, 3
    for step in plan:
        ents, chunks = [], []
        for r, n in step.items():
            ents.append(_entry(n, done[r], tables[r], slots[r]))
            chunks.append(proj[r][done[r]:done[r] + n])
        ctx = _ctx(ents)
        x = torch.cat(chunks).to(DEV)
        q = torch.full((x.shape[0], qs), 7.0, dtype=dtype, device=DEV)
        K.qk_conv_cache(x, w.t().contiguous().to(DEV), state, ctx, ctx.block_tables[0], ps, coef, every, q, kc, Hkv, D)
        assert torch.equal(x.cpu(), torch.cat(chunks))
        off = 0
        for r, n in step.items():
            got_q[r].append(q[off:off + n].cpu())
            off += n
            done[r] += n
    assert done == lens and K.conv_cache_status() == 0
    tol = 1e-5 if dtype == torch.float32 else 5e-3          # (bfloat16: relative, one rounding of the result)
    for r, n in lens.items():
        y = plain.causal_conv(proj[r][:, :Cw].double(), w.double())
        want_q = y[:, :qs] * plain.query_temperature(n, coef, every, F64)[:, None]
        assert ((torch.cat(got_q[r]).double() - want_q).abs() / (1 + want_q.abs())).max() < tol
        for p in range(n):
            page = tables[r][p // ps]
            got_k = kc[page, :, p % ps, :].reshape(-1).cpu().double()
            assert ((got_k - y[p, qs:]).abs() / (1 + y[p, qs:].abs())).max() < tol, (r, p)
        if taps > 1:                                            # the record: the last taps - 1 projected rows
            want = proj[r][max(0, n - (taps - 1)):, :Cw].double()
            assert torch.equal(state[slots[r], taps - 1 - want.shape[0]:].cpu().double(), want)


# ------------------------------------------------------------ attention
def _attention_case(seed, H_, Hkv, D, window, ctxs, qlens, ps, dtype, spike):
    """Requests with ``ctxs`` keys of which the last ``qlens`` are this step's queries.
    ``spike`` ("in" / "out" / None): for every request, the key just inside (or just outside)
    the window of its last query is made to dominate that query's scores in every head."""
    g = torch.Generator().manual_seed(seed)
    S = len(ctxs)
    pages_needed = [-(-c // ps) for c in ctxs]
    num_pages = sum(pages_needed) + 3
    order = torch.randperm(num_pages, generator=g).tolist()
    kc = torch.full((num_pages, Hkv, ps, D), 1e30, dtype=dtype)
    ks, qs_, tables = [], [], []
    for s in range(S):
        k = torch.randn(ctxs[s], Hkv, D, generator=g)
        q = torch.randn(ctxs[s], H_, D, generator=g)
        if spike is not None:
            j = ctxs[s] - 1 - (window - 1 if spike == "in" else window)
            if j >= 0:
                for c in range(Hkv):
                    qsum = q[ctxs[s] - 1, c * (H_ // Hkv):(c + 1) * (H_ // Hkv)].sum(0)
                    k[j, c] = 4.0 * qsum / qsum.norm() * math.sqrt(D)
        k, q = k.to(dtype), q.to(dtype)
        table = [order.pop() for _ in range(pages_needed[s])]
        for p in range(ctxs[s]):
            kc[table[p // ps], :, p % ps, :] = k[p]
        ks.append(k), qs_.append(q), tables.append(table)
    r1 = torch.rand(H_, generator=g) * 2
    r2 = torch.rand(H_, generator=g) * 0.5 + 0.01
    talk = torch.eye(H_) + 0.3 * torch.randn(H_, H_, generator=g)
    gate = [torch.randn(n, H_ * D, generator=g).to(dtype) for n in qlens]
    scale = 1.3 / math.sqrt(D)
    want = []
    for s in range(S):
        w = plain.attention_weights(qs_[s].double(), ks[s].double(), scale, r1.double(), r2.double(), window)
        o = plain.apply_weights(plain.mix_heads(w, talk.double()), ks[s].double())[-qlens[s]:]
        want.append(o * torch.sigmoid(gate[s].double()))
    ents = [_entry(qlens[s], ctxs[s] - qlens[s], tables[s]) for s in range(S)]
    q_step = torch.cat([qs_[s][-qlens[s]:].reshape(qlens[s], -1) for s in range(S)])
    return dict(kc=kc.to(DEV), q=q_step.to(DEV), gate=torch.cat(gate).to(DEV), r1=r1.to(DEV), r2=r2.to(DEV),
                talk=talk.to(DEV), scale=scale, want=torch.cat(want), entries=ents)


def _run_attention(case, H_, Hkv, D, window, ps, talk=True):
    from servelab_b200.ops import attention as A
    ctx = _ctx(case["entries"])
    out = torch.empty_like(case["q"])
    A.talk_attention(ctx, case["q"], case["kc"], case["kc"], out, ctx.block_tables[0], H_, Hkv, D, ps,
                     case["scale"], window, case["r1"], case["r2"], case["talk"] if talk else None,
                     case["gate"])
    return out.cpu().double()


SHAPES = [  # heads, kv heads, head size, window, page size
    (6, 2, 64, 44, 16), (6, 3, 16, 12, 8), (2, 1, 32, 33, 4), (4, 4, 16, 1000, 16), (3, 1, 24, 5, 8),
    (8, 2, 128, 70, 16), (6, 3, 64, 1, 16), (12, 4, 128, 50, 8), (5, 5, 48, 9, 16)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("spike", [None, "in", "out"])
@pytest.mark.parametrize("shape", SHAPES)
def test_attention_over_portions(dtype, spike, shape):
    """Prompt portions of unequal requests in one step (the plain kernel in float32, the
    tensor-core prefill instance in bfloat16): far keys, the window's two edges, a portion of
    two tokens, a first token, a single token beside portions."""
    H_, Hkv, D, window, ps = shape
    ctxs, qlens = [150, 37, 2, 1, 81], [90, 37, 2, 1, 1]
    case = _attention_case(11, H_, Hkv, D, window, ctxs, qlens, ps, dtype, spike)
    got = _run_attention(case, H_, Hkv, D, window, ps)
    err = (got - case["want"]).abs().max()
    assert err < (2e-4 if dtype == torch.float32 else 0.25), err     # values reach 4 sqrt(D)
    rel = (got - case["want"]).norm() / case["want"].norm()
    assert rel < (1e-5 if dtype == torch.float32 else 1.5e-2), rel


@pytest.mark.parametrize("spike", [None, "in", "out"])
@pytest.mark.parametrize("shape", SHAPES)
def test_attention_of_single_tokens(spike, shape):
    """Steps of single tokens in bfloat16 (the split-key decode instance, whose splits the
    mixing kernel combines) against the oracle and against the plain kernel on the same data;
    contexts shorter than, equal to and far beyond the window."""
    from servelab_b200.ops import attention as A
    H_, Hkv, D, window, ps = shape
    ctxs = [1, 2, window, window + 1, 64, 65, 700, 333]
    case = _attention_case(5, H_, Hkv, D, window, ctxs, [1] * len(ctxs), ps, torch.bfloat16, spike)
    got = _run_attention(case, H_, Hkv, D, window, ps)
    rel = (got - case["want"]).norm() / case["want"].norm()
    assert rel < 1.5e-2, rel
    A.force_generic = True
    try:
        twin = _run_attention(case, H_, Hkv, D, window, ps)
    finally:
        A.force_generic = False
    assert (got - twin).norm() / twin.norm() < 1.5e-2
    if D % 16 == 0:
        from servelab_b200.ops import kernels as K
        assert K.attention_status(D) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_without_mixed_heads(dtype):
    """The same kernels for a mixer that does not mix its heads: each head's own kv head only."""
    H_, Hkv, D, window, ps = 4, 2, 32, 20, 8
    for qlens in ([30, 1, 2], [1, 1, 1]):
        case = _attention_case(3, H_, Hkv, D, window, [64, 9, 40], qlens, ps, dtype, "in")
        case["talk"] = torch.eye(H_, device=DEV)            # what the oracle is to compute ...
        w = _run_attention(case, H_, Hkv, D, window, ps)
        got = _run_attention(case, H_, Hkv, D, window, ps, talk=False)       # ... without a matrix
        assert (got - w).abs().max() < (1e-5 if dtype == torch.float32 else 0.1)


# ------------------------------------------------------------ whole models
LENGTHS = [70, 45, 190, 33, 2, 1, 58]
TOL = {"float32": 1e-5, "bfloat16": 1.5e-2}       # about twice the worst error the tests print


@pytest.fixture(scope="module", params=["P", "Q", "R"])
def model(request, tmp_path_factory):
    cfg, seed, page = C.CASES[request.param]
    folder = C.make_model(str(tmp_path_factory.mktemp(f"dez_{request.param}")), cfg, seed)
    reqs = {f"r{i}": H.random_ids(n, cfg["vocab"], 100 * seed + i) for i, n in enumerate(LENGTHS)}
    pc, pw = plain.load_folder(folder)
    ref = {rid: plain.forward_logits(pc, pw, ids).float().numpy() for rid, ids in reqs.items()}
    return {"name": request.param, "cfg": cfg, "folder": folder, "page": page, "requests": reqs,
            "ref": ref, "plain": (pc, pw)}


def _bulk_tail(requests, tail):
    """Most of a request in one step, its last ``tail`` tokens one by one (a request of one
    token ends with its only step)."""
    steps = H.trace_bulk_tail(requests, tail=tail)
    last = {}
    for st in steps:
        for e in st["entries"]:
            last[e["id"]] = st
    for rid, st in last.items():
        if rid not in st["end"]:
            st["end"].append(rid)
    return steps


def _replay(model, dtype, steps, max_tokens=None, **kw):
    from servelab_b200.replay import TraceSession
    sess = TraceSession(model["folder"], dtype, max_tokens or H.peak_tokens(steps), page_size=model["page"],
                        max_live=4, poison_cache=True, **kw)
    got = H.collect(steps, H.run_session(sess, steps), model["cfg"]["vocab"])
    sess.cache.check_invariants()
    assert not sess.held and all(p.num_free() == p.num_pages for p in sess.cache.pools)
    assert sess.cache.slots.num_free() == 4
    return got, sess


def _compare(model, dtype, got):
    scale = max(float(np.abs(r).max()) for r in model["ref"].values())
    worst = 0.0
    for rid, ids in model["requests"].items():
        assert sorted(got[rid]) == list(range(len(ids))), f"{rid}: positions missing"
        for pos in range(len(ids)):
            err = float(np.abs(got[rid][pos] - model["ref"][rid][pos]).max())
            assert err <= TOL[dtype] * max(1.0, scale / 5), (
                f"config {model['name']} {dtype} request {rid}: first wrong position {pos} (err {err:.3e})")
            worst = max(worst, err)
    print(f"config {model['name']} {dtype}: worst abs logit error {worst:.3e} (logits up to {scale:.2f})")


def test_the_residual_stream_after_every_layer(model):
    """float32, one request: the stream each block leaves (with its pending update added)
    against the oracle's stream after that layer."""
    from servelab_b200.replay import TraceSession
    pc, pw = model["plain"]
    streams = []
    ids = model["requests"]["r1"]
    plain.forward_logits(pc, pw, ids, streams)
    sess = TraceSession(model["folder"], "float32", 64, page_size=model["page"])
    seen = []
    for block in sess.runner.model.blocks:
        def fwd(ctx, resid, delta, cache, owns, _f=block.forward):
            resid, delta = _f(ctx, resid, delta, cache, owns)
            seen.append(resid.double().cpu() + delta.materialize().double().cpu())
            return resid, delta
        block.forward = fwd
    sess.run_step({"step": 0, "entries": [{"id": "x", "tokens": ids, "want": []}], "end": ["x"]})
    assert len(seen) == len(streams)
    for i, (got, want) in enumerate(zip(seen, streams)):
        assert (got - want).abs().max() < 1e-4 * max(1.0, float(want.abs().max())), f"layer {i}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole(model, dtype):
    got, _ = _replay(model, dtype, H.trace_whole(model["requests"]))
    _compare(model, dtype, got)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompt_then_token_by_token_beyond_every_window(model, dtype):
    """The last 120 tokens one by one: every window (and the longest convolution) passes over
    decoded tokens, and windowed groups give pages back while the request still decodes."""
    steps = _bulk_tail(model["requests"], 120)
    got, _ = _replay(model, dtype, steps)
    _compare(model, dtype, got)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_down_to_two_tokens(model, dtype):
    got, _ = _replay(model, dtype, H.trace_portions(model["requests"]))
    _compare(model, dtype, got)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_with_pages_and_slots_used_again(model, dtype):
    steps = H.trace_mixed(model["requests"], seed=4)
    need = H.peak_tokens(steps)
    assert need < sum(-(-len(v) // 64) * 64 for v in model["requests"].values())
    assert len(model["requests"]) > 4                       # more requests than state slots
    got, _ = _replay(model, dtype, steps, need)
    _compare(model, dtype, got)


def test_float32_logits_do_not_depend_on_the_cut(model):
    whole, _ = _replay(model, "float32", H.trace_whole(model["requests"]))
    for steps in (H.trace_portions(model["requests"]), H.trace_mixed(model["requests"], seed=9),
                  _bulk_tail(model["requests"], 40)):
        got, _ = _replay(model, "float32", steps)
        for rid in whole:
            for pos in whole[rid]:
                assert np.abs(got[rid][pos] - whole[rid][pos]).max() <= 2e-6, (rid, pos)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_single_token_steps_through_replayed_graphs(model, dtype):
    """Steps of single tokens replay a captured graph (the convolution's state is indexed on
    the device and put back after the warm-up run): the same logits as eager steps."""
    steps = _bulk_tail(model["requests"], 40)
    eager, _ = _replay(model, dtype, steps)
    graphs, sess = _replay(model, dtype, steps, cuda_graphs=True)
    assert sess.runner.graph_replays > 0
    for rid in eager:
        for pos in eager[rid]:
            assert np.abs(graphs[rid][pos] - eager[rid][pos]).max() <= (2e-6 if dtype == "float32" else 1e-1)
    _compare(model, dtype, graphs)


def test_the_trace_runner_as_a_program(model, tmp_path):
    """bin/trace_run on a model folder, steps on standard input, logits in files: the mixed
    trace in bfloat16, rows against the oracle."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    steps = H.trace_mixed(model["requests"], seed=21)
    out = tmp_path / "out"
    proc = subprocess.run(
        [sys.executable, os.path.join(root, "bin", "trace_run"), "--model", model["folder"], "--dtype", "bfloat16",
         "--out", str(out), "--max-tokens", str(H.peak_tokens(steps)), "--page-size", str(model["page"])],
        input="".join(json.dumps(st) + "\n" for st in steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [ln for ln in proc.stdout.splitlines() if ln.startswith("done ")] == [f"done {st['step']}" for st in steps]
    V = model["cfg"]["vocab"]
    outputs = {st["step"]: np.fromfile(out / f"{st['step']}.f32", dtype="<f4").reshape(-1, V)
               for st in steps if any(e["want"] for e in st["entries"])}
    _compare(model, "bfloat16", H.collect(steps, outputs, V))


# --------------------------------------------------------------- generation
def _engine(model, dtype="float32", num_blocks=256, budget=2048, **kw):
    from servelab_b200.config import CacheConfig, SchedulerConfig
    from servelab_b200.engine.llm_engine import LLMEngine
    return LLMEngine(model["folder"], CacheConfig(block_size=model["page"], num_blocks=num_blocks),
                     SchedulerConfig(max_num_seqs=4, max_num_batched_tokens=budget), dtype=dtype, **kw)


def test_greedy_generation_through_the_engine(model):
    """The entry point and its scheduler (continuous batching, portions under a token budget,
    graphs, look-ahead) generate what the oracle generates, also with so few pages that requests
    are preempted and recomputed from a cleared state slot."""
    from servelab_b200.sampling import SamplingParams
    pc, pw = model["plain"]
    prompts = [model["requests"][r][:n] for r, n in (("r0", 41), ("r1", 3), ("r2", 77), ("r5", 1), ("r3", 20))]
    n_new = 14
    want = [plain.greedy(pc, pw, p, n_new) for p in prompts]
    sp = SamplingParams(temperature=0.0, max_tokens=n_new, ignore_eos=True)
    outs = _engine(model).generate(prompts, sp)
    assert [o.outputs[0].token_ids for o in outs] == want
    outs = _engine(model, budget=16, cuda_graphs=False).generate(prompts, sp)
    assert [o.outputs[0].token_ids for o in outs] == want
    few = -(-(77 + n_new) // model["page"]) + 2
    eng = _engine(model, num_blocks=few, budget=24)
    outs = eng.generate(prompts, sp)
    assert [o.outputs[0].token_ids for o in outs] == want
    eng.runner.cache.check_invariants()
    st = eng.stats()
    assert st["running"] == 0 and st["pages_used"] == [0] * len(st["pages_used"])


def test_command_line(model, tmp_path):
    """``python -m servelab_b200 --model <folder>`` chooses the model class by config.json and
    generates what the oracle generates; ``--random-weights config.json`` writes a model of the
    design from its config alone."""
    import json
    import os
    import subprocess
    import sys
    if model["name"] != "P":
        pytest.skip("one configuration is enough for the command line")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    pc, pw = model["plain"]
    want = plain.greedy(pc, pw, [3, 1, 4, 1, 5], 6)
    r = subprocess.run([sys.executable, "-m", "servelab_b200", "--model", model["folder"],
                        "--prompt-ids", "3,1,4,1,5", "--max-tokens", "6", "--temperature", "0",
                        "--dtype", "float32", "--ignore-eos", "--block-size", "8", "--num-blocks", "32"],
                       cwd=root, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert f"finish=length -> {want}" in r.stdout and "stats:" in r.stdout
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(C.R))
    r = subprocess.run([sys.executable, "-m", "servelab_b200", "--random-weights", str(cfg_path),
                        "--prompt-ids", "1,2,3", "--max-tokens", "5", "--temperature", "0.8", "--seed", "3",
                        "--ignore-eos", "--block-size", "4", "--num-blocks", "32"],
                       cwd=root, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "finish=length" in r.stdout, r.stderr[-2000:]
