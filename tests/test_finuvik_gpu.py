"""Finuvik through the engine (ModelRunner, the cache manager, the scheduler, LLM.generate, bin/trace_run) against
the plain float64 statement in tests/plain_finuvik.py, on small models made here with weights that make faults show."""
import math
import os

import numpy as np
import pytest
import torch

import plain_finuvik as P
from helpers import Replay, assert_close, random_ids, write_model

pytestmark = pytest.mark.gpu


def _layer(heads, kv, dim, vdim, rh, rdim, rvdim, ff, ls=0.7, rs=1.1, q_temp=None, scale=None, weights_of=None):
    left = dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale if scale is not None else dim ** -0.5)
    if q_temp:
        left["q_temp"] = dict(coef=q_temp[0], every=q_temp[1])
    e = dict(type="parallel", mixer=dict(left=left, left_scale=ls, right=dict(heads=rh, dim=rdim, vdim=rvdim), right_scale=rs),
             mlp=dict(ff=ff, kind="dense") if ff else None)
    if weights_of is not None:
        e["weights_of"] = weights_of
    return e


def _cfg(width, vocab, max_positions, eps, layers):
    return dict(architecture="Finuvik", width=width, vocab=vocab, max_positions=max_positions, norm=dict(eps=eps), layers=layers)


# X: grouped key/value heads, a query temperature that steps every 8 positions, a layer run twice with the same
# tensors, a layer whose key and value heads have one size and as many key/value heads as query heads, no query
# temperature and no feed-forward, and that layer's tensors used once more: two cache groups, four states.
_X0 = _layer(4, 2, 16, 24, 2, 16, 40, 96, q_temp=(0.5, 8), scale=0.3)
_X2 = _layer(2, 2, 32, 32, 3, 8, 16, None, ls=1.2, rs=0.4)
CFG_X = _cfg(64, 97, 160, 1e-6, [_X0, dict(_X0, weights_of=0), _X2, dict(_X2, weights_of=2)])
# Y: one key/value head under six query heads, value heads smaller than key heads, a recurrent branch with one
# head, longer contexts (the temperature steps at 100, 200, ...), every layer with tensors of its own.
CFG_Y = _cfg(96, 211, 700, 1e-5, [_layer(6, 1, 24, 8, 1, 32, 64, 64, q_temp=(0.3, 100)),
                                  _layer(3, 3, 8, 40, 4, 4, 8, 160, ls=0.5, rs=0.5, q_temp=(0.25, 1))])
CONFIGS = {"X": CFG_X, "Y": CFG_Y}
PAGE = {"X": 8, "Y": 16}


def make_tensors(cfg, seed):
    """Weights that make faults show: projections large enough for a peaked softmax (scores of a few units, up to
    about ten where the query temperature is highest: single keys carry weight, while the bfloat16 rounding of
    queries and keys still moves a score by less than a tenth), distance penalties that matter but leave far keys
    alive, forget gates between fast and very slow, norm weights away from zero."""
    g = torch.Generator().manual_seed(seed)
    D = cfg["width"]

    def normal(*shape, std):
        return torch.empty(*shape).normal_(0.0, std, generator=g)

    def uniform(*shape, lo, hi):
        return torch.empty(*shape).uniform_(lo, hi, generator=g)

    t = {"embed": normal(cfg["vocab"], D, std=0.7), "pos": normal(cfg["max_positions"], D, std=0.4),
         "final.norm": normal(D, std=0.2), "head": normal(cfg["vocab"], D, std=1.0 / math.sqrt(D))}
    for i, lay in enumerate(cfg["layers"]):
        if lay.get("weights_of") is not None:
            continue
        L, R, p = lay["mixer"]["left"], lay["mixer"]["right"], f"l{i}."
        t[p + "norm1"] = normal(D, std=0.2)
        t[p + "mix.left.q"] = normal(L["heads"] * L["dim"], D, std=1.6 / math.sqrt(D))
        t[p + "mix.left.k"] = normal(L["kv_heads"] * L["dim"], D, std=1.6 / math.sqrt(D))
        t[p + "mix.left.v"] = normal(L["kv_heads"] * L["vdim"], D, std=1.0 / math.sqrt(D))
        t[p + "mix.left.r1"] = uniform(L["heads"], lo=0.1, hi=1.0)
        t[p + "mix.left.r2"] = uniform(L["heads"], lo=0.02, hi=0.6)
        t[p + "mix.left.o"] = normal(D, L["heads"] * L["vdim"], std=0.7 / math.sqrt(L["heads"] * L["vdim"]))
        t[p + "mix.right.q"] = normal(R["heads"] * R["dim"], D, std=1.0 / math.sqrt(D))
        t[p + "mix.right.f"] = normal(R["heads"] * R["dim"], D, std=2.0 / math.sqrt(D))
        t[p + "mix.right.f.b"] = normal(R["heads"] * R["dim"], std=1.0)
        t[p + "mix.right.lower"] = uniform(R["heads"] * R["dim"], lo=0.0, hi=0.995)
        t[p + "mix.right.v"] = normal(R["heads"] * R["vdim"], D, std=1.0 / math.sqrt(D))
        t[p + "mix.right.norm"] = uniform(R["vdim"], lo=0.5, hi=1.5)
        t[p + "mix.right.o"] = normal(D, R["heads"] * R["vdim"], std=0.7 / math.sqrt(R["heads"] * R["vdim"]))
        if lay.get("mlp"):
            F = lay["mlp"]["ff"]
            t[p + "norm2"] = normal(D, std=0.2)
            t[p + "mlp.gate"] = normal(F, D, std=1.0 / math.sqrt(D))
            t[p + "mlp.up"] = normal(F, D, std=1.0 / math.sqrt(D))
            t[p + "mlp.down"] = normal(D, F, std=0.7 / math.sqrt(F))
    return t


def make_model(folder, which, seed=0, dtype=torch.float32):
    tensors = {k: v.to(torch.bfloat16).float() for k, v in make_tensors(CONFIGS[which], seed).items()}
    return write_model(str(folder), CONFIGS[which], tensors, dtype), tensors


def oracle(tensors, cfg, ids, dtype):
    return P.forward(tensors, cfg, ids, store=P.to_bf16 if dtype == "bfloat16" else P._keep).numpy()


def runner_for(folder, which, dtype, pages=120, seqs=4, graphs=False):
    from mini_llm_b200.config.base import EngineConfig
    from mini_llm_b200.engine.runner import ModelRunner
    return ModelRunner(folder, EngineConfig(dtype=dtype, page_size=PAGE[which], num_pages=pages, max_num_seqs=seqs,
                                            use_cuda_graphs=graphs))


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for which in CONFIGS:
        folder, tensors = make_model(tmp_path_factory.mktemp("finuvik_" + which), which, seed=3)
        out[which] = (folder, tensors)
    return out


def test_layers_one_by_one_in_float32(models):
    """The residual stream after every layer run (a layer that runs twice counts twice) against the oracle's."""
    from mini_llm_b200 import ops
    from mini_llm_b200.engine.runner import StepEntry
    for which in CONFIGS:
        folder, tensors = models[which]
        ids = random_ids(41, CONFIGS[which]["vocab"], 5)
        res = []
        P.forward(tensors, CONFIGS[which], ids, residuals=res)
        r = runner_for(folder, which, "float32")
        r.add_request("a")
        ctx = r.prepare_step([StepEntry("a", ids, [0])])
        m = r.model
        with ops.stream_scope():
            x = m.embedding.forward(ctx, m.positions)
            for i, (entry, cache) in enumerate(zip(m.spec.schedule, m._caches)):
                layer = m.layers[entry.layer]
                x = layer.arrangement(layer, x, ctx, cache)
                got = x.double().cpu()
                assert (got - res[i]).abs().max() < 3e-5 * res[i].abs().max(), (which, i)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["X", "Y"])
def test_whole_prompts_then_token_by_token(models, which, dtype):
    from mini_llm_b200.engine.runner import StepEntry
    folder, tensors = models[which]
    cfg = CONFIGS[which]
    n = 150 if which == "X" else 330             # Y crosses the temperature steps at 100, 200, 300 and a split of keys
    ids = random_ids(n, cfg["vocab"], 7)
    want = oracle(tensors, cfg, ids, dtype)
    r = runner_for(folder, which, dtype)
    r.add_request("w")
    got = r.step([StepEntry("w", ids, list(range(n)))]).cpu().numpy()
    assert_close(got, want, dtype, "whole")
    r.finish_request("w")
    # most of it in one step, the rest one by one (long decoding: 60 tokens, through the same pages and slot again)
    r.add_request("d")
    head = n - 60
    rows = [r.step([StepEntry("d", ids[:head], [0, 1, 2, head - 1])]).cpu().numpy()]
    for t in range(head, n):
        rows.append(r.step([StepEntry("d", [ids[t]], [0])]).cpu().numpy())
    assert_close(np.concatenate(rows), want[[0, 1, 2, head - 1] + list(range(head, n))], dtype, "decode")
    # from the very first token on, one by one: the first tokens of a sequence
    r.finish_request("d")
    r.add_request("f")
    rows = [r.step([StepEntry("f", [ids[t]], [0])]).cpu().numpy() for t in range(20)]
    assert_close(np.concatenate(rows), want[:20], dtype, "first tokens")
    r.finish_request("f")
    r.cache.check()
    assert r.cache.num_live == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["X", "Y"])
def test_portions_of_many_sizes(models, which, dtype):
    from mini_llm_b200.engine.runner import StepEntry
    folder, tensors = models[which]
    cfg = CONFIGS[which]
    n = 157
    ids = random_ids(n, cfg["vocab"], 11)
    want = oracle(tensors, cfg, ids, dtype)
    r = runner_for(folder, which, dtype)
    for cuts in ([2, 2, 3, 64, 1, 31, 2, 17, 33, 2], [65, 63, 2, 27], [7] * 22 + [3]):
        assert sum(cuts) == n
        r.add_request("p")
        rows, at = [], 0
        for c in cuts:
            rows.append(r.step([StepEntry("p", ids[at:at + c], list(range(c)))]).cpu().numpy())
            at += c
        assert_close(np.concatenate(rows), want, dtype, f"portions {cuts[:4]}")
        r.finish_request("p")
    r.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["X", "Y"])
@pytest.mark.parametrize("graphs", [False, True])
def test_unequal_requests_batched_with_pages_and_slots_used_again(models, which, dtype, graphs):
    """Five requests through three slots and a pool that cannot hold them all at once: portions beside single
    tokens, requests that sit a step out, slots and pages that are given back and taken by the next request,
    whose state must start from zero.  Every row equals the request run alone (the oracle)."""
    from mini_llm_b200.engine.runner import StepEntry
    folder, tensors = models[which]
    cfg = CONFIGS[which]
    lens = {"a": 90, "b": 13, "c": 121, "d": 2, "e": 64}
    ids = {k: random_ids(n, cfg["vocab"], 20 + i) for i, (k, n) in enumerate(lens.items())}
    want = {k: oracle(tensors, cfg, v, dtype) for k, v in ids.items()}
    plan = {"a": [30, 2, 1, 1, 40, 1, 1, 14], "b": [2, 1, 1, 9], "c": [64, 1, 0, 50, 2, 1, 1, 1, 1], "d": [2],
            "e": [1, 1, 1, 1, 1, 59]}
    ps = PAGE[which]
    r = runner_for(folder, which, dtype, pages=(90 + 16 + 121 + 64) // ps + 6, seqs=3, graphs=graphs)
    waiting, live, at, got = ["a", "b", "c", "d", "e"], [], {k: 0 for k in lens}, {k: [] for k in lens}
    steps = 0
    while waiting or live:
        while waiting and len(live) < 3:
            k = waiting.pop(0)
            r.add_request(k)
            live.append(k)
        entries = []
        for k in live:
            c = plan[k].pop(0)
            if c:
                entries.append(StepEntry(k, ids[k][at[k]:at[k] + c], list(range(c))))
        out = r.step(entries).cpu().numpy()
        o = 0
        for e in entries:
            c = len(e.tokens)
            got[e.req].append(out[o:o + c])
            o += c
            at[e.req] += c
        for k in list(live):
            if not plan[k]:
                r.finish_request(k)
                live.remove(k)
        steps += 1
        r.cache.check()
    for k in lens:
        assert_close(np.concatenate(got[k]), want[k], dtype, f"request {k}")
    assert r.cache.num_live == 0
    assert all(g.allocator.num_in_use == 0 for g in r.cache.groups)


def test_a_slot_that_is_used_again_starts_from_zero(models):
    """One slot: the second request gets the first one's slot and pages."""
    from mini_llm_b200.engine.runner import StepEntry
    folder, tensors = models["X"]
    cfg = CONFIGS["X"]
    r = runner_for(folder, "X", "float32", pages=8, seqs=1)
    for seed in (1, 2, 3):
        ids = random_ids(50, cfg["vocab"], seed)
        r.add_request(seed)
        got = r.step([StepEntry(seed, ids, [0, 25, 49])]).cpu().numpy()
        assert_close(got, oracle(tensors, cfg, ids, "float32")[[0, 25, 49]], "float32", f"request {seed}")
        r.finish_request(seed)


def test_layers_that_share_tensors_keep_caches_of_their_own(models):
    from mini_llm_b200.cache.manager import PagedNeed, StateNeed
    folder, _ = models["X"]
    r = runner_for(folder, "X", "float32")
    assert len(r.model.layers) == 2 and len(r.spec.schedule) == 4
    units = [e.cache_unit for e in r.spec.schedule]
    assert len(set(units)) == 4
    assert len(r.cache.groups) == 2 and len(r.cache.states) == 4       # two kinds of pages, a state per run
    ptrs = {c.k_pages.data_ptr() for c in r.model._caches} | {c.state.data_ptr() for c in r.model._caches}
    assert len(ptrs) == 8
    g0 = r.cache.groups[r.cache.group_of_layer[units[0]]]
    assert g0.need == PagedNeed(kv_heads=2, head_dim=16, v_head_dim=24) and g0.pool is None and g0.pool_v.shape[-1] == 24
    g1 = r.cache.groups[r.cache.group_of_layer[units[2]]]
    assert g1.need.value_dim == 32 and g1.pool is not None
    assert r.cache.state_layers[units[3]] == StateNeed((3, 8, 16), "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(models, dtype):
    """LLM.generate (scheduler, prompt portions under a small token budget, decoding several requests together,
    slots used again) gives the oracle's greedy tokens; where the oracle's two best logits are closer than the
    comparison rule allows, either token is taken and the oracle follows the engine."""
    from mini_llm_b200 import LLM, SamplingParams
    folder, tensors = models["X"]
    cfg = CONFIGS["X"]
    prompts = [random_ids(n, cfg["vocab"], 40 + n) for n in (33, 5, 70, 1, 18)]
    new = 12
    llm = LLM(folder, dtype=dtype, page_size=8, num_pages=60, max_num_seqs=3, max_num_batched_tokens=48, prefill_chunk=32)
    outs = llm.generate(prompts, SamplingParams(max_new_tokens=new, ignore_eos=True))
    margin = 1e-3 if dtype == "float32" else 0.15
    for p, out in zip(prompts, outs):
        assert len(out) == new
        seq = list(p)
        for tok in out:
            logits = oracle(tensors, cfg, seq, dtype)[-1]
            best = int(np.argmax(logits))
            assert tok == best or logits[best] - logits[tok] < margin, (len(p), len(seq))
            seq.append(tok)
    assert llm.runner.cache.num_live == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_with_graphs(models, dtype, tmp_path):
    """bin/trace_run on a Finuvik folder: config.json picks the model class; steps that come back are replayed as
    CUDA graphs, and a replayed step advances the recurrent state once."""
    folder, tensors = models["Y"]
    cfg = CONFIGS["Y"]
    ids = {k: random_ids(n, cfg["vocab"], 60 + i) for i, (k, n) in enumerate({"p": 70, "q": 45}.items())}
    want = {k: oracle(tensors, cfg, v, dtype) for k, v in ids.items()}
    os.makedirs(tmp_path / "out")
    rp = Replay(folder, dtype, str(tmp_path / "out"), 192, page_size=PAGE["Y"])
    got = {k: [] for k in ids}
    at = {k: 0 for k in ids}
    plan = [[("p", 40), ("q", 30)]] + [[("p", 1), ("q", 1)]] * 15 + [[("p", 15)]]
    for n, step in enumerate(plan):
        entries = [(k, ids[k][at[k]:at[k] + c], list(range(c))) for k, c in step]
        end = [k for k, c in step if at[k] + c == len(ids[k])]
        out = rp.step(entries, end)
        o = 0
        for k, c in step:
            got[k].append(out[o:o + c])
            o += c
            at[k] += c
    assert rp.close() == 0
    assert rp.stats["graph_replays"] >= 13
    for k in ids:
        assert_close(np.concatenate(got[k]), want[k], dtype, f"replayed request {k}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_contexts_and_a_layer_that_borrows_from_a_later_one(tmp_path, dtype):
    """2,300 tokens (more than a step's scratch holds at first: it grows), keys thousands of positions back, temperature
    steps at 512 and 1000, a layer whose tensors are a later layer's, key heads of 40 (no tensor-core kernel) beside 64:
    whole, then in portions of 700 and single tokens, against the oracle at rows on both sides of every edge."""
    from mini_llm_b200.config.base import EngineConfig
    from mini_llm_b200.engine.runner import ModelRunner, StepEntry
    a = _layer(6, 3, 40, 72, 2, 48, 96, 200, q_temp=(0.2, 512))
    b = _layer(4, 4, 64, 64, 1, 16, 200, None, ls=0.6, rs=1.3, q_temp=(0.3, 1000))
    cfg = _cfg(136, 301, 2400, 1e-5, [a, dict(b, weights_of=2), b, dict(a, weights_of=0)])
    tensors = {k: v.to(torch.bfloat16).float() for k, v in make_tensors(cfg, 11).items()}
    folder = write_model(str(tmp_path / "long"), cfg, tensors)
    n = 2300
    ids = random_ids(n, cfg["vocab"], 1)
    want = oracle(tensors, cfg, ids, dtype)
    r = ModelRunner(folder, EngineConfig(dtype=dtype, page_size=16, num_pages=300, max_num_seqs=2))
    rows = [0, 1, 255, 256, 511, 512, 1023, 1024, 2047, 2048, 2299]
    r.add_request("w")
    assert_close(r.step([StepEntry("w", ids, rows)]).cpu().numpy(), want[rows], dtype, "whole")
    r.finish_request("w")
    r.add_request("p")
    got, at = [], 0
    for c in [700, 700, 700, 180] + [1] * 20:
        got.append(r.step([StepEntry("p", ids[at:at + c], [c - 1])]).cpu().numpy()[0])
        at += c
    idx = np.cumsum([700, 700, 700, 180] + [1] * 20) - 1
    assert_close(np.stack(got), want[idx], dtype, "portions and single tokens")
    assert r.graph_replays >= 15


def test_command_line_with_random_weights_and_sampling(models, tmp_path):
    """bin/mini_llm: the random-weights mode writes a Finuvik folder from a config.json; greedy tokens from the command
    line equal LLM.generate's; temperature sampling gives other tokens, and others again for another seed."""
    import json
    import subprocess
    import sys
    from helpers import ROOT
    from mini_llm_b200 import LLM, SamplingParams
    cfg_path = tmp_path / "cfg.json"
    cfg_path.write_text(json.dumps(CFG_Y))
    out_dir = tmp_path / "written"
    cli = [sys.executable, os.path.join(ROOT, "bin", "mini_llm")]
    prompts = ["5 17 3 90 9 100 4", "40 2 2 31"]
    tail = ["--dtype", "float32", "--max-new-tokens", "6", "--ignore-eos", "--max-batch-num", "2"]
    for p in prompts:
        tail += ["--prompt-ids", p]
    # one call writes the folder from the config and a seed, and generates greedily from it
    r = subprocess.run(cli + ["--random-config", str(cfg_path), "--seed", "7", "--write-model", str(out_dir)] + tail,
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and os.path.isfile(out_dir / "model.safetensors"), r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.endswith("[DONE]")]
    got = [[int(t) for t in l.replace("[DONE]", "").split()] for l in lines]
    llm = LLM(str(out_dir), dtype="float32", max_num_seqs=2)
    want = llm.generate([[int(t) for t in p.split()] for p in prompts], SamplingParams(max_new_tokens=6, ignore_eos=True))
    assert got == want
    runs = []
    for seed in ("3", "4"):
        r = subprocess.run(cli + ["--model", str(out_dir)] + tail + ["--temperature", "1.5", "--sample-seed", seed],
                           capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        runs.append(r.stdout)
    assert runs[0] != runs[1] and runs[0] != "\n".join(lines) + "\n"


def test_key_heads_whose_size_is_no_multiple_of_8(tmp_path):
    """Key rows are padded in the pages (the padding stays zero); everything else takes the size as it is."""
    from mini_llm_b200.engine.runner import StepEntry
    cfg = _cfg(40, 50, 64, 1e-5, [_layer(2, 1, 12, 10, 1, 6, 9, 24, q_temp=(0.4, 4)), _layer(3, 3, 5, 5, 2, 3, 3, None)])
    tensors = {k: v.to(torch.bfloat16).float() for k, v in make_tensors(cfg, 4).items()}
    folder = write_model(str(tmp_path / "odd"), cfg, tensors)
    ids = random_ids(50, cfg["vocab"], 9)
    for dtype in ("float32", "bfloat16"):
        want = oracle(tensors, cfg, ids, dtype)
        from mini_llm_b200.config.base import EngineConfig
        from mini_llm_b200.engine.runner import ModelRunner
        r = ModelRunner(folder, EngineConfig(dtype=dtype, page_size=8, num_pages=20, max_num_seqs=2, use_cuda_graphs=False))
        r.add_request("a")
        rows = [r.step([StepEntry("a", ids[:33], list(range(33)))]).cpu().numpy()]
        for t in range(33, 50):
            rows.append(r.step([StepEntry("a", [ids[t]], [0])]).cpu().numpy())
        assert_close(np.concatenate(rows), want, dtype, "odd sizes")


def test_sizes_no_kernel_takes_are_refused_at_construction(tmp_path):
    from mini_llm_b200.config.base import ConfigError, EngineConfig
    from mini_llm_b200.engine.runner import ModelRunner
    cfg = _cfg(64, 50, 32, 1e-5, [_layer(2, 1, 16, 16, 1, 256, 256, 32)])      # a state of 256 x 256 per head
    folder = write_model(str(tmp_path / "bad"), cfg, make_tensors(cfg, 0))
    with pytest.raises(ConfigError, match="threads"):
        ModelRunner(folder, EngineConfig(dtype="float32", num_pages=4))
