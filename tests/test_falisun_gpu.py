"""Falisun through the engine (ModelRunner, the cache manager, the scheduler, LLM.generate, bin/trace_run) against the
plain float64 statement in tests/plain_falisun.py, on small models made here with weights that make faults show."""
import os

import numpy as np
import pytest
import torch

import plain_falisun as P
from falisun_models import CONFIGS, PAGE, config, latent, layer, make_tensors, mamba, moe
from helpers import Replay, random_ids, write_model

pytestmark = pytest.mark.gpu


def oracle(tensors, cfg, ids, dtype):
    return P.forward(tensors, cfg, ids, store=P.to_bf16 if dtype == "bfloat16" else P._keep).numpy()


def close(got, want, dtype, what):
    """float32, row by row: relative error at most 4e-5 (twice the rule of the other models' tests: every branch's
    result, a sum of expert outputs that partly cancel, is normed again before it is added, which carries the sum's
    relative rounding error into the stream).  bfloat16: a router may send a token whose candidate experts score alike
    to the other one when a bfloat16 rounding upstream falls the other way, and that token then differs by more than
    rounding, by as much as two experts differ (and, through the cache and the state, so do some after it): the
    median row within 1e-2 and all but three in a hundred within 3e-2.  (The float32 runs hold every row; the kernels
    that only bfloat16 steps use are held row by row in tests/test_falisun_kernels_gpu.py.)"""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape and np.isfinite(got).all(), what
    err = np.linalg.norm(got - want, axis=1) / np.maximum(np.linalg.norm(want, axis=1), 1e-12)
    if dtype == "float32":
        assert err.max() <= 4e-5, f"{what}: row {err.argmax()}: relative error {err.max():.3e}"
        return
    assert np.median(err) <= 1e-2 and (err <= 3e-2).mean() >= 0.97, \
        f"{what}: {np.sort(err)[-5:]} median {np.median(err):.3e}, {(err <= 3e-2).mean():.2f} within 3e-2"


def runner_for(folder, which, dtype, pages=120, seqs=4, graphs=False):
    from mini_llm_b200.config.base import EngineConfig
    from mini_llm_b200.engine.runner import ModelRunner
    return ModelRunner(folder, EngineConfig(dtype=dtype, page_size=PAGE[which], num_pages=pages, max_num_seqs=seqs,
                                            use_cuda_graphs=graphs))


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for which in CONFIGS:
        tensors = make_tensors(CONFIGS[which], seed=3)
        folder = write_model(str(tmp_path_factory.mktemp("falisun_" + which)), CONFIGS[which], tensors, torch.bfloat16)
        out[which] = (folder, tensors)
    return out


def test_layers_one_by_one_in_float32(models):
    """The residual stream after every layer against the oracle's."""
    from mini_llm_b200 import ops
    from mini_llm_b200.engine.runner import StepEntry
    for which in CONFIGS:
        folder, tensors = models[which]
        ids = random_ids(75, CONFIGS[which]["vocab"], 5)
        res = []
        P.forward(tensors, CONFIGS[which], ids, layers_out=res)
        r = runner_for(folder, which, "float32")
        r.add_request("a")
        ctx = r.prepare_step([StepEntry("a", ids, [0])])
        m = r.model
        with ops.stream_scope():
            x = m.embedding.forward(ctx, m.positions)
            for i, (entry, cache) in enumerate(zip(m.spec.schedule, m._caches)):
                lay = m.layers[entry.layer]
                x = lay.arrangement(lay, x, ctx, cache)
                assert (x.double().cpu() - res[i]).abs().max() < 3e-5 * res[i].abs().max(), (which, i)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["P", "Q"])
def test_whole_prompts_then_token_by_token(models, which, dtype):
    from mini_llm_b200.engine.runner import StepEntry
    folder, tensors = models[which]
    cfg = CONFIGS[which]
    n = 330                                    # past a split of 256 keys and, in P, ten times YaRN's original context
    ids = random_ids(n, cfg["vocab"], 7)
    want = oracle(tensors, cfg, ids, dtype)
    r = runner_for(folder, which, dtype)
    r.add_request("w")
    got = r.step([StepEntry("w", ids, list(range(n)))]).cpu().numpy()
    close(got, want, dtype, "whole")
    r.finish_request("w")
    # most of it in one step, the rest one by one: long decoding through the pages and the slot just given back
    r.add_request("d")
    head = n - 90
    rows = [r.step([StepEntry("d", ids[:head], [0, 1, 2, head - 1])]).cpu().numpy()]
    for t in range(head, n):
        rows.append(r.step([StepEntry("d", [ids[t]], [0])]).cpu().numpy())
    close(np.concatenate(rows), want[[0, 1, 2, head - 1] + list(range(head, n))], dtype, "decode")
    r.finish_request("d")
    # from the very first token on, one by one: the first tokens of a sequence (the convolution's zeros, one key)
    r.add_request("f")
    rows = [r.step([StepEntry("f", [ids[t]], [0])]).cpu().numpy() for t in range(20)]
    close(np.concatenate(rows), want[:20], dtype, "first tokens")
    r.finish_request("f")
    r.cache.check()
    assert r.cache.num_live == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["P", "Q"])
def test_portions_of_many_sizes(models, which, dtype):
    """Cuts shorter than the convolution's reach (1, 2 and 3 tokens), mid-page, mid-chunk, across a split."""
    from mini_llm_b200.engine.runner import StepEntry
    folder, tensors = models[which]
    cfg = CONFIGS[which]
    n = 290
    ids = random_ids(n, cfg["vocab"], 11)
    want = oracle(tensors, cfg, ids, dtype)
    r = runner_for(folder, which, dtype)
    for cuts in ([2, 2, 3, 64, 1, 31, 2, 17, 33, 2, 1, 1, 2, 129], [65, 63, 2, 27, 99, 34], [7] * 41 + [3]):
        assert sum(cuts) == n
        r.add_request("p")
        rows, at = [], 0
        for c in cuts:
            rows.append(r.step([StepEntry("p", ids[at:at + c], list(range(c)))]).cpu().numpy())
            at += c
        close(np.concatenate(rows), want, dtype, f"portions {cuts[:4]}")
        r.finish_request("p")
    r.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["P", "Q"])
@pytest.mark.parametrize("graphs", [False, True])
def test_unequal_requests_batched_with_pages_and_slots_used_again(models, which, dtype, graphs):
    """Five requests through three slots and a pool that cannot hold them all at once: portions beside single tokens,
    requests that sit a step out, slots and pages given back and taken by the next request, whose states must start
    from zero.  Every row equals the request run alone (the oracle)."""
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
        r.cache.check()
    for k in lens:
        close(np.concatenate(got[k]), want[k], dtype, f"request {k}")
    assert r.cache.num_live == 0
    assert all(g.allocator.num_in_use == 0 for g in r.cache.groups)


def test_a_request_alone_and_in_a_batch(models):
    """What else is in the step changes nothing beyond rounding (a product of more rows may take another kernel):
    a request's rows alone and beside two others, in float32."""
    from mini_llm_b200.engine.runner import StepEntry
    for which in CONFIGS:
        folder, _ = models[which]
        cfg = CONFIGS[which]
        a, b, c = (random_ids(n, cfg["vocab"], 70 + n) for n in (37, 9, 64))
        r = runner_for(folder, which, "float32")
        r.add_request("a")
        alone = [r.step([StepEntry("a", a[:30], [29])]).clone()]
        alone += [r.step([StepEntry("a", [t], [0])]).clone() for t in a[30:]]
        r.finish_request("a")
        for k in "abc":
            r.add_request(k)
        r.step([StepEntry("c", c[:5], []), StepEntry("b", b[:3], [])])
        both = [r.step([StepEntry("b", b[3:], []), StepEntry("a", a[:30], [29]), StepEntry("c", c[5:40], [0])])[:1].clone()]
        for i, t in enumerate(a[30:]):
            both.append(r.step([StepEntry("c", [c[40 + i]], [0]), StepEntry("a", [t], [0])])[1:2].clone())
        a1, a2 = torch.cat(alone).double(), torch.cat(both).double()
        assert ((a1 - a2).norm(dim=1) / a1.norm(dim=1)).max() < 2e-5, which


def test_a_slot_that_is_used_again_starts_from_zero(models):
    """One slot: the second request gets the first one's slot (state and convolution inputs) and pages."""
    from mini_llm_b200.engine.runner import StepEntry
    folder, tensors = models["P"]
    cfg = CONFIGS["P"]
    r = runner_for(folder, "P", "float32", pages=8, seqs=1)
    for seed in (1, 2, 3):
        ids = random_ids(50, cfg["vocab"], seed)
        r.add_request(seed)
        got = r.step([StepEntry(seed, ids, [0, 25, 49])]).cpu().numpy()
        close(got, oracle(tensors, cfg, ids, "float32")[[0, 25, 49]], "float32", f"request {seed}")
        r.finish_request(seed)


def test_a_layer_that_reads_another_layers_rows_has_no_pool_of_its_own(models):
    from mini_llm_b200.cache.manager import PagedNeed, StateNeed
    folder, _ = models["Q"]
    r = runner_for(folder, "Q", "float32")
    caches = r.model._caches
    assert caches[2].k_pages.data_ptr() == caches[1].k_pages.data_ptr() and not caches[2].write and caches[1].write
    assert caches[3].k_pages.data_ptr() != caches[1].k_pages.data_ptr()
    assert len(r.cache.groups) == 2 and sorted(len(g.layers) for g in r.cache.groups) == [1, 1]
    g = r.cache.groups[r.cache.group_of_layer[1]]
    assert g.need == PagedNeed(kv_heads=1, head_dim=152, values_in_keys=True) and g.pool is None and g.pool_v is None
    assert g.v_pages(0) is None and g.pool_k.shape[-1] == 152
    # one state per request: the heads' states and the last taps - 1 inputs of the convolution
    assert r.cache.state_layers[0] == StateNeed((6 * 64 * 16 + 2 * (96 + 2 * 3 * 64),), "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(models, dtype):
    """LLM.generate (scheduler, prompt portions under a small token budget, several requests decoding together, slots
    used again) gives the oracle's greedy tokens; where the oracle's two best logits are closer than the comparison
    rule allows, either token is taken and the oracle follows the engine."""
    from mini_llm_b200 import LLM, SamplingParams
    folder, tensors = models["P"]
    cfg = CONFIGS["P"]
    prompts = [random_ids(n, cfg["vocab"], 40 + n) for n in (33, 5, 70, 1, 18)]
    new = 12
    llm = LLM(folder, dtype=dtype, page_size=8, num_pages=60, max_num_seqs=3, max_num_batched_tokens=48, prefill_chunk=32)
    outs = llm.generate(prompts, SamplingParams(max_new_tokens=new, ignore_eos=True))
    margin = 1e-3 if dtype == "float32" else 0.25
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
    """bin/trace_run on a Falisun folder: config.json picks the model class; steps that come back are replayed as CUDA
    graphs, and a replayed step advances the states once."""
    folder, tensors = models["Q"]
    cfg = CONFIGS["Q"]
    ids = {k: random_ids(n, cfg["vocab"], 60 + i) for i, (k, n) in enumerate({"p": 70, "q": 45}.items())}
    want = {k: oracle(tensors, cfg, v, dtype) for k, v in ids.items()}
    os.makedirs(tmp_path / "out")
    rp = Replay(folder, dtype, str(tmp_path / "out"), 192, page_size=PAGE["Q"])
    got = {k: [] for k in ids}
    at = {k: 0 for k in ids}
    plan = [[("p", 40), ("q", 30)]] + [[("p", 1), ("q", 1)]] * 15 + [[("p", 15)]]
    for step in plan:
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
        close(np.concatenate(got[k]), want[k], dtype, f"replayed request {k}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_contexts(tmp_path, dtype):
    """1,500 tokens: keys a thousand positions back and several splits, a state carried over 1,500 steps; whole, then
    in portions and single tokens, at rows on both sides of every split edge."""
    from mini_llm_b200.config.base import EngineConfig
    from mini_llm_b200.engine.runner import ModelRunner, StepEntry
    cfg = config(72, 131, 1e-5, [
        layer("latent_attention", latent(4, 16, 16, 16, 64, 0.25, scaling=dict(factor=8.0, original=256, fast=32.0, slow=1.0)), None),
        layer("mamba2", mamba(3, 32, 16, 1, 3, 1), moe(4, 2, 32, shared=32)),
        layer("latent_attention", latent(9, 8, 16, 8, 64, 0.3, scaling=dict(factor=8.0, original=256, fast=32.0, slow=1.0), kv_from=0), None)])
    tensors = make_tensors(cfg, 11)
    folder = write_model(str(tmp_path / "long"), cfg, tensors, torch.bfloat16)
    n = 1500
    ids = random_ids(n, cfg["vocab"], 1)
    want = oracle(tensors, cfg, ids, dtype)
    r = ModelRunner(folder, EngineConfig(dtype=dtype, page_size=16, num_pages=200, max_num_seqs=2))
    rows = [0, 1, 255, 256, 257, 511, 512, 1023, 1024, 1279, 1280, 1499]
    r.add_request("w")
    close(r.step([StepEntry("w", ids, rows)]).cpu().numpy(), want[rows], dtype, "whole")
    r.finish_request("w")
    r.add_request("p")
    got, at = [], 0
    cuts = [700, 324, 255, 201] + [1] * 20
    for c in cuts:
        got.append(r.step([StepEntry("p", ids[at:at + c], [c - 1])]).cpu().numpy()[0])
        at += c
    close(np.stack(got), want[np.cumsum(cuts) - 1], dtype, "portions and single tokens")
    assert r.graph_replays >= 15


def test_command_line_with_random_weights(tmp_path):
    """bin/mini_llm: the random-weights mode writes a Falisun folder from a config.json; greedy tokens from the command
    line equal LLM.generate's."""
    import json
    import subprocess
    import sys
    from helpers import ROOT
    from mini_llm_b200 import LLM, SamplingParams
    cfg_path = tmp_path / "cfg.json"
    cfg_path.write_text(json.dumps(CONFIGS["Q"]))
    out_dir = tmp_path / "written"
    cli = [sys.executable, os.path.join(ROOT, "bin", "mini_llm")]
    prompts = ["5 17 3 90 9 100 4", "40 2 2 31"]
    tail = ["--dtype", "float32", "--max-new-tokens", "6", "--ignore-eos", "--max-batch-num", "2"]
    for p in prompts:
        tail += ["--prompt-ids", p]
    r = subprocess.run(cli + ["--random-config", str(cfg_path), "--seed", "7", "--write-model", str(out_dir)] + tail,
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and os.path.isfile(out_dir / "model.safetensors"), r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.endswith("[DONE]")]
    got = [[int(t) for t in l.replace("[DONE]", "").split()] for l in lines]
    llm = LLM(str(out_dir), dtype="float32", max_num_seqs=2)
    want = llm.generate([[int(t) for t in p.split()] for p in prompts], SamplingParams(max_new_tokens=6, ignore_eos=True))
    assert got == want


def test_sizes_that_happen_to_be_one_or_equal(tmp_path):
    """One head, one group, one expert per token out of one group of two, one tap, a latent as wide as the model, value
    heads as wide as key heads: nothing rests on two sizes being different or larger than 1."""
    from mini_llm_b200.config.base import EngineConfig
    from mini_llm_b200.engine.runner import ModelRunner, StepEntry
    cfg = config(32, 40, 1e-5, [
        layer("mamba2", mamba(1, 32, 8, 1, 1, 1), moe(2, 1, 32, groups=(1, 1), shared=32)),
        layer("latent_attention", latent(1, 32, 32, 32, 32, 1.0, dims=32), moe(2, 2, 8, groups=(2, 2))),
        layer("mamba2", mamba(8, 4, 1, 8, 2, 8), None)])
    tensors = make_tensors(cfg, 4)
    folder = write_model(str(tmp_path / "ones"), cfg, tensors, torch.bfloat16)
    ids = random_ids(60, cfg["vocab"], 9)
    for dtype in ("float32", "bfloat16"):
        want = oracle(tensors, cfg, ids, dtype)
        r = ModelRunner(folder, EngineConfig(dtype=dtype, page_size=8, num_pages=20, max_num_seqs=2, use_cuda_graphs=False))
        r.add_request("a")
        rows = [r.step([StepEntry("a", ids[:33], list(range(33)))]).cpu().numpy()]
        for t in range(33, 60):
            rows.append(r.step([StepEntry("a", [ids[t]], [0])]).cpu().numpy())
        close(np.concatenate(rows), want, dtype, "ones")


@pytest.mark.parametrize("kind", ["attention_only", "mamba_only"])
def test_models_of_one_kind_of_layer(tmp_path, kind):
    """Only pages and no state, or only states and no pages: whole, in portions and token by token, two requests."""
    from mini_llm_b200.config.base import EngineConfig
    from mini_llm_b200.engine.runner import ModelRunner, StepEntry
    if kind == "attention_only":
        layers = [layer("latent_attention", latent(2, 8, 8, 8, 16, 0.4, base=50.0), moe(4, 2, 16, shared=8)),
                  layer("latent_attention", latent(3, 16, 8, 8, 16, 0.3, base=50.0, kv_from=0), None),
                  layer("latent_attention", latent(2, 8, 8, 8, 16, 0.4, base=50.0), None)]
    else:
        layers = [layer("mamba2", mamba(2, 16, 16, 1, 4, 1), None), layer("mamba2", mamba(4, 8, 24, 2, 2, 2), moe(4, 2, 16, shared=8))]
    cfg = config(48, 61, 1e-5, layers)
    tensors = make_tensors(cfg, 6)
    folder = write_model(str(tmp_path / kind), cfg, tensors, torch.bfloat16)
    ids = {k: random_ids(n, cfg["vocab"], 30 + n) for k, n in (("a", 70), ("b", 41))}
    want = {k: oracle(tensors, cfg, v, "float32") for k, v in ids.items()}
    r = ModelRunner(folder, EngineConfig(dtype="float32", page_size=8, num_pages=20, max_num_seqs=2))
    assert (len(r.cache.groups) == 0) == (kind == "mamba_only") and (len(r.cache.states) == 0) == (kind == "attention_only")
    for k in ids:
        r.add_request(k)
    got = {k: [] for k in ids}
    out = r.step([StepEntry("a", ids["a"][:50], list(range(50))), StepEntry("b", ids["b"][:3], [0, 1, 2])]).cpu().numpy()
    got["a"].append(out[:50]); got["b"].append(out[50:])
    out = r.step([StepEntry("b", ids["b"][3:40], list(range(37))), StepEntry("a", [ids["a"][50]], [0])]).cpu().numpy()
    got["b"].append(out[:37]); got["a"].append(out[37:])
    for t in range(51, 70):
        entries = [StepEntry("a", [ids["a"][t]], [0])] + ([StepEntry("b", [ids["b"][40]], [0])] if t == 51 else [])
        out = r.step(entries).cpu().numpy()
        got["a"].append(out[:1])
        if t == 51:
            got["b"].append(out[1:])
    for k in ids:
        close(np.concatenate(got[k]), want[k], "float32", f"{kind} {k}")
        r.finish_request(k)
    r.cache.check()


def test_sizes_no_kernel_takes_are_refused_at_construction(tmp_path):
    from mini_llm_b200.config.base import ConfigError, EngineConfig
    from mini_llm_b200.engine.runner import ModelRunner
    cfg = config(64, 50, 1e-5, [layer("mamba2", mamba(2, 16, 512, 1, 4, 1), None)])      # a state of 512 rows per head
    folder = write_model(str(tmp_path / "bad"), cfg, make_tensors(cfg, 0))
    with pytest.raises(ConfigError, match="rows per head"):
        ModelRunner(folder, EngineConfig(dtype="float32", num_pages=4))
