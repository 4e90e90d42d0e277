"""Finuvik without a GPU: its config.json reader, the model description it builds (layers that share tensors become
runs with caches of their own), the cache manager's handling of what its mixer needs, the random-weights writer,
and the plain oracle's own consistency (a recurrence cut into portions, prefix stability)."""
import copy
import json
import os

import pytest
import torch

import plain_finuvik as P

import mini_llm_b200 as m
from mini_llm_b200.cache.manager import CacheManager, PagedNeed, StateNeed
from mini_llm_b200.config.base import ConfigError, get_architecture
from mini_llm_b200.parts.model import Model


def _layer(weights_of=None, mlp=True, q_temp=True):
    left = dict(heads=4, kv_heads=2, dim=16, vdim=24, scale=0.25)
    if q_temp:
        left["q_temp"] = dict(coef=0.5, every=8)
    e = dict(type="parallel", mixer=dict(left=left, left_scale=0.7, right=dict(heads=2, dim=8, vdim=40), right_scale=1.1),
             mlp=dict(ff=96, kind="dense") if mlp else None)
    if weights_of is not None:
        e["weights_of"] = weights_of
    return e


def _cfg(layers=None):
    return dict(architecture="Finuvik", width=64, vocab=97, max_positions=160, norm=dict(eps=1e-6),
                layers=layers if layers is not None else [_layer(), _layer(weights_of=0), _layer(mlp=False, q_temp=False)])


def test_config_reads_every_size_and_constant():
    cfg = m.config_from_dict(_cfg())
    assert cfg.architecture == "Finuvik" and (cfg.width, cfg.vocab, cfg.max_positions, cfg.norm_eps) == (64, 97, 160, 1e-6)
    a, b, c = cfg.layers
    assert (a.left.heads, a.left.kv_heads, a.left.dim, a.left.vdim, a.left.scale) == (4, 2, 16, 24, 0.25)
    assert (a.left.q_temp_coef, a.left.q_temp_every) == (0.5, 8) and (c.left.q_temp_coef, c.left.q_temp_every) == (0.0, 1)
    assert (a.right.heads, a.right.dim, a.right.vdim) == (2, 8, 40) and (a.left_scale, a.right_scale, a.ff) == (0.7, 1.1, 96)
    assert b.weights_of == 0 and cfg.weight_layer(1) == 0 and c.ff is None
    assert m.config_from_dict(cfg.to_dict()).layers == cfg.layers
    # the list form of the architecture key works too
    d = _cfg()
    d["architectures"] = [d.pop("architecture")]
    assert m.config_from_dict(d).architecture == "Finuvik"


@pytest.mark.parametrize("edit,match", [
    (lambda d: d.pop("vocab"), "vocab"),
    (lambda d: d["norm"].pop("eps"), "eps"),
    (lambda d: d["layers"][0].update(type="serial"), "type"),
    (lambda d: d["layers"][0]["mixer"]["left"].update(kv_heads=3), "multiple"),
    (lambda d: d["layers"][0]["mlp"].update(kind="routed"), "kind"),
    (lambda d: d["layers"][1].update(weights_of=7), "weights_of"),
    (lambda d: d["layers"][1].update(weights_of=1), "weights_of"),
    (lambda d: d["layers"][1]["mixer"]["right"].update(vdim=48), "differs"),
    (lambda d: d["layers"][0]["mixer"]["left"]["q_temp"].update(every=0), "every"),
    (lambda d: d.update(layers=[]), "layers"),
])
def test_config_faults_are_named(edit, match):
    d = copy.deepcopy(_cfg())
    edit(d)
    with pytest.raises(ConfigError, match=match):
        m.config_from_dict(d)


def test_description_turns_shared_tensors_into_runs_with_private_caches():
    cfg = m.config_from_dict(_cfg([_layer(weights_of=2), _layer(mlp=False), _layer(), _layer(weights_of=0)]))
    spec = get_architecture("Finuvik").build_spec(cfg)
    assert len(spec.layers) == 2                                   # config layers 1 and 2 carry tensors
    assert [(e.layer, e.private_cache) for e in spec.schedule] == [(1, True), (0, False), (1, False), (1, True)]
    assert len({e.cache_unit for e in spec.schedule}) == 4
    assert spec.layers[0].ff is None and spec.layers[0].ff_norm is None and spec.layers[1].ff is not None
    names = {ref.canonical for _, ps in spec.all_part_specs() for ref in ps.weights.values()}
    assert "l1.mix.left.q" in names and "l2.mlp.gate" in names and "l1.norm2" not in names and "l0.norm1" not in names
    model = Model(spec)
    needs = model.layer_needs()
    assert len(needs) == 4
    for need in needs.values():
        assert need == [PagedNeed(kv_heads=2, head_dim=16, v_head_dim=24), StateNeed((2, 8, 40), "float32")]
    cm = CacheManager(needs, page_size=4, num_pages=6, max_num_seqs=2, dtype=torch.float32, device="cpu")
    assert len(cm.groups) == 1 and len(cm.states) == 4
    g = cm.groups[0]
    assert g.pool is None and g.pool_k.shape == (4, 6, 2, 4, 16) and g.pool_v.shape == (4, 6, 2, 4, 24)
    assert g.bytes_per_token(2) == 4 * 2 * (16 + 24) * 2
    caches = [model.layer_cache(cm, e) for e in spec.schedule]
    assert all(c.write and c.group == 0 and c.state is not None for c in caches)
    assert len({c.k_pages.data_ptr() for c in caches}) == 4 and len({c.state.data_ptr() for c in caches}) == 4
    # a slot handed out again is zero in every run's state
    cm.admit("a")
    for t in cm.states.values():
        t[cm.slot("a")].fill_(3.0)
    cm.release("a")
    cm.admit("b")
    assert all(float(t[cm.slot("b")].abs().sum()) == 0.0 for t in cm.states.values())


def test_cache_manager_refuses_two_needs_of_one_kind():
    with pytest.raises(TypeError):
        CacheManager({0: [PagedNeed(1, 8), PagedNeed(1, 16)]}, page_size=4, num_pages=2, max_num_seqs=1, allocate=False)


def test_random_weights_folder_has_the_designs_tensor_names(tmp_path):
    folder = m.write_random_model(_cfg(), 5, str(tmp_path / "f"), dtype="bfloat16")
    from safetensors import safe_open
    with safe_open(os.path.join(folder, "model.safetensors"), "pt") as f:
        names = set(f.keys())
        assert f.get_tensor("l0.mix.left.o").shape == (64, 4 * 24) and f.get_tensor("l0.mix.right.f.b").shape == (16,)
        assert f.get_tensor("l0.mix.right.norm").shape == (40,) and f.get_tensor("l2.mix.left.r1").shape == (4,)
    assert {"embed", "pos", "final.norm", "head", "l0.norm1", "l0.norm2", "l0.mlp.down", "l2.norm1"} <= names
    assert not any(n.startswith("l1.") for n in names) and "l2.norm2" not in names and "l2.mlp.up" not in names
    assert json.load(open(os.path.join(folder, "config.json")))["architecture"] == "Finuvik"


# ------------------------------------------------------------------------------------------------ the oracle itself
def test_oracle_recurrence_in_portions_equals_the_whole():
    g = torch.Generator().manual_seed(0)
    q, f, v = torch.randn(30, 2, 5, generator=g).double(), torch.rand(30, 2, 5, generator=g).double(), torch.randn(30, 2, 7, generator=g).double()
    o, S = P.gated_recurrence(q, f, v)
    o1, S1 = P.gated_recurrence(q[:11], f[:11], v[:11])
    o2, S2 = P.gated_recurrence(q[11:], f[11:], v[11:], S1)
    assert torch.allclose(torch.cat([o1, o2]), o, atol=1e-12) and torch.allclose(S2, S, atol=1e-12)
    # closed form of one row: S_t[i] = sum_s (prod_{s<r<=t} f_r[i]) (1 - f_s[i]) v_s
    t, i = 9, 3
    want = sum(torch.prod(f[s + 1:t + 1, 0, i]) * (1 - f[s, 0, i]) * v[s, 0] for s in range(t + 1))
    _, St = P.gated_recurrence(q[:t + 1], f[:t + 1], v[:t + 1])
    assert torch.allclose(St[0, i], want, atol=1e-12)


def test_oracle_logits_of_a_prefix_do_not_depend_on_what_follows():
    from test_finuvik_gpu import CFG_X, make_tensors
    t = make_tensors(CFG_X, 1)
    ids = list(range(3, 40))
    a = P.forward(t, CFG_X, ids)
    b = P.forward(t, CFG_X, ids[:20])
    assert torch.allclose(a[:20], b, atol=1e-10)
    assert P.query_temperature(torch.tensor([0, 6, 7, 15, 16]), 0.5, 8).tolist() == pytest.approx(
        [1.0, 1.0, 1 + 0.5 * 0.6931471805599453, 1 + 0.5 * 1.0986122886681098, 1 + 0.5 * 1.0986122886681098])
    assert P.distance_bias(2, 3, 1, torch.tensor([2.0]).double(), torch.tensor([0.5]).double())[0].flatten().tolist() == pytest.approx(
        [2 * 0.4054651081081644, 0.0, 0.0, 2 * 0.6931471805599453, 2 * 0.4054651081081644, 0.0])
