"""Falisun without a GPU: the configuration reader and its errors, the model description (schedule, cache needs, tensor
names), the random-weights folder, the rotation table, and the plain statement against itself."""
import copy
import json
import math

import pytest
import torch

import plain_falisun as P
from falisun_models import CFG_P, CFG_Q, config, latent, layer, make_tensors, mamba, moe


def _spec(cfg):
    import mini_llm_b200  # noqa: F401
    from mini_llm_b200.config.base import config_from_dict, get_architecture
    c = config_from_dict(cfg)
    return c, get_architecture(c.architecture).build_spec(c)


def test_every_size_is_read_per_layer():
    c, spec = _spec(CFG_P)
    assert c.architecture == "Falisun" and c.vocab == 97 and c.width == 64 and c.norm_eps == 1e-6 and c.max_positions is None
    a, m, b, m2 = (l.mixer for l in c.layers)
    assert (a.heads, a.dim, a.rot_dim, a.vdim, a.kv_rank, a.scale, a.rot_base, a.kv_from) == (3, 16, 8, 24, 40, 0.3, 100.0, None)
    assert a.rot_scaling == dict(factor=4.0, original=32.0, fast=8.0, slow=1.0)
    assert (m.heads, m.vdim, m.state, m.groups, m.conv, m.norm_groups) == (4, 12, 20, 2, 4, 1)
    assert b.kv_from == 0 and b.heads == 5 and (m2.conv, m2.norm_groups) == (2, 2)
    f0, f1, f2, f3 = (l.mlp for l in c.layers)
    assert (f0.experts, f0.top, f0.expert_ff, f0.groups, f0.keep, f0.shared_ff) == (6, 2, 24, 3, 2, 40)
    assert f1 is None and (f2.groups, f2.keep, f2.shared_ff, f2.top) == (1, 1, None, 1) and f3.shared_ff == 8
    assert [(e.layer, e.cache_of) for e in spec.schedule] == [(0, 0), (1, 1), (2, 0), (3, 3)]
    assert spec.layers[1].ff is None and spec.layers[1].ff_join is None and spec.layers[0].ff_join is not None
    assert all(l.arrangement == "sandwich" for l in spec.layers)
    assert spec.positions.kind == "none" and spec.head.kind == "tied" and spec.max_positions is None


def test_cache_needs_and_tensor_names():
    from mini_llm_b200.cache.manager import CacheManager, PagedNeed, StateNeed
    from mini_llm_b200.parts.model import Model
    _, spec = _spec(CFG_Q)
    model = Model(spec)
    needs = model.layer_needs()
    assert needs[0] == StateNeed((6 * 64 * 16 + 2 * 480,), "float32")
    assert needs[1] == PagedNeed(kv_heads=1, head_dim=152, values_in_keys=True) and needs[2] is None
    assert needs[3] == PagedNeed(kv_heads=1, head_dim=32, values_in_keys=True)       # 24 + 4, padded to 16-byte pieces
    cm = CacheManager(needs, page_size=8, num_pages=4, max_num_seqs=2, allocate=False)
    assert len(cm.groups) == 2 and cm.groups[0].bytes_per_token(2) == 152 * 2
    names = {ref.canonical for _, ps in spec.all_part_specs() for ref in ps.weights.values()}
    assert {"embed", "final.norm", "l0.mix.in", "l0.mix.conv.b", "l0.mix.A_log", "l1.mix.dkv.norm", "l1.mix.uk", "l1.ls1",
            "l1.norm1b", "l2.mix.g", "l2.mlp.e4.down", "l2.mlp.router", "l3.mlp.shared.up", "l3.norm2b", "l3.ls2"} <= names
    assert not {"l2.mix.dkv", "l2.mix.dkv.norm", "l1.norm2", "l1.ls2", "head", "pos"} & names
    assert names == set(make_tensors(CFG_Q, 0))


@pytest.mark.parametrize("change,match", [
    (lambda c: c["layers"][0].update(type="attention"), "type must be one of"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "names no other layer"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "keeps no latents"),
    (lambda c: c["layers"][2]["mixer"].update(kv_rank=48), "differs from it"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=6) or c["layers"][0]["mixer"]["rot"].update(dims=7), "must be even"),
    (lambda c: c["layers"][1]["mixer"].update(groups=3), "not a multiple of groups"),
    (lambda c: c["layers"][1]["mixer"].update(norm_groups=5), "norm_groups"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "exceeds"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), "experts in 4 groups"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "kind must be one of"),
    (lambda c: c.pop("norm"), "missing required key 'norm'"),
    (lambda c: c["layers"][3]["mixer"].pop("state"), "state must be an integer"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].update(factor=0), "must be positive"),
])
def test_config_errors(change, match):
    from mini_llm_b200.config.base import ConfigError
    cfg = copy.deepcopy(CFG_P)
    change(cfg)
    with pytest.raises(ConfigError, match=match):
        _spec(cfg)


def test_a_layer_may_not_read_rows_of_a_later_layer():
    from mini_llm_b200.config.base import ConfigError
    cfg = config(32, 20, 1e-5, [layer("latent_attention", latent(1, 8, 8, 8, 16, 0.3, kv_from=1), None),
                                layer("latent_attention", latent(1, 8, 8, 8, 16, 0.3), None)])
    with pytest.raises(ConfigError, match="runs before"):
        _spec(cfg)


def test_random_weights_folder_loads_by_name(tmp_path):
    from mini_llm_b200 import write_random_model
    from mini_llm_b200.weights.safetensors_io import Checkpoint
    out = write_random_model(CFG_P, 5, str(tmp_path / "m"), dtype="bfloat16")
    ck = Checkpoint(out)
    assert set(ck.names()) == set(make_tensors(CFG_P, 0))
    assert tuple(ck.shape("l1.mix.in")) == (2 * 48 + 2 * 2 * 20 + 4, 64) and tuple(ck.shape("l1.mix.conv")) == (48 + 80, 4)
    assert tuple(ck.shape("l2.mix.uk")) == (5 * 8, 40) and tuple(ck.shape("l0.mix.dkv")) == (48, 64)
    with open(tmp_path / "m" / "config.json") as f:
        assert json.load(f)["architecture"] == "Falisun"


def test_rotation_table_against_the_plain_statement():
    from mini_llm_b200.parts.rotary import rotary_table
    for dims, base, sc in ((8, 100.0, dict(factor=4.0, original=32, fast=8.0, slow=1.0)), (32, 10000.0, None),
                           (64, 10000.0, dict(factor=40.0, original=4096, fast=32.0, slow=1.0)), (0, 10.0, None)):
        f, m = rotary_table(dims, base, sc)
        pf, pm = P.rotary_frequencies(dims, base, sc)
        assert len(f) == dims // 2 and m == pytest.approx(pm)
        assert torch.allclose(torch.tensor(f, dtype=torch.float64), pf, rtol=1e-12, atol=0)
    # fast pairs keep their frequency, slow ones are divided by the factor, the factor on cos and sin grows with ln(factor)
    f, m = rotary_table(64, 10000.0, dict(factor=40.0, original=4096, fast=32.0, slow=1.0))
    assert f[0] == 1.0 and f[31] == pytest.approx(10000.0 ** (-62 / 64) / 40.0) and m == pytest.approx(0.1 * math.log(40.0) + 1.0)


def test_plain_statement_against_itself():
    """A prefix's logits do not depend on what follows; the scan equals its closed form for one state row; the router
    keeps to the best groups; a rotation by position p and a rotation by q differ by the angle of p - q."""
    t = make_tensors(CFG_Q, 1)
    ids = torch.randint(0, CFG_Q["vocab"], (40,), generator=torch.Generator().manual_seed(0)).tolist()
    full = P.forward(t, CFG_Q, ids)
    assert torch.allclose(P.forward(t, CFG_Q, ids[:23]), full[:23], rtol=1e-9, atol=1e-9)
    g = torch.Generator().manual_seed(1)
    T, N, Pd = 9, 3, 2
    x, B, C = (torch.randn(T, 1, n, generator=g, dtype=torch.float64) for n in (Pd, N, N))
    dt = torch.rand(T, 1, generator=g, dtype=torch.float64)
    A_log, D = torch.tensor([0.3], dtype=torch.float64), torch.tensor([0.7], dtype=torch.float64)
    y = P.selective_scan(x, B, C, dt, A_log, D, 1)
    a = -math.exp(0.3)
    want = sum(math.exp(a * float(dt[s + 1:, 0].sum())) * float(dt[s, 0]) * float(B[s, 0] @ C[T - 1, 0]) * x[s, 0] for s in range(T))
    assert torch.allclose(y[T - 1, 0], want + 0.7 * x[T - 1, 0], rtol=1e-10)
    h = torch.randn(50, 16, generator=g, dtype=torch.float64)
    s, chosen, w = P.route(h, torch.randn(12, 16, generator=g, dtype=torch.float64), dict(experts=12, top=2, groups=dict(count=3, keep=1)))
    best_group = s.view(50, 3, 4).max(-1).values.argmax(-1)
    assert torch.equal(chosen // 4, best_group[:, None].expand(-1, 2)) and torch.allclose(w.sum(-1), torch.ones(50, dtype=torch.float64))
    u = torch.randn(1, 8, generator=g, dtype=torch.float64)
    r5, r9 = P.rotate(u, torch.tensor([5]), 8, 100.0, None), P.rotate(u, torch.tensor([9]), 8, 100.0, None)
    assert torch.allclose(P.rotate(r5, torch.tensor([4]), 8, 100.0, None), r9, rtol=1e-5, atol=1e-6)     # angles are 32-bit


def test_a_slot_that_is_used_again_is_zero_in_the_state():
    from mini_llm_b200.cache.manager import CacheManager, PagedNeed, StateNeed
    cm = CacheManager({0: StateNeed((7,), "float32"), 1: PagedNeed(1, 16, values_in_keys=True), 2: None}, page_size=4,
                      num_pages=6, max_num_seqs=1, dtype=torch.float32, device="cpu")
    assert cm.groups[0].pool_k.shape == (1, 6, 1, 4, 16) and cm.groups[0].v_pages(0) is None
    cm.admit("a")
    cm.states[0][cm.slot("a")] += 3.0
    assert cm.reserve("a", 9) and cm.num_free_pages(0) == 3
    cm.commit("a", 9)
    cm.release("a")
    cm.admit("b")
    assert cm.slot("b") == 0 and float(cm.states[0][0].abs().sum()) == 0.0 and cm.num_free_pages(0) == 6
    cm.check()
