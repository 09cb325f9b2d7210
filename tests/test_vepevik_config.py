"""CPU checks of the Vepevik architecture: configuration reader, assembly into parts, tensor names
and shapes against a checkpoint's, what the cache manager is asked to keep (pages that a chunk
leaves behind come back), and the plain implementation's own consistency."""

import copy

import pytest
import torch

import plain_vepevik as P
from vepevik_configs import CONFIGS, RANKS, prompt, random_state

from mini_infer_b200.cache.manager import CacheManager
from mini_infer_b200.config import ConfigError, load_config
from mini_infer_b200.parts import DecoderModel, KVNeed, StateNeed
from mini_infer_b200.weights.loader import WeightLoadError, check_names


def build(which):
    arch, cfg = load_config(CONFIGS[which])
    return cfg, DecoderModel(arch.assemble(cfg))


@pytest.mark.parametrize("which", list(CONFIGS))
def test_names_and_shapes_fit_a_checkpoint(which):
    cfg, model = build(which)
    state = random_state(CONFIGS[which], seed=1, ranks=RANKS[which])
    check_names(model, {n: tuple(t.shape) for n, t in state.items()})
    assert len(model.blocks) == len(cfg.layers)
    assert model.graph_safe()
    # the ranks of the low-rank products are the checkpoint's: any rank fits, another shape does not
    other = random_state(CONFIGS[which], seed=1, ranks=(RANKS[which][0] + 2, RANKS[which][1] + 1))
    check_names(model, {n: tuple(t.shape) for n, t in other.items()})
    # the first blending layer's factor is never used: a checkpoint may carry it or not; the others' are needed
    blending = [f"l{i}.mix.vmix" for i, l in enumerate(CONFIGS[which]["layers"]) if l["mixer"].get("v_mix")]
    if blending:
        check_names(model, {n: tuple(t.shape) for n, t in state.items() if n != blending[0]})
    for name in blending[1:]:
        with pytest.raises(Exception, match="missing"):
            check_names(model, {n: tuple(t.shape) for n, t in state.items() if n != name})
    broken = {n: tuple(t.shape) for n, t in state.items()}
    broken["embed"] = broken["embed"][::-1]
    del broken["final.norm"]
    broken["surplus"] = (1,)
    with pytest.raises(WeightLoadError) as e:
        check_names(model, broken)
    assert e.value.missing == ["final.norm"] and e.value.unexpected == ["surplus"]
    assert [m[0] for m in e.value.mismatched] == ["embed"]


def test_what_the_cache_keeps():
    _, model = build("A")
    needs = model.cache_needs()
    assert needs[0].kv is None and needs[0].state == StateNeed((3, 16, 24), torch.float32)
    assert needs[1].kv == KVNeed(2, 24, None, 16, 7) and needs[1].state is None
    # convolution tail of two inputs over q, k, v channels, then the matrix states
    assert needs[2].kv is None and needs[2].state == StateNeed((2 * (2 * 2 * 12 + 4 * 20) + 4 * 12 * 20,), torch.float32)
    assert needs[3].kv == KVNeed(2, 24, None, 16, 20)
    cm = CacheManager(needs, page_size=8, num_pages=4, max_requests=2)
    assert [(g.head_dim, g.value_dim, g.chunk) for g in cm.groups] == [(24, 16, 7), (24, 16, 20)]
    _, model = build("B")          # no chunks, and a chunk of one position
    cm = CacheManager(model.cache_needs(), page_size=16, num_pages=4, max_requests=2)
    assert [(g.head_dim, g.value_dim, g.chunk) for g in cm.groups] == [(10, 14, None), (16, None, 1)]


def test_chunked_groups_give_pages_back_as_chunks_end():
    _, model = build("A")
    cm = CacheManager(model.cache_needs(), page_size=8, num_pages=5, max_requests=2)   # chunks of 7 and 20
    cm.add_request("a")
    cm.plan_append([("a", 30)])
    for _ in range(300):           # far more tokens than the pool has slots
        cm.plan_append([("a", 1)])
        cm.check()
    # never more than a chunk's pages and the page of the next position are held
    assert cm.num_free_pages(0) >= 5 - 2 and cm.num_free_pages(1) >= 5 - 4
    cm.free_request("a")
    assert [cm.num_free_pages(g) for g in range(2)] == [5, 5]


@pytest.mark.parametrize("edit,words", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c["layers"][0].update(type="other"), "none of"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.5]), "one decay per head"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "cannot share"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(keep=1, count=6), "fewer than top"),
    (lambda c: c["layers"][2]["mixer"].pop("conv"), "conv"),
    (lambda c: c["layers"][0]["mlp"].update(kind="other"), "neither"),
])
def test_configurations_that_are_refused(edit, words):
    raw = copy.deepcopy(CONFIGS["A"])
    edit(raw)
    with pytest.raises(ConfigError, match=words):
        load_config(raw)


def test_plain_implementation_is_causal_and_a_chunk_is_a_chunk():
    cfg = CONFIGS["A"]
    state = random_state(cfg, seed=5, ranks=RANKS["A"])
    toks = prompt(cfg, 30, salt=9)
    full = P.vepevik_forward(state, cfg, toks)
    assert torch.allclose(P.vepevik_forward(state, cfg, toks[:13]), full[:13], atol=1e-12)
    # the attention alone: a change reaches the positions behind it in its own chunk and no other
    m = cfg["layers"][1]["mixer"]
    W = P.sub({k: v.double() for k, v in state.items()}, "l1.mix.")
    h = torch.randn(25, cfg["width"], dtype=torch.float64, generator=torch.Generator().manual_seed(2))
    a, _ = P.chunked_attention(h, W, list(range(25)), m, 1e-5, None, True)
    h2 = h.clone()
    h2[9] += 1.0
    b, _ = P.chunked_attention(h2, W, list(range(25)), m, 1e-5, None, True)
    changed = (a - b).abs().max(dim=1).values > 1e-9
    size = m["mask"]["size"]                                  # 7: position 9 lies in the chunk 7..13
    assert changed[9:2 * size].all() and not changed[2 * size:].any() and not changed[:9].any()


def test_plain_router_keeps_to_the_best_groups():
    router = {"experts": 6, "top": 2, "scale": 1.5, "groups": {"count": 3, "keep": 1}}
    z = torch.tensor([2.0, -1.0, 1.9, 1.8, 0.0, 0.1], dtype=torch.float64)    # groups (0,1) (2,3) (4,5)
    idx, w, _, _ = P.route(z, router)
    assert idx == [0, 1]                                      # the best group alone, although 2 and 3 score higher than 1
    s = torch.softmax(z, dim=0)
    assert torch.allclose(w, s[[0, 1]] / s[[0, 1]].sum() * 1.5)
    router["groups"]["keep"] = 2
    assert P.route(z, router)[0] == [0, 2]
    router.pop("groups")
    router["top"] = 3
    assert P.route(z, router)[0] == [0, 2, 3]


def test_plain_recurrences_against_their_closed_forms():
    """Retention as an explicit sum over the past, and the delta rule's state after one token."""
    H, T = 20, 9
    g = torch.Generator().manual_seed(4)
    h = torch.randn(T, H, dtype=torch.float64, generator=g)
    m = {"heads": 2, "dim": 6, "vdim": 4, "decay": [0.8, 0.3]}
    W = {n: torch.randn(r, H, dtype=torch.float64, generator=g) for n, r in (("q", 12), ("k", 12), ("v", 8), ("g", 8))}
    W["o"] = torch.eye(8, dtype=torch.float64)
    got = P.retention(h, W, list(range(T)), m, 1e-6)
    q, k, v = (h @ W[n].T for n in "qkv")
    o = torch.zeros(T, 2, 4, dtype=torch.float64)
    for t in range(T):
        for j in range(t + 1):
            for hd in range(2):
                s = (q[t, hd * 6:hd * 6 + 6] @ k[j, hd * 6:hd * 6 + 6]) * 6 ** -0.5 * m["decay"][hd] ** (t - j)
                o[t, hd] += s * v[j, hd * 4:hd * 4 + 4]
    want = P.rms_unit(o, 1e-6).reshape(T, 8) * P.silu(h @ W["g"].T)
    assert torch.allclose(got, want, atol=1e-10)
