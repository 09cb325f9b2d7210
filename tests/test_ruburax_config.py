"""CPU checks of the Ruburax architecture: configuration reader, assembly into parts, tensor names
and shapes against a checkpoint's, which cache layer a layer writes or reads, what the cache manager is
asked to keep, and the plain implementation's own consistency."""

import copy

import pytest
import torch

import plain_ruburax as P
from ruburax_configs import CONFIGS, prompt, random_state

from mini_infer_b200.config import ConfigError, load_config
from mini_infer_b200.parts import DecoderModel, KVNeed, StateNeed
from mini_infer_b200.weights.loader import WeightLoadError, check_names


def build(which):
    arch, cfg = load_config(CONFIGS[which])
    return cfg, DecoderModel(arch.assemble(cfg))


@pytest.mark.parametrize("which", list(CONFIGS))
def test_names_and_shapes_fit_a_checkpoint(which):
    cfg, model = build(which)
    state = random_state(CONFIGS[which], seed=1)
    check_names(model, {n: tuple(t.shape) for n, t in state.items()})
    assert len(model.blocks) == len(cfg.layers)
    assert model.graph_safe()
    broken = {n: tuple(t.shape) for n, t in state.items()}
    broken["embed"] = broken["embed"][::-1]
    del broken["final.norm"]
    broken["surplus"] = (1,)
    with pytest.raises(WeightLoadError) as e:
        check_names(model, broken)
    assert e.value.missing == ["final.norm"] and e.value.unexpected == ["surplus"]
    assert [m[0] for m in e.value.mismatched] == ["embed"]


def test_layers_that_read_another_layers_keys_and_what_the_cache_keeps():
    _, model = build("C")
    # layer 4 reads layer 0's keys and values: five cache layers for six layers
    assert [(e.layer, e.cache, e.writes_cache) for e in model.schedule] == \
        [(0, 0, True), (1, 1, True), (2, 2, True), (3, 3, True), (4, 0, False), (5, 4, True)]
    assert all(e.after is not None for e in model.schedule)      # the per-layer token input stands behind every layer
    reader = model.blocks[4].mixer
    assert not reader.own_kv and set(reader.param_decls()) == {"q", "q.b", "q.norm", "sink", "o"}
    needs = model.cache_needs()
    assert needs[0].kv == KVNeed(3, 12, None, 9, None) and needs[0].state is None
    assert needs[1].kv is None and needs[1].state == StateNeed((5, 30), torch.float32)
    # the parallel layer: pages for its attention; the matrix with its normaliser column and the running maxima
    assert needs[2].kv == KVNeed(1, 20, None, 28, None)
    assert needs[2].state == StateNeed((2 * 7 * (5 + 1) + 2,), torch.float32)
    assert needs[4].kv == KVNeed(3, 32, None, None, None)
    _, model = build("B")
    assert all(e.after is None for e in model.schedule)          # no token_side in the configuration: no such part
    assert "side.embed" not in {e.name for e in model.expected_tensors()}
    assert "l0.norm2" not in {e.name for e in model.expected_tensors()}      # a layer without a feed-forward


def test_the_side_table_is_one_tensor_declared_by_every_layer():
    _, model = build("A")
    names = [e.name for e in model.expected_tensors()]
    assert names.count("side.embed") == 1
    assert model.after[2].col0 == 2 * 6 and model.after[2].table_width == 4 * 6


def test_configurations_that_are_refused():
    base = CONFIGS["A"]
    def broken(change):
        cfg = copy.deepcopy(base)
        change(cfg)
        return cfg
    cases = [
        lambda c: c.pop("residual_mult"),
        lambda c: c.pop("logit_scale"),
        lambda c: c["layers"][1]["mixer"].pop("scale"),
        lambda c: c["layers"][1]["mixer"].update(kv_heads=3),
        lambda c: c["layers"][1]["mixer"]["rot"].update(dims=26),
        lambda c: c["layers"][2]["mixer"].update(kv_from=2),            # itself
        lambda c: c["layers"][2]["mixer"].update(kv_from=0),            # not an attention layer
        lambda c: c["layers"][2]["mixer"].update(vdim=8),               # other sizes than the layer it reads
        lambda c: c["layers"][3]["mixer"]["right"].update(gate_cap=0.0),
        lambda c: c["layers"][1]["mlp"]["router"].update(top=13),
        lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=5),
        lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(keep=1, count=12),
        lambda c: c["layers"][0]["mlp"].update(kind="other"),
        lambda c: c["layers"][0].update(type="window"),
        lambda c: c["layers"][0]["mixer"].update(blocks=5),
        lambda c: c["token_side"].update(dim=0),
    ]
    for change in cases:
        with pytest.raises(ConfigError):
            load_config(broken(change))
    # a reader of a reader is refused as well
    cfg = copy.deepcopy(base)
    cfg["layers"].append(copy.deepcopy(cfg["layers"][2]))
    cfg["layers"][4]["mixer"]["kv_from"] = 2
    with pytest.raises(ConfigError):
        load_config(cfg)


def test_plain_implementation_is_consistent():
    """A prefix's logits do not depend on what follows; the residual factor and the logit factor act where
    they should; a layer that reads another's keys differs from one with keys of its own."""
    cfg = CONFIGS["A"]
    state = random_state(cfg, seed=2)
    toks = prompt(cfg, 20, salt=1)
    full = P.ruburax_logits(state, cfg, toks)
    assert torch.allclose(P.ruburax_logits(state, cfg, toks[:9]), full[:9], atol=1e-9)
    doubled = copy.deepcopy(cfg)
    doubled["logit_scale"] = 2 * cfg["logit_scale"]
    assert torch.allclose(P.ruburax_logits(state, doubled, toks), 2 * full, atol=1e-9)
    streams = []
    P.ruburax_logits(state, cfg, toks, streams=streams)
    assert len(streams) == len(cfg["layers"])
    # the router: an expert outside the kept groups is never chosen, even where its score is the largest
    router = {"experts": 6, "top": 2, "scale": 1.0, "groups": {"count": 3, "keep": 1}}
    z = torch.tensor([5.0, -5.0, 1.0, 1.2, -5.0, -5.0], dtype=torch.float64)
    ids, weights, _ = P.choose_experts(z, torch.zeros(6, dtype=torch.float64), router)
    assert sorted(ids) == [2, 3]                 # the middle group's two best sum highest; expert 0 stays out
    ids, weights, _ = P.choose_experts(z, torch.tensor([0.0, 0.9, 0, 0, 0, 0], dtype=torch.float64), router)
    assert sorted(ids) == [0, 1] and abs(weights[ids.index(1)] - float(torch.sigmoid(z[1]))) < 1e-12   # the weight has no correction
