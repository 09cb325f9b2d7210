"""The Vepevik architecture in the engine against the plain implementation (``plain_vepevik``):
every mechanism alone at the kernel level, then whole models of three small configurations
under every way of cutting the work, in float32 and bfloat16, long decoding, and greedy generation
through the scheduler.  Weights and inputs are made so that a fault shows: a key that stands out
just inside and just outside a chunk and at a page's border, a far key under a slow decay, states that
must be zeroed when a slot is used again, caches filled with NaN where nothing was written."""

from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_vepevik as P
import trace_util as T
from vepevik_configs import CONFIGS, PAGE_SIZE, RANKS, attention, config, prompt, random_state

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

LENGTHS = {"A": [3, 19, 64, 90, 41], "B": [1, 2, 37, 70], "C": [50, 5, 33, 81]}
# A router logit this close to the first one left out is a close call (bfloat16 activations move a
# logit by about 0.01): the other expert is as good an answer, and through keys, values and states it
# reaches the tokens behind, so a request is compared up to its first close call.
CLOSE_CALL = {"float32": 1e-3, "bfloat16": 0.05}
MIN_CHECKED = {"float32": 0.5, "bfloat16": 0.15}


def ops():
    from mini_infer_b200.csrc import ops as o
    return o


def requests_for(which):
    return {f"r{i}": prompt(CONFIGS[which], n, salt=i) for i, n in enumerate(LENGTHS[which])}


_plain_cache = {}


def plain_with_margins(state, cfg, toks):
    m = []
    logits = P.vepevik_forward(state, cfg, toks, torch.float64, margins=m).numpy()
    n_moe = sum(1 for l in cfg["layers"] if l.get("mlp") and l["mlp"]["kind"] == "moe")
    margin = np.array(m).reshape(n_moe, len(toks)).min(axis=0) if n_moe else np.full(len(toks), np.inf)
    return logits, margin


def plain_for(which):
    """float64 logits of every request, and per request and position its closest router call."""
    if which not in _plain_cache:
        cfg = CONFIGS[which]
        state = random_state(cfg, seed=11, ranks=RANKS[which])
        logits, margins = {}, {}
        for rid, toks in requests_for(which).items():
            logits[rid], margins[rid] = plain_with_margins(state, cfg, toks)
        _plain_cache[which] = (state, logits, margins)
    return _plain_cache[which]


def make_runner(which, dtype, steps=None, num_blocks=None, max_requests=4, cuda_graph=False):
    from mini_infer_b200.engine import ModelRunner

    state, _, _ = plain_for(which)
    ps = PAGE_SIZE[which]
    if num_blocks is None:
        num_blocks = T.max_tokens_needed(steps) // ps
    runner = ModelRunner.from_state_dict(CONFIGS[which], state, dtype=dtype, block_size=ps, num_blocks=num_blocks,
                                         max_requests=max_requests, cuda_graph=cuda_graph)
    for st in runner.cache.storage:
        st.fill_(float("nan"))            # a slot that was never written must never be read
    for arena in runner.cache.state_arenas.values():
        arena.fill_(float("nan"))         # a state must be zeroed when its slot is handed out
    return runner


def compare(which, dtype, got):
    _, want, margins = plain_for(which)
    scale = max(float(np.abs(w).max()) for w in want.values())
    tol = T.tolerance(dtype, scale)
    checked = total = over = 0
    for rid, w in want.items():
        assert got[rid].shape == w.shape
        close = margins[rid] < CLOSE_CALL[dtype]
        keep = np.arange(int(np.nonzero(close)[0][0]) if close.any() else len(w))
        total += len(w)
        checked += len(keep)
        assert np.isfinite(got[rid]).all(), f"{rid}: non-finite logits"
        if dtype == "bfloat16":
            # A head's output is divided by its root mean square: where a head of a few channels nearly
            # cancels, bfloat16 rounding of q, k and v moves the row by several percent (float32 shows that
            # the arithmetic is right).  Such rows are few and stay within a few bounds; a wrong key, page
            # or state moves most rows by tens of percent.
            err = np.abs(got[rid][keep] - w[keep]).max(axis=1)
            over += int((err > float(tol)).sum())
            assert (err <= 4 * float(tol)).all(), f"{which} {rid}: position {keep[int(err.argmax())]} differs " \
                                                  f"by {err.max():.3g} (bound {float(tol):.3g})"
            continue
        bad = T.first_bad(got[rid][keep], w[keep], tol)
        assert bad is None, f"{which} {dtype} {rid}: position {keep[bad]} differs by " \
                            f"{np.abs(got[rid][keep[bad]] - w[keep[bad]]).max():.3g} (bound {float(tol):.3g})"
    assert over <= max(2, 0.03 * checked), f"{over} of {checked} rows are over the bound"
    assert checked >= MIN_CHECKED[dtype] * total, f"only {checked} of {total} rows were compared"


CUTTINGS = {"whole": T.cut_whole, "last_decoded": T.cut_last_decoded, "portions": T.cut_portions,
            "mixed": T.cut_mixed}


@pytest.mark.parametrize("cutting", list(CUTTINGS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["A", "B", "C"])
def test_engine_matches_plain_under_every_cutting(which, dtype, cutting):
    """Whole prompts, prefill then token-by-token decoding, portions down to two tokens, and mixed
    batches of unequal requests in which slots and pages are freed and used again."""
    requests = requests_for(which)
    steps = CUTTINGS[cutting](requests)
    runner = make_runner(which, dtype, steps)
    got = T.collect(steps, T.replay_in_process(runner, steps), CONFIGS[which]["vocab"])
    runner.cache.check()
    assert runner.cache.num_requests == 0
    for gi, pool in enumerate(runner.cache.pools):
        assert runner.cache.num_free_pages(gi) == pool.num_pages
    compare(which, dtype, got)


@pytest.mark.parametrize("which", ["A", "B", "C"])
def test_float32_logits_do_not_depend_on_the_cutting(which):
    """In float32 every sum runs in an order that depends on the position alone: the logits of a
    position are the same bits whole, in portions, decoded, or beside other requests."""
    requests = requests_for(which)
    results = {}
    for name, cut in CUTTINGS.items():
        steps = cut(requests)
        runner = make_runner(which, "float32", steps)
        results[name] = T.collect(steps, T.replay_in_process(runner, steps), CONFIGS[which]["vocab"])
    for name in ("last_decoded", "portions", "mixed"):
        for rid in requests:
            assert np.array_equal(results[name][rid], results["whole"][rid]), f"{which} {name} {rid}"


@pytest.mark.parametrize("which,n_pages", [("A", 6), ("C", 12)])
def test_long_decoding_over_chunk_edges_and_captured_steps(which, n_pages):
    """One short prompt, then 180 tokens one by one (chunks end under decoded tokens, their pages come
    back to a pool that is far smaller than the sequence), kernel by kernel and as captured graphs."""
    from mini_infer_b200.engine import StepEntry

    cfg = CONFIGS[which]
    state, _, _ = plain_for(which)
    toks = prompt(cfg, 186, salt=77)
    want, margin = plain_with_margins(state, cfg, toks)
    close = np.nonzero(margin < CLOSE_CALL["float32"])[0]
    upto = int(close[0]) if close.size else len(toks)
    assert upto > 100
    tol = T.tolerance("float32", float(np.abs(want).max()))
    results = []
    for graph in (False, True):
        # config A: chunks of 7 and 20 positions in pages of 8; C: a group without chunks keeps all 186 tokens
        runner = make_runner(which, "float32", num_blocks=n_pages, cuda_graph=graph)
        runner.add_request("a")
        rows = [runner.step([StepEntry("a", toks[:6], list(range(6)))]).logits.cpu().numpy()]
        for t in toks[6:]:
            rows.append(runner.step([StepEntry("a", [t], [0])]).logits.cpu().numpy())
        got = np.concatenate(rows)
        assert T.first_bad(got[:upto], want[:upto], tol) is None
        runner.free_request("a")
        runner.cache.check()
        results.append(got)
    assert np.array_equal(results[0], results[1])        # a captured step computes what the step itself does


def test_greedy_generation_through_the_scheduler():
    """Greedy tokens from the engine's own entry point (scheduler, sampler, cache) equal the plain
    implementation's, fed its own tokens, for several prompts generated together."""
    from mini_infer_b200.engine import ContinuousScheduler, Request
    from mini_infer_b200.sampling import SamplingParams

    which = "A"
    cfg = CONFIGS[which]
    state, _, _ = plain_for(which)
    prompts = [prompt(cfg, n, salt=200 + i) for i, n in enumerate([4, 21, 9])]
    n_new = 12
    runner = make_runner(which, "float32", num_blocks=32)
    sched = ContinuousScheduler(runner, max_concurrent=3, max_tokens_per_step=16)
    results = sched.generate([Request(prompt=p, sampling_params=SamplingParams(), max_tokens=n_new) for p in prompts])
    sched.stop()
    for p, r in zip(prompts, results):
        assert len(r.tokens) == n_new
        seq = list(p)
        for tok in r.tokens:
            logits = P.vepevik_forward(state, cfg, seq, torch.float64)[-1]
            top2 = torch.topk(logits, 2).values
            if float(top2[0] - top2[1]) > 1e-3:     # the plain choice is not a close call
                assert tok == int(logits.argmax()), f"after {len(seq)} tokens"
            seq.append(tok)
    runner.cache.check()
    assert runner.cache.num_requests == 0


def test_generation_from_a_model_folder(tmp_path):
    """A folder with config.json and model.safetensors through ``generate_ids``, the call behind the command line."""
    import json

    from mini_infer_b200.engine.api import generate_ids
    from mini_infer_b200.weights.safetensors_io import write_safetensors

    cfg = CONFIGS["B"]
    state = random_state(cfg, seed=11, ranks=RANKS["B"])
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    write_safetensors(str(tmp_path / "model.safetensors"), state)
    p = prompt(cfg, 11, salt=300)
    got = generate_ids(str(tmp_path), [p], max_tokens=5, dtype="float32", device=DEV)[0]
    seq = list(p)
    for tok in got:
        logits = P.vepevik_forward(state, cfg, seq, torch.float64)[-1]
        top2 = torch.topk(logits, 2).values
        if float(top2[0] - top2[1]) > 1e-3:
            assert tok == int(logits.argmax())
        seq.append(tok)


# ----------------------------------------------------------------------------- mechanisms alone


def rnd(*shape, seed, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def ctx_for(q_lens, slots):
    """The part of a step context the state kernels read."""
    starts = np.concatenate([[0], np.cumsum(q_lens)[:-1]]).astype(np.int32)
    i32 = lambda a: torch.tensor(np.asarray(a, dtype=np.int32), device=DEV)
    return SimpleNamespace(q_start=i32(starts), q_len=i32(q_lens), state_slot=i32(slots), n_requests=len(q_lens),
                           n_tokens=int(sum(q_lens)), decode_only=all(n == 1 for n in q_lens),
                           host_q_len=list(q_lens))


@pytest.mark.parametrize("d,dv,rot,norm", [(24, 16, 8, True), (10, 14, 10, True), (64, 64, 64, False), (7, 3, 2, True),
                                           (128, 48, 32, True), (20, 28, 0, True)])
def test_head_norm_half_rotation_and_value_blend(d, dv, rot, norm):
    """RMS norm over the head with a gain shared by the heads, then the rotation of pairs (i, i + rot/2)
    on the first ``rot`` dimensions, then a factor; values blended with another layer's; all in place,
    against the plain functions, at positions from 0 to a million."""
    M, nq, nkv = 9, 4, 2
    width = nq * d + nkv * d + nkv * dv + 5          # some columns behind, which must stay untouched
    packed = rnd(M, width, seed=8)
    pos = [0, 1, 2, 3, 100, 101, 4095, 1000000, 8]
    base, eps, lam = 300.0, 1e-5, 0.3
    qg, kg = rnd(d, seed=9) + 1, rnd(d, seed=10) + 1
    other = rnd(M, nkv * dv, seed=11)
    freq = (base ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)) if rot else None
    dev = packed.to(DEV).clone()
    ops().qk_norm_rope_store(dev, 0, nq * d, (nq + nkv) * d, nq, nkv, d, dv,
                             q_gain=qg.to(DEV) if norm else None, k_gain=kg.to(DEV) if norm else None, eps=eps,
                             rot=rot, positions=torch.tensor(pos, dtype=torch.int32, device=DEV),
                             freq=freq.to(DEV) if rot else None, q_scale=0.5, k_scale=2.0, v_other=other.to(DEV),
                             blend=torch.tensor([lam], device=DEV))
    got = dev.cpu().double()
    x = packed.double()
    for off, n, gain, factor in ((0, nq, qg, 0.5), (nq * d, nkv, kg, 2.0)):
        heads = x[:, off:off + n * d].reshape(M, n, d)
        if norm:
            heads = P.rms_norm(heads, gain.double(), eps)
        if rot:
            heads = P.rotate_half_layout(heads, pos, base, rot)
        want = heads.reshape(M, n * d) * factor
        assert (got[:, off:off + n * d] - want).abs().max() <= 3e-6 * max(1.0, want.abs().max())
    v0 = (nq + nkv) * d
    want_v = (1 - lam) * x[:, v0:v0 + nkv * dv] + lam * other.double()
    assert (got[:, v0:v0 + nkv * dv] - want_v).abs().max() <= 1e-6
    assert torch.equal(got[:, v0 + nkv * dv:], x[:, v0 + nkv * dv:])     # the columns behind are not touched


@pytest.mark.parametrize("heads,dk,dv,dtype,portions", [
    (2, 12, 36, torch.float32, (1, 17, 2, 1, 1, 20, 3)), (1, 64, 32, torch.float32, (1, 17, 2, 1, 1, 20, 3)),
    (3, 9, 5, torch.float32, (2, 1, 40, 1)),
    (2, 24, 40, torch.bfloat16, (300, 1, 140, 129)), (1, 128, 64, torch.bfloat16, (513,)),   # chunks side by side
    (2, 16, 8, torch.float32, (700, 1, 1, 2))])
def test_retention_state_and_a_far_key(heads, dk, dv, dtype, portions):
    """The matrix state under one fixed decay per head through portions and decoded tokens against the
    plain token loop.  The first head decays slowly and its third key is a hundred times the others: what
    the last tokens read is that key's value, hundreds of tokens back."""
    Tn = sum(portions)
    decay = [0.9995, 0.6, 0.97][:heads]
    stride = heads * (2 * dk + dv) + 3
    stride += (-stride) % 8
    packed = rnd(Tn, stride, seed=50).to(dtype)
    packed[-1, :dk] = packed[2, heads * dk:heads * dk + dk]      # the last query points along the third key
    packed[2, heads * dk:heads * dk + dk] *= 100.0
    q, k = packed[:, :heads * dk], packed[:, heads * dk:2 * heads * dk]
    v = packed[:, 2 * heads * dk:2 * heads * dk + heads * dv]
    S = torch.zeros(heads, dk, dv, dtype=torch.float64)
    want = torch.empty(Tn, heads, dv, dtype=torch.float64)
    dec = torch.tensor(decay, dtype=torch.float32).double()      # the kernel holds the decays in fp32
    for t in range(Tn):
        kt, vt = k[t].double().reshape(heads, dk), v[t].double().reshape(heads, dv)
        S = dec[:, None, None] * S + kt[:, :, None] * vt[:, None, :]
        want[t] = torch.einsum("hkv,hk->hv", S, q[t].double().reshape(heads, dk) * dk ** -0.5)
    far = (want[-1, 0] - dec[0] ** (Tn - 3) * (k[2, :dk].double() @ q[-1, :dk].double()) * dk ** -0.5 * v[2, :dv].double())
    assert far.abs().max() < 0.2 * want[-1, 0].abs().max()       # the far key is most of what the last token reads
    state = torch.full((3, heads, dk, dv), float("nan"), device=DEV)
    state[1].zero_()
    dev = packed.to(DEV)
    got, t0 = [], 0
    for n in portions:
        sl = dev[t0:t0 + n]
        o = ops().gla_scan(sl[:, :heads * dk], sl[:, heads * dk:2 * heads * dk],
                           sl[:, 2 * heads * dk:2 * heads * dk + heads * dv], None, None, 1.0, dk ** -0.5, heads, dk,
                           dv, state, ctx_for([n], [1]), head_decay=torch.tensor(decay, device=DEV))
        got.append(o.cpu().double())
        t0 += n
    got = torch.cat(got).reshape(Tn, heads, dv)
    assert (got - want).abs().max() <= 3e-5 * max(1.0, want.abs().max())
    assert (state[1].cpu().double() - S).abs().max() <= 3e-5 * max(1.0, S.abs().max())
    assert torch.isnan(state[0]).all() and torch.isnan(state[2]).all()
    gate = rnd(Tn, heads * dv, seed=54)
    out = torch.empty(Tn, heads * dv, device=DEV)
    ops().headnorm_gate(got.reshape(Tn, heads * dv).float().to(DEV), torch.ones(dv, device=DEV), gate.to(DEV), out,
                        heads, dv, 1e-5, "silu", 1.0)
    ref = P.rms_unit(got, 1e-5).reshape(Tn, heads * dv) * P.silu(gate.double())
    assert (out.cpu().double() - ref).abs().max() <= 1e-5 * max(1.0, ref.abs().max())


@pytest.mark.parametrize("heads,dk,dv,rot,portions", [(2, 24, 40, 8, (1, 150, 1, 2)), (3, 16, 8, 16, (40, 1, 1)),
                                                     (1, 72, 33, 36, (3, 300))])
def test_rotated_queries_and_keys_enter_the_recurrence_unrounded(heads, dk, dv, rot, portions):
    """From bfloat16 projections the rotation leaves q and k in fp32 rows of their own (the packed
    columns stay as they were) and the scan reads them beside bfloat16 values: against the plain
    rotation and token loop in float64 the output is as close as fp32 arithmetic gets, which a second
    rounding of q and k to bfloat16 would miss by a hundred times."""
    Tn, base = sum(portions), 700.0
    decay = [0.99, 0.8, 0.95][:heads]
    hk, hv = heads * dk, heads * dv
    stride = 2 * hk + hv + 6
    stride += (-stride) % 8
    packed = rnd(Tn, stride, seed=60).to(torch.bfloat16)
    pos = list(range(5000, 5000 + Tn))
    x = packed.double()
    q = P.rotate_half_layout(x[:, :hk].reshape(Tn, heads, dk), pos, base, rot)
    k = P.rotate_half_layout(x[:, hk:2 * hk].reshape(Tn, heads, dk), pos, base, rot)
    v = x[:, 2 * hk:2 * hk + hv].reshape(Tn, heads, dv)
    dec = torch.tensor(decay, dtype=torch.float32).double()
    S = torch.zeros(heads, dk, dv, dtype=torch.float64)
    want = torch.empty(Tn, heads, dv, dtype=torch.float64)
    for t in range(Tn):
        S = dec[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        want[t] = torch.einsum("hkv,hk->hv", S, q[t] * dk ** -0.5)
    dev = packed.to(DEV)
    qk = torch.full((Tn, 2 * hk), float("nan"), device=DEV)
    freq = base ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)
    ops().qk_norm_rope_store(dev, 0, hk, None, heads, heads, dk, dv, rot=rot,
                             positions=torch.tensor(pos, dtype=torch.int32, device=DEV), freq=freq.to(DEV), qk_out=qk)
    assert torch.equal(dev.cpu(), packed)                      # nothing is written back
    assert (qk[:, :hk].cpu().double().reshape(Tn, heads, dk) - q).abs().max() <= 3e-6 * q.abs().max()
    assert (qk[:, hk:].cpu().double().reshape(Tn, heads, dk) - k).abs().max() <= 3e-6 * k.abs().max()
    state = torch.zeros(2, heads, dk, dv, device=DEV)
    got, t0 = [], 0
    for n in portions:
        o = ops().gla_scan(qk[t0:t0 + n, :hk], qk[t0:t0 + n, hk:], dev[t0:t0 + n, 2 * hk:2 * hk + hv], None, None, 1.0,
                           dk ** -0.5, heads, dk, dv, state, ctx_for([n], [1]),
                           head_decay=torch.tensor(decay, device=DEV))
        got.append(o.cpu().double())
        t0 += n
    got = torch.cat(got).reshape(Tn, heads, dv)
    assert (got - want).abs().max() <= 3e-5 * max(1.0, want.abs().max())
    assert (state[1].cpu().double() - S).abs().max() <= 3e-5 * max(1.0, S.abs().max())


DELTA_SHORT = ({0: 23, 1: 9}, [(1, 2), (2, 1), (7, 0), (1, 1), (3, 5), (9, 0)])
DELTA_LONG = ({0: 200, 1: 37}, [(130, 30), (1, 0), (69, 7)])


@pytest.mark.parametrize("heads,kvh,dk,dv,taps,dtype,bound,plan", [
    (4, 2, 12, 20, 3, torch.float32, 2e-5, DELTA_SHORT), (2, 2, 32, 8, 2, torch.float32, 2e-5, DELTA_SHORT),
    (3, 1, 7, 5, 1, torch.float32, 2e-5, DELTA_SHORT), (2, 2, 24, 36, 5, torch.float32, 2e-5, DELTA_LONG),
    (6, 3, 64, 48, 4, torch.bfloat16, 3e-2, DELTA_LONG), (2, 1, 128, 40, 4, torch.bfloat16, 3e-2, DELTA_SHORT),
    (1, 1, 200, 33, 2, torch.float32, 2e-5, DELTA_SHORT)])
def test_delta_rule_carries_state_and_convolution_tail(heads, kvh, dk, dv, taps, dtype, bound, plan):
    """Convolution tail and matrix state through portions of 1, 2 and more tokens, two requests in one
    launch in slots that lie apart, against the plain mixer over the whole sequence."""
    Hd, ra, rg = 16, 3, 2
    total, cuts = plan
    gk, hk, hv = kvh * dk, heads * dk, heads * dv
    C = 2 * gk + hv
    W = {"q": rnd(gk, Hd, seed=20, scale=0.4), "k": rnd(gk, Hd, seed=21, scale=0.4), "v": rnd(hv, Hd, seed=22, scale=0.4),
         "q.conv": rnd(gk, taps, seed=23, scale=0.6), "k.conv": rnd(gk, taps, seed=24, scale=0.6),
         "v.conv": rnd(hv, taps, seed=25, scale=0.6), "b": rnd(heads, Hd, seed=26, scale=0.5),
         "A_log": rnd(heads, seed=27) - 0.5, "norm": rnd(dv, seed=28, scale=0.1) + 1, "a1": rnd(ra, Hd, seed=29),
         "a2": rnd(hk, ra, seed=30), "dt_bias": rnd(hk, seed=31, scale=1.5) - 1.0, "g1": rnd(rg, Hd, seed=32),
         "g2": rnd(hv, rg, seed=33), "o": torch.eye(hv)}
    W = {n: w.to(dtype).float() for n, w in W.items()}
    m = {"heads": heads, "kv_heads": kvh, "dim": dk, "vdim": dv, "conv": taps}
    hs = {r: rnd(n, Hd, seed=40 + r).to(dtype).float() for r, n in total.items()}
    W64 = {n: w.double() for n, w in W.items()}
    want = {r: P.channel_delta(hs[r].double(), W64, m, 1e-5) for r in total}
    s_off = (taps - 1) * C
    state = torch.full((4, s_off + heads * dk * dv), float("nan"), device=DEV)
    slots = {0: 3, 1: 1}
    for s in slots.values():
        state[s].zero_()
    f32 = lambda t: t.float().to(DEV).contiguous()
    w_in = torch.cat([W[n] for n in ("q", "k", "v", "b", "a1", "g1")]).double()
    conv_w = f32(torch.cat([W["q.conv"], W["k.conv"], W["v.conv"]]))
    done = {0: 0, 1: 0}
    got = {r: [] for r in total}
    for n0, n1 in cuts:
        lens = [n for n in (n0, n1) if n]
        who = [r for r, n in ((0, n0), (1, n1)) if n]
        h = torch.cat([hs[r][done[r]:done[r] + n] for r, n in zip(who, lens)])
        proj = (h.double() @ w_in.T).to(dtype).to(DEV)
        ctx = ctx_for(lens, [slots[r] for r in who])
        x = proj[:, :C]
        u = torch.empty((h.shape[0], C), dtype=dtype, device=DEV)
        ops().causal_conv(x, None, conv_w, None, state, ctx, u, act="silu")
        a = proj[:, C + heads:C + heads + ra].double()
        z = (a @ W["a2"].double().T.to(DEV)).float().contiguous()
        gate = (proj[:, C + heads + ra:].double() @ W["g2"].double().T.to(DEV)).to(dtype).contiguous()
        o = ops().delta_scan(u[:, :gk], u[:, gk:2 * gk], u[:, 2 * gk:], z, f32(W["dt_bias"]), f32(W["A_log"]),
                             proj[:, C:C + heads], dk ** -0.5, 1e-6, heads, kvh, dk, dv, state, s_off, ctx,
                             conv_in=x, taps=taps)
        out = torch.empty((h.shape[0], hv), dtype=dtype, device=DEV)
        ops().headnorm_gate(o, f32(W["norm"]), gate, out, heads, dv, 1e-5, "sigmoid", 1.0)
        row = 0
        for r, n in zip(who, lens):
            got[r].append(out[row:row + n].cpu().double())
            row += n
            done[r] += n
    for r in total:
        assert done[r] == total[r]
        g = torch.cat(got[r])
        assert (g - want[r]).abs().max() <= bound * max(1.0, want[r].abs().max()), f"request {r}"
    assert torch.isnan(state[0]).all() and torch.isnan(state[2]).all()      # other slots are never touched


@pytest.mark.parametrize("E,top,ff,H,M,groups,scale", [
    (6, 2, 20, 40, 33, (3, 2), 1.5), (10, 2, 24, 48, 70, (5, 1), 2.5), (5, 1, 12, 40, 5, None, 2.0),
    (4, 4, 16, 36, 9, None, 1.0), (8, 3, 8, 40, 200, (4, 2), 0.7), (3, 2, 10, 36, 7, (3, 3), 1.0),
    (64, 4, 16, 64, 50, (8, 3), 1.0), (12, 6, 72, 64, 130, (2, 1), 1.0)])
@pytest.mark.parametrize("dtype,bound", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_grouped_router_and_gated_experts(E, top, ff, H, M, groups, scale, dtype, bound):
    """The router's choice within the best groups, the weights as shares of the softmax over all experts
    times a factor, and the weighted sum of ``down(silu(gate x) * up x)``, against the plain token loop."""
    x = rnd(M, H, seed=60).to(dtype)
    W = {"router": rnd(E, H, seed=61, scale=0.5).to(dtype)}
    for e in range(E):
        W[f"e{e}.gate"] = rnd(ff, H, seed=100 + e, scale=0.4).to(dtype)
        W[f"e{e}.up"] = rnd(ff, H, seed=200 + e, scale=0.4).to(dtype)
        W[f"e{e}.down"] = rnd(H, ff, seed=300 + e, scale=0.2).to(dtype)
    router = {"experts": E, "top": top, "scale": scale}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    mlp = {"kind": "moe", "router": router, "expert": {"ff": ff}}
    margins = []
    W64 = {k: v.double() for k, v in W.items()}
    want = P.moe(x.double(), W64, mlp, margins)
    ok = torch.tensor(margins) > 1e-4
    assert ok.sum() >= 0.8 * M
    dx = x.to(DEV)
    ids, wts = ops().moe_route(dx, W["router"].to(DEV), top, all_scores=True, groups=groups[0] if groups else 0,
                               keep_groups=groups[1] if groups else 0, scale=scale)
    z = x.double() @ W64["router"].T
    for t in range(M):
        if not ok[t]:
            continue
        idx, w, _, _ = P.route(z[t], router)
        assert ids[t].cpu().tolist() == idx, f"token {t}"
        assert (wts[t].cpu().double() - w).abs().max() < 1e-5 * scale
    gate_up = torch.stack([torch.cat([W[f"e{e}.gate"], W[f"e{e}.up"]]) for e in range(E)]).to(DEV).contiguous()
    down = torch.stack([W[f"e{e}.down"] for e in range(E)]).to(DEV).contiguous()
    out = ops().moe_experts(dx, ids, wts, gate_up, down, float("inf"), 1.0, None, up_offset=0.0)
    assert (out.cpu().double() - want)[ok].abs().max() <= bound * max(1.0, want.abs().max())


@pytest.mark.parametrize("dtype,bound", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_clamped_dense_unit_normalised_embedding_and_gates_per_head(dtype, bound):
    M, H, I = 11, 40, 24
    x = rnd(M, H, seed=70).to(dtype)
    W = {"gate": rnd(I, H, seed=71, scale=0.4).to(dtype), "up": rnd(I, H, seed=72, scale=0.4).to(dtype),
         "down": rnd(H, I, seed=73, scale=0.2).to(dtype)}
    limit = 0.9                                               # both clamps bite: |gate x| and |up x| reach 2 and more
    gu = (x.double() @ torch.cat([W["gate"], W["up"]]).double().T)
    assert (gu.abs() > limit).float().mean() > 0.2
    act = ops().clamped_glu(gu.to(dtype).to(DEV), limit, 1.702, 1.0)
    g = torch.clamp(gu[:, :I].to(dtype).double(), max=limit)
    u = torch.clamp(gu[:, I:].to(dtype).double(), min=-limit, max=limit)
    want = g * torch.sigmoid(1.702 * g) * (u + 1.0)
    assert (act.cpu().double() - want).abs().max() <= bound * max(1.0, want.abs().max())
    if dtype == torch.float32:
        full = P.dense_ff(x.double(), {k: v.double() for k, v in W.items()}, limit)
        assert (act.cpu().double() @ W["down"].double().T - full).abs().max() <= 1e-4
    # the embedding with a norm of its own starts the fp32 stream
    table, gain = rnd(17, H, seed=74).to(dtype), rnd(H, seed=75, scale=0.2) + 1
    ids = torch.tensor([3, 0, 16, 3, 9], dtype=torch.int32)
    got = ops().embedding_rmsnorm(table.to(DEV), ids.to(DEV), gain.to(DEV), 1e-5)
    assert got.dtype == torch.float32
    ref = P.rms_norm(table.double()[ids.long()], gain.double(), 1e-5)
    assert (got.cpu().double() - ref).abs().max() <= 2e-6 * ref.abs().max()
    # one gate per head
    heads, dv = 3, 5
    o, gate = rnd(M, heads * dv, seed=76).to(dtype), rnd(M, heads, seed=77).to(dtype)
    out = torch.empty(M, heads * dv, dtype=dtype, device=DEV)
    ops().gate_mul(o.to(DEV), gate.to(DEV), out, "sigmoid", 1.0, per=dv)
    ref = (o.double().reshape(M, heads, dv) * torch.sigmoid(gate.double())[:, :, None]).reshape(M, heads * dv)
    assert (out.cpu().double() - ref).abs().max() <= bound / 4 * max(1.0, ref.abs().max())


def chunk_runner(chunk, n_tokens, page, dtype="float32", sizes=(2, 1, 16, 12)):
    """A runner of one attention layer (``sizes``: query heads, key heads, key size, value size) whose planner,
    pages and choice of kernel the kernel-level test borrows."""
    from mini_infer_b200.engine import ModelRunner

    cfg = config([attention(*sizes, chunk, None, 64.0, False, None)], vocab=8, width=16, eps=1e-6)
    runner = ModelRunner.from_state_dict(cfg, random_state(cfg, seed=3), dtype=dtype, block_size=page,
                                         num_blocks=-(-n_tokens // page) + 1, max_requests=2)
    for st in runner.cache.storage:
        st.fill_(float("nan"))
    return runner


# keys and values of two sizes (the kernel for rows of two sizes, or CUDA cores); of one size: in bfloat16 the
# tensor-core kernels (mma.sync for 32-wide heads, tcgen05 for prompt portions of 64- and 128-wide heads, the balanced
# kernel for single tokens), with and without shared key heads
@pytest.mark.parametrize("sizes", [(2, 1, 16, 12), (2, 2, 32, 32), (4, 2, 64, 64), (8, 1, 128, 128)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_chunk_edges_page_borders_and_far_keys(dtype, sizes):
    """One key is made to stand out (it points where the queries point, all others across): a query in its
    chunk and behind it returns its value, a query of the next chunk or before it does not.  The key sits at a
    chunk's first and last position, at a page's last and first slot, and hundreds of tokens back with no
    chunks at all; the tokens come as one prompt, in portions cut inside chunks, and one by one."""
    from mini_infer_b200.engine import StepEntry

    nq, nkv, d, dv = sizes
    td = torch.float32 if dtype == "float32" else torch.bfloat16

    def run(chunk, n_tokens, marked, page, portions):
        runner = chunk_runner(chunk, n_tokens, page, dtype, sizes)
        mixer = runner.model.blocks[0].mixer
        assert (mixer.chunk, mixer.scale) == (chunk, 64.0)
        runner.add_request("a")
        packed = torch.zeros(n_tokens, (nq + nkv) * d + nkv * dv)
        packed[:, 0:nq * d:d] = 1.0                          # queries: e0
        for kh in range(nkv):
            packed[:, (nq + kh) * d + 1] = 1.0               # keys: e1 ...
            packed[marked, (nq + kh) * d + 1] = 0.0
            packed[marked, (nq + kh) * d] = 1.0              # ... the marked key: e0
        packed[:, (nq + nkv) * d:] = 1.0                     # values: ones, the marked value: tens
        packed[marked, (nq + nkv) * d:] = 10.0
        outs, t0 = [], 0
        for n in portions:
            ctx, caches, _, _ = runner.stepper.plan([StepEntry("a", [0] * n, [])])
            runner.stepper.apply_table_updates(ctx)
            cache = caches[0]
            dev = packed[t0:t0 + n].to(td).to(DEV)
            ops().qk_norm_rope_store(dev, 0, nq * d, (nq + nkv) * d, nq, nkv, d, dv,
                                     slots=ctx.groups[cache.group].slots, kcache=cache.k, vcache=cache.v)
            out = torch.empty(n, nq * dv, dtype=td, device=DEV)
            mixer._attend(dev[:, :nq * d], out, cache, ctx)
            outs.append(out.float().cpu())
            t0 += n
        assert t0 == n_tokens
        return torch.cat(outs)

    # the marked key's score is 64 above the others: its weight is 1 to fp32 precision
    def cuttings(n):
        yield [n]
        yield [1] * n
        sizes, rest = [], n
        for s in (5, 2, 13, 1, 3, 29, 2, 17, 7) * 10:
            if rest <= 0:
                break
            sizes.append(min(s, rest))
            rest -= sizes[-1]
        yield sizes

    for chunk, page, marked in ((11, 8, 15), (11, 8, 11), (11, 8, 21), (16, 16, 31), (16, 16, 32), (6, 4, 13),
                                (1, 4, 5), (40, 8, 0), (40, 16, 39)):
        for portions in cuttings(70):
            out = run(chunk, 70, marked, page, portions)
            for i in range(70):
                sees = i >= marked and i // chunk == marked // chunk
                assert torch.allclose(out[i], torch.full_like(out[i], 10.0 if sees else 1.0), atol=1e-3), \
                    (chunk, page, marked, i, portions[:4])
    for portions in ([700], [690] + [1] * 10):               # no chunks: a key 696 tokens back
        out = run(None, 700, 3, 16, portions)
        assert torch.allclose(out[3:], torch.full_like(out[3:], 10.0), atol=1e-3)
        assert torch.allclose(out[:3], torch.full_like(out[:3], 1.0), atol=1e-3)


def test_first_tokens_of_a_sequence_and_slots_used_again():
    """A request's first tokens (alone, as a pair, as a longer prompt) start from zero state and empty
    convolution tails whatever the slot held before: the same prompt gives the same logits in a fresh
    runner and in slots that other requests have just left."""
    from mini_infer_b200.engine import StepEntry

    which = "C"
    cfg = CONFIGS[which]
    toks = prompt(cfg, 40, salt=5)
    other = prompt(cfg, 55, salt=6)
    fresh = make_runner(which, "float32", num_blocks=16)
    fresh.add_request("x")
    want = fresh.step([StepEntry("x", toks, list(range(len(toks))))]).logits.cpu().numpy()
    state, _, _ = plain_for(which)
    plain, margin = plain_with_margins(state, cfg, toks)
    upto = int(np.nonzero(margin < CLOSE_CALL["float32"])[0][0]) if (margin < CLOSE_CALL["float32"]).any() else 40
    assert upto >= 3
    assert T.first_bad(want[:upto], plain[:upto], T.tolerance("float32", float(np.abs(plain).max()))) is None
    runner = make_runner(which, "float32", num_blocks=16, max_requests=2)
    for first in (1, 2, 17):
        for rid in ("p", "q"):                               # fill both slots and leave them
            runner.add_request(rid)
            runner.step([StepEntry(rid, other, [])])
        runner.free_request("q")
        runner.free_request("p")
        runner.add_request("a")
        rows = [runner.step([StepEntry("a", toks[:first], list(range(first)))]).logits.cpu().numpy(),
                runner.step([StepEntry("a", toks[first:], list(range(len(toks) - first)))]).logits.cpu().numpy()]
        runner.free_request("a")
        assert np.array_equal(np.concatenate(rows), want), f"first portion of {first}"
    runner.cache.check()
