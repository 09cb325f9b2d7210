"""Small Ruburax configurations and random weights for tests (none of them a real model's sizes).

The configurations differ from one another in every size: heads against key heads (equal, grouped,
one key head), key against value size, sizes that are no multiple of 4 or 16, partial, full and no
rotation, frequency rescales with other bands, attention layers that read an earlier layer's keys and
values (right behind it and across other layers), one to five convolution taps, one block and several,
caps of the gates from 3 to 20, one expert per token and all of them, groups of three and four experts
and none, shared experts and none, layers without a feed-forward, models without a per-layer token
input, residual and logit factors that differ from each other and from 1.
"""

from __future__ import annotations

import torch


def dense(ff):
    return {"kind": "dense", "ff": ff}


def experts(n, top, ff, scale=1.0, groups=None, shared=None):
    router = {"experts": n, "top": top, "scale": scale}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    mlp = {"kind": "moe", "router": router, "expert": {"ff": ff}}
    if shared:
        mlp["shared"] = {"ff": shared}
    return mlp


def rglru(width, blocks, conv, mlp):
    return {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": conv}, "mlp": mlp}


def rot(dims, base, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling:
        r["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return r


def attn(heads, kv_heads, dim, vdim, scale, rotation=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rotation:
        m["rot"] = rotation
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def attention(mixer, mlp):
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def parallel(left, right, scales, mlp):
    heads, dim, vdim, cap = right
    return {"type": "parallel", "mlp": mlp,
            "mixer": {"left": left, "right": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap},
                      "left_scale": scales[0], "right_scale": scales[1]}}


def config(layers, *, vocab, width, eps, mult, logit_scale, side=None):
    cfg = {"architecture": "Ruburax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult,
           "logit_scale": logit_scale, "layers": layers}
    if side:
        cfg["token_side"] = {"dim": side}
    return cfg


CONFIGS = {
    # every mixer; an attention that reads the layer right before it; grouped experts with a shared one
    "A": config([rglru(32, 4, 3, dense(40)),
                 attention(attn(4, 2, 24, 16, 0.3, rot(12, 1000.0, (4.0, 2.0, 6.0, 40))), experts(12, 3, 20, 1.5, (4, 2), 24)),
                 attention(attn(4, 2, 24, 16, 0.3, rot(12, 1000.0, (4.0, 2.0, 6.0, 40)), kv_from=1), experts(6, 2, 16, 2.5)),
                 parallel(attn(6, 3, 16, 8, 0.25, rot(16, 50.0)), (3, 12, 20, 5.0), (0.6, 0.8), experts(9, 4, 12, 0.7, (3, 2), 8))],
                vocab=59, width=48, eps=1e-5, mult=0.7, logit_scale=1.3, side=6),
    # no per-layer token input; a parallel layer first, whose attention's keys and values the last layer reads;
    # layers without a feed-forward; heads that share nothing; no rotation in one attention; factors of 1
    "B": config([parallel(attn(2, 2, 10, 14, 0.4), (1, 32, 8, 20.0), (1.0, 0.5), None),
                 attention(attn(3, 1, 16, 16, 0.25, rot(4, 30.0)), experts(5, 1, 12, 2.0)),
                 rglru(24, 1, 1, experts(8, 8, 8, 1.0, (2, 2), 16)),
                 attention(attn(2, 2, 20, 12, 0.2), None),
                 attention(attn(2, 2, 10, 14, 0.35, kv_from=0), dense(28))],
                vocab=53, width=40, eps=1e-6, mult=1.0, logit_scale=1.0),
    # odd sizes; an attention that reads keys and values across three other layers; five taps; a cap of 3
    "C": config([attention(attn(6, 3, 12, 9, 0.29, rot(12, 300.0, (8.0, 1.0, 4.0, 64))), dense(36)),
                 rglru(30, 5, 5, experts(3, 2, 10, 1.0, (3, 3))),
                 parallel(attn(2, 1, 20, 28, 0.2, rot(10, 7.0, (2.0, 0.5, 3.0, 16))), (2, 7, 5, 3.0), (0.3, 1.2), dense(20)),
                 rglru(12, 2, 2, None),
                 attention(attn(6, 3, 12, 9, 0.31, rot(12, 300.0, (8.0, 1.0, 4.0, 64)), kv_from=0), experts(8, 2, 12, 1.25, (2, 1), 4)),
                 attention(attn(3, 3, 32, 32, 0.18, rot(32, 10000.0)), experts(4, 4, 16))],
                vocab=47, width=36, eps=1e-5, mult=0.4, logit_scale=0.8, side=3),
}

PAGE_SIZE = {"A": 8, "B": 16, "C": 16}


def random_state(cfg: dict, seed: int) -> dict[str, torch.Tensor]:
    """Random weights as a checkpoint would hold them (values that bfloat16 represents exactly, so
    that both engine dtypes and the float64 plain implementation start from the same numbers)."""
    g = torch.Generator().manual_seed(seed)
    H = cfg["width"]
    n_layers = len(cfg["layers"])

    def mat(*shape, std=None):
        std = std if std is not None else shape[-1] ** -0.5
        return (torch.randn(*shape, generator=g) * std).to(torch.bfloat16)

    def vec(n, mean=0.0, std=0.1):
        return (mean + torch.randn(n, generator=g) * std).to(torch.bfloat16)

    def attention_tensors(q, m, biased, sink):
        nq, nkv, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        out = {q + "q": mat(nq * d, H), q + "q.norm": vec(d, 1.0, 0.3), q + "o": mat(H, nq * dv)}
        if m.get("kv_from") is None:
            out.update({q + "k": mat(nkv * d, H), q + "v": mat(nkv * dv, H), q + "k.norm": vec(d, 1.0, 0.3)})
        if biased:
            out[q + "q.b"] = vec(nq * d, 0.0, 0.3)
            if m.get("kv_from") is None:
                out.update({q + "k.b": vec(nkv * d, 0.0, 0.3), q + "v.b": vec(nkv * dv, 0.0, 0.3)})
        if sink:
            out[q + "sink"] = vec(nq, 0.5, 1.0)
        return out

    st = {"embed": mat(cfg["vocab"], H, std=1.0), "final.norm": vec(H, 1.0)}
    side = cfg.get("token_side")
    if side:
        st["side.embed"] = mat(cfg["vocab"], n_layers * side["dim"], std=1.0)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        st[p + "norm1"] = vec(H, 1.0)
        m = layer["mixer"]
        q = p + "mix."
        if layer["type"] == "rglru":
            C, B, taps = m["width"], m["blocks"], m["conv"]
            bw = C // B
            st.update({q + "y": mat(C, H), q + "y.b": vec(C), q + "x": mat(C, H), q + "x.b": vec(C),
                       q + "conv": mat(C, taps, std=0.6), q + "conv.b": vec(C),
                       q + "ra": mat(B, bw, bw), q + "ra.b": vec(B * bw).reshape(B, bw),
                       q + "ri": mat(B, bw, bw), q + "ri.b": vec(B * bw).reshape(B, bw),
                       q + "lam": vec(C, -1.0, 1.5), q + "o": mat(H, C)})
        elif layer["type"] == "attention":
            st.update(attention_tensors(q, m, True, True))
        else:
            st.update(attention_tensors(q + "left.", m["left"], False, False))
            r = m["right"]
            hk, hv, n = r["heads"] * r["dim"], r["heads"] * r["vdim"], r["heads"]
            q = q + "right."
            st.update({q + "q": mat(hk, H), q + "k": mat(hk, H), q + "v": mat(hv, H), q + "g": mat(hv, H),
                       q + "o": mat(H, hv), q + "norm": vec(hv, 1.0, 0.3),
                       q + "i": mat(n, H, std=3.0 * H ** -0.5), q + "i.b": vec(n, 0.0, 1.0),
                       q + "f": mat(n, H, std=3.0 * H ** -0.5), q + "f.b": vec(n, 3.0, 2.0)})
        mlp = layer.get("mlp")
        q = p + "mlp."
        if mlp:
            st[p + "norm2"] = vec(H, 1.0)
        if mlp and mlp["kind"] == "dense":
            st.update({q + "gate": mat(mlp["ff"], H, std=0.3), q + "up": mat(mlp["ff"], H, std=0.3),
                       q + "down": mat(H, mlp["ff"])})
        elif mlp:
            ff, E = mlp["expert"]["ff"], mlp["router"]["experts"]
            st[q + "router"] = mat(E, H, std=4.0 * H ** -0.5)
            st[q + "correction"] = vec(E, 0.0, 0.3)
            for e in range(E):
                st.update({f"{q}e{e}.gate": mat(ff, H, std=0.3), f"{q}e{e}.up": mat(ff, H, std=0.3),
                           f"{q}e{e}.down": mat(H, ff)})
            if mlp.get("shared"):
                sf = mlp["shared"]["ff"]
                st.update({q + "shared.gate": mat(sf, H, std=0.3), q + "shared.up": mat(sf, H, std=0.3),
                           q + "shared.down": mat(H, sf), q + "shared.sg": mat(1, H, std=3.0 * H ** -0.5)})
        if side:
            q = p + "side."
            st.update({q + "gate": mat(side["dim"], H), q + "proj": mat(H, side["dim"]), q + "norm": vec(H, 1.0)})
    return st


def prompt(cfg: dict, n: int, salt: int) -> list[int]:
    g = torch.Generator().manual_seed(4000 + salt)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()
