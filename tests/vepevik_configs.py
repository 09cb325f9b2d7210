"""Small Vepevik configurations and random weights for tests (none of them a real model's sizes).

The configurations differ from one another in every size: heads against key heads, key against
value size, sizes that are no multiple of 4 or 16, partial, full and no rotation, chunks of 1, 7, 16
(a page) and 20 positions and none, one to five convolution taps, decays near 0 and near 1, one
expert per token and all of them, groups of experts and none, layers without a feed-forward, value
blending in all, some and one of a model's attention layers.
"""

from __future__ import annotations

import torch


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def experts(n, top, ff, scale=1.0, groups=None):
    router = {"experts": n, "top": top, "scale": scale}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "router": router, "expert": {"ff": ff}}


def retention(heads, dim, vdim, decay, rot, mlp):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    if rot:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    return {"type": "retention", "mixer": m, "mlp": mlp}


def delta(heads, kv_heads, dim, vdim, conv, mlp):
    return {"type": "channel_delta", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def attention(heads, kv_heads, dim, vdim, chunk, rot, scale, v_mix, mlp):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "v_mix": v_mix}
    if chunk:
        m["mask"] = {"size": chunk}
    if rot:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def config(layers, *, vocab, width, eps):
    return {"architecture": "Vepevik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


CONFIGS = {
    # every mixer once and attention twice; both blend values, with chunks of 7 and of 20 positions
    "A": config([retention(3, 16, 24, (0.9, 0.97, 0.995), (8, 100.0), dense(40, 0.8)),
                 attention(4, 2, 24, 16, 7, (8, 1000.0), 0.3, True, experts(6, 2, 20, 1.5, (3, 2))),
                 delta(4, 2, 12, 20, 3, None),
                 attention(4, 2, 24, 16, 20, (24, 50.0), 0.25, True, experts(4, 4, 16))],
                vocab=59, width=48, eps=1e-5),
    # recurrent layers first; an attention without chunks, rotation or blending; one that is the only blending
    # layer (its blend is never used) and sees its own position only
    "B": config([delta(2, 2, 32, 8, 2, dense(24, 2.0)),
                 attention(2, 2, 10, 14, None, None, 0.4, False, experts(5, 1, 12, 2.0)),
                 retention(1, 64, 32, (0.5,), (64, 10000.0), experts(8, 3, 8, 0.7, (4, 2))),
                 attention(3, 1, 16, 16, 1, (4, 30.0), 0.25, True, None)],
                vocab=53, width=40, eps=1e-6),
    # blending layers with another attention between them; a chunk that is one page; odd sizes; one tap and five
    "C": config([attention(6, 3, 12, 8, 16, (12, 300.0), 0.29, True, dense(36, 1.0)),
                 delta(3, 1, 7, 5, 1, experts(3, 2, 10, 1.0, (3, 3))),
                 attention(2, 1, 20, 28, 5, None, 0.2, False, None),
                 retention(2, 10, 6, (0.999, 0.05), None, experts(2, 1, 32)),
                 attention(3, 3, 32, 8, None, (16, 7.0), 0.18, True, dense(20, 0.5)),
                 delta(2, 2, 24, 36, 5, experts(6, 2, 12, 1.25, (2, 1)))],
                vocab=47, width=36, eps=1e-5),
}

PAGE_SIZE = {"A": 8, "B": 16, "C": 16}
RANKS = {"A": (5, 3), "B": (2, 4), "C": (3, 6)}      # of the decay's and the gate's low-rank products


def random_state(cfg: dict, seed: int, ranks=(4, 4)) -> dict[str, torch.Tensor]:
    """Random weights as a checkpoint would hold them (values that bfloat16 represents exactly, so
    that both engine dtypes and the float64 plain implementation start from the same numbers)."""
    g = torch.Generator().manual_seed(seed)
    H = cfg["width"]

    def mat(*shape, std=None):
        std = std if std is not None else shape[-1] ** -0.5
        return (torch.randn(*shape, generator=g) * std).to(torch.bfloat16)

    def vec(n, mean=0.0, std=0.1):
        return (mean + torch.randn(n, generator=g) * std).to(torch.bfloat16)

    st = {"embed": mat(cfg["vocab"], H, std=1.0), "embed.norm": vec(H, 1.0), "final.norm": vec(H, 1.0)}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        st[p + "norm1"] = vec(H, 1.0)
        if layer.get("mlp") or i % 2 == 0:      # a layer without a feed-forward may carry its second norm or not
            st[p + "norm2"] = vec(H, 1.0)
        m = layer["mixer"]
        q = p + "mix."
        if layer["type"] == "retention":
            hk, hv = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            st.update({q + "q": mat(hk, H), q + "k": mat(hk, H), q + "v": mat(hv, H), q + "g": mat(hv, H),
                       q + "o": mat(H, hv)})
        elif layer["type"] == "channel_delta":
            gk, hk, hv = m["kv_heads"] * m["dim"], m["heads"] * m["dim"], m["heads"] * m["vdim"]
            taps = m["conv"]
            st.update({q + "q": mat(gk, H), q + "q.conv": mat(gk, taps, std=0.6),
                       q + "k": mat(gk, H), q + "k.conv": mat(gk, taps, std=0.6),
                       q + "v": mat(hv, H), q + "v.conv": mat(hv, taps, std=0.6),
                       q + "b": mat(m["heads"], H), q + "A_log": vec(m["heads"], -0.5, 1.0),
                       q + "norm": vec(m["vdim"], 1.0),
                       q + "a1": mat(ranks[0], H), q + "a2": mat(hk, ranks[0], std=1.0),
                       q + "dt_bias": vec(hk, -1.0, 1.5),
                       q + "g1": mat(ranks[1], H), q + "g2": mat(hv, ranks[1], std=1.0), q + "o": mat(H, hv)})
        else:
            nq, nkv, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            st.update({q + "q": mat(nq * d, H), q + "k": mat(nkv * d, H), q + "v": mat(nkv * dv, H),
                       q + "q.norm": vec(d, 1.0, 0.3), q + "k.norm": vec(d, 1.0, 0.3),
                       q + "g": mat(nq, H), q + "o": mat(H, nq * dv)})
            if m.get("v_mix"):
                st[q + "vmix"] = vec(1, 0.4, 0.1).reshape(())
        mlp = layer.get("mlp")
        q = p + "mlp."
        if mlp and mlp["kind"] == "dense":
            st.update({q + "gate": mat(mlp["ff"], H, std=0.3), q + "up": mat(mlp["ff"], H, std=0.3),
                       q + "down": mat(H, mlp["ff"])})
        elif mlp:
            ff = mlp["expert"]["ff"]
            st[q + "router"] = mat(mlp["router"]["experts"], H, std=4.0 * H ** -0.5)
            for e in range(mlp["router"]["experts"]):
                st.update({f"{q}e{e}.gate": mat(ff, H, std=0.3), f"{q}e{e}.up": mat(ff, H, std=0.3),
                           f"{q}e{e}.down": mat(H, ff)})
    return st


def prompt(cfg: dict, n: int, salt: int) -> list[int]:
    g = torch.Generator().manual_seed(3000 + salt)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()
