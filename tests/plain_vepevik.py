"""A plain, slow implementation of the Vepevik decoder, for tests only.

Whole sequences from position 0, no cache, no batching, token-by-token loops where the
mathematics is a recurrence, one function per mechanism, sharing no code with the package under
test.  Everything runs on the CPU in the dtype of the tensors it is given (tests use float64).

Notation: ``h [T, width]`` is a mixer's or feed-forward's input; a stored ``[out, in]`` matrix
``W`` applied to rows is written ``h @ W.T``.  ``cfg`` is the raw configuration mapping.
"""

from __future__ import annotations

import math

import torch


# ------------------------------------------------------------------------------- small pieces


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """``x / sqrt(mean(x^2) + eps)`` over the last dimension."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return rms_unit(x, eps) * w


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.logaddexp(z, torch.zeros_like(z))


def rotate_half_layout(x: torch.Tensor, positions, base: float, dims: int) -> torch.Tensor:
    """``x [T, heads, d]``: of the first ``dims`` dimensions, ``i`` is paired with ``i + dims/2`` and
    the pair turned by the angle ``p * base^(-2i/dims)``; the other dimensions pass."""
    out = x.clone()
    p = torch.as_tensor(positions, dtype=x.dtype)
    half = dims // 2
    for i in range(half):
        ang = p * (base ** (-2.0 * i / dims))
        c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
        u, v = x[..., i], x[..., i + half]
        out[..., i] = u * c - v * s
        out[..., i + half] = v * c + u * s
    return out


def short_conv(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """Per channel ``out[t, c] = sum_j w[c, j] x[t - (taps - 1 - j), c]`` with zeros before the start:
    the last column of ``w`` meets the current token."""
    T, C = x.shape
    taps = w.shape[1]
    out = torch.zeros_like(x)
    for t in range(T):
        for j in range(taps):
            src = t - (taps - 1 - j)
            if src >= 0:
                out[t] = out[t] + w[:, j] * x[src]
    return out


# ------------------------------------------------------------------------------- mixers


def retention(h: torch.Tensor, W: dict, positions, m: dict, eps: float) -> torch.Tensor:
    """Linear attention with one fixed decay per head and no normaliser:
    ``S_t = decay S_(t-1) + k_t v_t^T``, ``o_t = S_t^T q_t``; q and k rotated, k scaled by
    ``dim^-1/2`` afterwards; each head's ``o`` brought to unit RMS, the heads gated by
    ``silu(W_g h)`` and projected."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ W["q"].T).reshape(T, H, dk)
    k = (h @ W["k"].T).reshape(T, H, dk)
    v = (h @ W["v"].T).reshape(T, H, dv)
    rot = m.get("rot")
    if rot:
        q = rotate_half_layout(q, positions, rot["base"], rot["dims"])
        k = rotate_half_layout(k, positions, rot["base"], rot["dims"])
    k = k * dk ** -0.5
    decay = torch.tensor(m["decay"], dtype=h.dtype)
    S = torch.zeros(H, dk, dv, dtype=h.dtype)
    o = torch.empty(T, H, dv, dtype=h.dtype)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    o = rms_unit(o, eps).reshape(T, H * dv)
    return (o * silu(h @ W["g"].T)) @ W["o"].T


def channel_delta(h: torch.Tensor, W: dict, m: dict, eps: float) -> torch.Tensor:
    """The gated delta rule with a decay per head and key channel.  q, k (``kv_heads`` heads of
    ``dim``) and v (``heads`` of ``vdim``) each pass a short convolution and SiLU; q and k become
    unit vectors per head (q also times ``dim^-1/2``).  Per head, with its key head's q and k:
    ``S <- g * S`` (rows), ``u = beta (v - S^T k)``, ``S <- S + k u^T``, ``o = S^T q``."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    per = H // G
    q = silu(short_conv(h @ W["q"].T, W["q.conv"])).reshape(T, G, dk)
    k = silu(short_conv(h @ W["k"].T, W["k.conv"])).reshape(T, G, dk)
    v = silu(short_conv(h @ W["v"].T, W["v.conv"])).reshape(T, H, dv)
    q = q / torch.sqrt((q * q).sum(dim=-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(dim=-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ W["b"].T)                                        # [T, H]
    dt = softplus((h @ W["a1"].T) @ W["a2"].T + W["dt_bias"]).reshape(T, H, dk)
    g = torch.exp(-torch.exp(W["A_log"])[None, :, None] * dt)                # [T, H, dk]
    S = torch.zeros(H, dk, dv, dtype=h.dtype)
    o = torch.empty(T, H, dv, dtype=h.dtype)
    for t in range(T):
        for hd in range(H):
            kk, qq = k[t, hd // per], q[t, hd // per]
            Sh = g[t, hd][:, None] * S[hd]
            u = beta[t, hd] * (v[t, hd] - Sh.T @ kk)
            Sh = Sh + kk[:, None] * u[None, :]
            S[hd] = Sh
            o[t, hd] = Sh.T @ qq
    o = rms_unit(o, eps) * W["norm"]
    gate = torch.sigmoid((h @ W["g1"].T) @ W["g2"].T)
    return (o.reshape(T, H * dv) * gate) @ W["o"].T


def chunked_attention(h: torch.Tensor, W: dict, positions, m: dict, eps: float, v_first, is_first_vmix: bool):
    """Softmax attention in which position ``i`` sees ``j <= i`` of its own chunk only
    (``i // size == j // size``; no mask entry: all of the past).  q and k get an RMS norm per head
    with a shared gain, then the rotation; values may be blended with those of the first blending
    layer; every head's output is scaled by ``sigmoid(W_g h)``.  Returns the output and this layer's
    values (what a later layer blends in)."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    per = H // G
    q = rms_norm((h @ W["q"].T).reshape(T, H, dk), W["q.norm"], eps)
    k = rms_norm((h @ W["k"].T).reshape(T, G, dk), W["k.norm"], eps)
    v = (h @ W["v"].T).reshape(T, G, dv)
    rot = m.get("rot")
    if rot:
        q = rotate_half_layout(q, positions, rot["base"], rot["dims"])
        k = rotate_half_layout(k, positions, rot["base"], rot["dims"])
    if m.get("v_mix") and not is_first_vmix:
        lam = W["vmix"]
        v = (1.0 - lam) * v + lam * v_first
    size = (m.get("mask") or {}).get("size")
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for i in range(T):
        lo = (positions[i] // size) * size - positions[0] if size else 0
        lo = max(lo, 0)
        for hd in range(H):
            s = (k[lo:i + 1, hd // per] @ q[i, hd]) * m["scale"]
            out[i, hd] = torch.softmax(s, dim=0) @ v[lo:i + 1, hd // per]
    gate = torch.sigmoid(h @ W["g"].T)                                        # [T, H]
    out = out * gate[:, :, None]
    return out.reshape(T, H * dv) @ W["o"].T, v


# ------------------------------------------------------------------------------- feed-forward


def dense_ff(h: torch.Tensor, W: dict, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ W["gate"].T, max=limit)
    u = torch.clamp(h @ W["up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W["down"].T


def route(z: torch.Tensor, router: dict):
    """From one token's router logits: the chosen experts and their weights.  Scores are the
    softmax over all experts; experts lie in ``groups.count`` equal groups of neighbours, a group
    counts as its best score, only the best ``groups.keep`` groups may give experts; the ``top``
    best of those are chosen and weighted by their scores over the sum of these, times ``scale``.
    Also returns the scores with the experts of other groups struck out, and the kept groups' margin."""
    E, top = router["experts"], router["top"]
    s = torch.softmax(z, dim=0)
    allowed = torch.ones(E, dtype=torch.bool)
    groups = router.get("groups")
    group_margin = float("inf")
    if groups:
        n, keep = groups["count"], groups["keep"]
        best = s.reshape(n, E // n).max(dim=1).values
        kept = torch.topk(best, keep).indices
        if keep < n:
            ordered = torch.sort(best, descending=True).values
            group_margin = float(torch.log(ordered[keep - 1] / ordered[keep]))
        allowed = torch.zeros(n, E // n, dtype=torch.bool)
        allowed[kept] = True
        allowed = allowed.reshape(E)
    masked = torch.where(allowed, s, torch.full_like(s, -1.0))
    idx = torch.topk(masked, top).indices
    w = s[idx]
    w = w / (w.sum() + 1e-20) * router.get("scale", 1.0)
    return idx.tolist(), w, masked, group_margin


def moe(h: torch.Tensor, W: dict, mlp: dict, margins: list | None = None) -> torch.Tensor:
    """Every token through its chosen experts ``W_down (silu(W_gate h) * W_up h)``, weighted.
    ``margins`` collects per token how far the last chosen expert's logit lies above the best one's left out
    (the logarithm of the ratio of their scores; or the last kept group's above the best one's left out, if
    that is closer)."""
    router = mlp["router"]
    z = h @ W["router"].T
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        idx, w, masked, group_margin = route(z[t], router)
        if margins is not None:
            margin = group_margin
            if router["top"] < router["experts"]:
                ordered = torch.sort(masked, descending=True).values
                last, nxt = ordered[router["top"] - 1], ordered[router["top"]]
                if nxt > 0:                                  # (an expert struck out is no rival)
                    margin = min(margin, float(torch.log(last / nxt)))
            margins.append(margin)
        x = h[t:t + 1]
        for wt, e in zip(w, idx):
            y = (silu(x @ W[f"e{e}.gate"].T) * (x @ W[f"e{e}.up"].T)) @ W[f"e{e}.down"].T
            out[t] += wt * y[0]
    return out


# ------------------------------------------------------------------------------- the model


def sub(W: dict, prefix: str) -> dict:
    return {k[len(prefix):]: v for k, v in W.items() if k.startswith(prefix)}


def vepevik_forward(state: dict, cfg: dict, tokens, dtype=torch.float64, return_layers: bool = False,
                    margins: list | None = None):
    """Logits ``[T, vocab]`` of one sequence from position 0 (and, on request, the residual stream
    after every layer)."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in state.items()}
    eps = cfg["norm"]["eps"]
    T = len(tokens)
    positions = list(range(T))
    x = rms_norm(W["embed"][torch.as_tensor(tokens, dtype=torch.long)], W["embed.norm"], eps)
    streams = []
    v_first = None
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        a = rms_norm(x, W[p + "norm1"], eps)
        m = layer["mixer"]
        Wm = sub(W, p + "mix.")
        if layer["type"] == "retention":
            mix = retention(a, Wm, positions, m, eps)
        elif layer["type"] == "channel_delta":
            mix = channel_delta(a, Wm, m, eps)
        elif layer["type"] == "attention":
            first = bool(m.get("v_mix")) and v_first is None
            mix, v = chunked_attention(a, Wm, positions, m, eps, v_first, first)
            if first:
                v_first = v
        else:
            raise ValueError(layer["type"])
        x = x + mix
        mlp = layer.get("mlp")
        if mlp:
            b = rms_norm(x, W[p + "norm2"], eps)
            Wf = sub(W, p + "mlp.")
            if mlp["kind"] == "dense":
                x = x + dense_ff(b, Wf, mlp["limit"])
            elif mlp["kind"] == "moe":
                x = x + moe(b, Wf, mlp, margins)
            else:
                raise ValueError(mlp["kind"])
        streams.append(x)
    logits = rms_norm(x, W["final.norm"], eps) @ W["embed"].T
    if return_layers:
        return logits, torch.stack(streams)
    return logits
