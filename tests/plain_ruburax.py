"""A plain, slow implementation of the Ruburax decoder, for tests only.

Whole sequences from position 0, no cache, no batching, token-by-token loops where the
mathematics is a recurrence, one function per mechanism, sharing no code with the package under
test.  Everything runs on the CPU in the dtype of the tensors it is given (tests use float64).

Notation: ``h [T, width]`` is a mixer's or feed-forward's input; a stored ``[out, in]`` matrix
``W`` applied to rows is written ``h @ W.T``.  ``cfg`` is the raw configuration mapping, ``W`` the
tensors of one part under their local names.
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


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.logaddexp(z, torch.zeros_like(z))


def log_sigmoid(z: torch.Tensor) -> torch.Tensor:
    return -softplus(-z)


def rotation_frequencies(rot: dict) -> list[float]:
    """``base^(-2i/dims)`` for ``i < dims/2``; with ``scaling`` the long waves are slowed down: a wave
    shorter than ``original/high`` keeps its frequency, one longer than ``original/low`` gets
    ``f / factor``, and between the two the frequency is the blend ``(1 - s) f / factor + s f`` with
    ``s = (original / wavelength - low) / (high - low)``."""
    dims, base = int(rot["dims"]), float(rot["base"])
    freqs = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return freqs
    factor, low, high, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
    out = []
    for f in freqs:
        wave = 2.0 * math.pi / f
        if wave < orig / high:
            out.append(f)
        elif wave > orig / low:
            out.append(f / factor)
        else:
            s = (orig / wave - low) / (high - low)
            out.append((1.0 - s) * f / factor + s * f)
    return out


def rotate_half_layout(x: torch.Tensor, positions, rot: dict | None) -> torch.Tensor:
    """``x [T, heads, d]``: of the first ``dims`` dimensions, ``i`` is paired with ``i + dims/2`` and the
    pair ``(u, v)`` turned by the angle ``a = p * f_i`` into ``(u cos a - v sin a, v cos a + u sin a)``;
    the other dimensions pass."""
    if not rot or not rot.get("dims"):
        return x
    out = x.clone()
    p = torch.as_tensor(positions, dtype=x.dtype)
    half = int(rot["dims"]) // 2
    for i, f in enumerate(rotation_frequencies(rot)):
        ang = p * f
        c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
        u, v = x[..., i], x[..., i + half]
        out[..., i] = u * c - v * s
        out[..., i + half] = v * c + u * s
    return out


def short_conv(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Per channel ``out[t, c] = b[c] + sum_j w[c, j] x[t - (taps - 1 - j), c]`` with zeros before the
    start: the last column of ``w`` meets the current token."""
    T, C = x.shape
    taps = w.shape[1]
    out = torch.zeros_like(x) + b
    for t in range(T):
        for j in range(taps):
            src = t - (taps - 1 - j)
            if src >= 0:
                out[t] = out[t] + w[:, j] * x[src]
    return out


# ------------------------------------------------------------------------------- mixers


def attention_keys_values(h: torch.Tensor, W: dict, positions, m: dict, eps: float, biased: bool):
    """The keys (normed, then rotated) and values a layer keeps: ``k [T, G, dim]``, ``v [T, G, vdim]``."""
    T = h.shape[0]
    G, d, dv = m["kv_heads"], m["dim"], m["vdim"]
    k, v = h @ W["k"].T, h @ W["v"].T
    if biased:
        k, v = k + W["k.b"], v + W["v.b"]
    k = rms_norm(k.reshape(T, G, d), W["k.norm"], eps)
    return rotate_half_layout(k, positions, m.get("rot")), v.reshape(T, G, dv)


def softmax_attention(h: torch.Tensor, W: dict, positions, m: dict, eps: float, *, biased: bool, sink: bool,
                      keys_values=None):
    """Causal attention of ``heads`` query heads over ``kv_heads`` key/value heads (query head ``a`` reads
    key/value head ``a // (heads / kv_heads)``); queries and keys get an RMS norm over the head with a gain
    shared by the heads, then the rotation; the score is ``q . k * scale``.  With ``sink`` the softmax's
    denominator also holds ``exp(sink_a)``, a term with nothing behind it: it only takes weight away.  ``keys_values``: another
    layer's ``(k, v)`` in the place of this layer's own.  Returns ``(output, (k, v))``."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = h @ W["q"].T
    if biased:
        q = q + W["q.b"]
    q = rotate_half_layout(rms_norm(q.reshape(T, H, d), W["q.norm"], eps), positions, m.get("rot"))
    if keys_values is None:
        keys_values = attention_keys_values(h, W, positions, m, eps, biased)
    k, v = keys_values
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for a in range(H):
        g = a // (H // G)
        for t in range(T):
            s = (k[: t + 1, g] @ q[t, a]) * float(m["scale"])
            if sink:
                s = torch.cat([s, W["sink"][a].reshape(1).to(s.dtype)])
            p = torch.softmax(s, dim=0)
            out[t, a] = p[: t + 1] @ v[: t + 1, g]
    return out.reshape(T, H * dv) @ W["o"].T, keys_values


def matrix_memory(h: torch.Tensor, W: dict, m: dict, eps: float) -> torch.Tensor:
    """Per head a matrix ``S [dim, vdim]``, a vector ``n [dim]`` and a running maximum ``mx`` (all from 0):
    with the capped log gates ``i = cap tanh((W_i h + b_i) / cap)`` and ``f = logsigmoid(cap tanh((W_f h
    + b_f) / cap))``, ``mx' = max(f + mx, i)``, ``S' = exp(f + mx - mx') S + exp(i - mx') k v^T``, ``n'``
    likewise with ``k``, and ``o = S'^T q / (max(|n' . q|, exp(-mx')) + 1e-6)`` with ``q`` times ``dim^-1/2``.
    Each head's ``o`` is brought to unit RMS; the heads times a gain, times ``sigmoid(W_g h)``, projected."""
    T = h.shape[0]
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = (h @ W["q"].T).reshape(T, H, d) * d ** -0.5
    k = (h @ W["k"].T).reshape(T, H, d)
    v = (h @ W["v"].T).reshape(T, H, dv)
    gi = cap * torch.tanh((h @ W["i"].T + W["i.b"]) / cap)
    gf = log_sigmoid(cap * torch.tanh((h @ W["f"].T + W["f.b"]) / cap))
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for a in range(H):
        S = torch.zeros(d, dv, dtype=h.dtype)
        n = torch.zeros(d, dtype=h.dtype)
        mx = torch.zeros((), dtype=h.dtype)
        for t in range(T):
            new = torch.maximum(gf[t, a] + mx, gi[t, a])
            keep, take = torch.exp(gf[t, a] + mx - new), torch.exp(gi[t, a] - new)
            S = keep * S + take * torch.outer(k[t, a], v[t, a])
            n = keep * n + take * k[t, a]
            mx = new
            den = torch.maximum(torch.abs(n @ q[t, a]), torch.exp(-mx)) + 1e-6
            o[t, a] = (S.T @ q[t, a]) / den
    o = rms_unit(o, eps).reshape(T, H * dv) * W["norm"]
    return (o * torch.sigmoid(h @ W["g"].T)) @ W["o"].T


def recurrent_unit(h: torch.Tensor, W: dict, m: dict) -> torch.Tensor:
    """Two branches: ``y = gelu_tanh(W_y h + b)`` and ``u = conv(W_x h + b)``; ``u`` cut into ``blocks`` parts
    with gates ``r = sigmoid(A_r u + b_r)`` and ``i = sigmoid(A_i u + b_i)`` per part; ``a = exp(-8 r
    softplus(lam))``, ``S_t = a S_(t-1) + sqrt(1 - a^2) i u`` from ``S = 0``; output ``W_o (S y)``."""
    T = h.shape[0]
    C, B = m["width"], m["blocks"]
    y = gelu_tanh(h @ W["y"].T + W["y.b"])
    u = short_conv(h @ W["x"].T + W["x.b"], W["conv"], W["conv.b"])
    ub = u.reshape(T, B, C // B)
    r = torch.sigmoid(torch.einsum("boi,tbi->tbo", W["ra"], ub) + W["ra.b"]).reshape(T, C)
    i = torch.sigmoid(torch.einsum("boi,tbi->tbo", W["ri"], ub) + W["ri.b"]).reshape(T, C)
    a = torch.exp(-8.0 * r * softplus(W["lam"]))
    S = torch.zeros(C, dtype=h.dtype)
    out = torch.zeros(T, C, dtype=h.dtype)
    for t in range(T):
        S = a[t] * S + torch.sqrt(1.0 - a[t] * a[t]) * i[t] * u[t]
        out[t] = S
    return (out * y) @ W["o"].T


# ------------------------------------------------------------------------------- feed-forwards


def gated_unit(h: torch.Tensor, W: dict, prefix: str = "") -> torch.Tensor:
    return (silu(h @ W[prefix + "gate"].T) * (h @ W[prefix + "up"].T)) @ W[prefix + "down"].T


def choose_experts(z: torch.Tensor, correction: torch.Tensor, router: dict):
    """One token: scores ``s = sigmoid(z)``, choice scores ``s + correction``.  With groups, a group's score
    is the sum of its two largest choice scores and only experts of the best ``keep`` groups stay in the
    race.  Returns the ``top`` experts by choice score, their weights ``s * scale`` (as they are, whatever they sum to), and
    how close the call was: the smallest gap between something taken and something left (groups, experts)."""
    E, top = int(router["experts"]), int(router["top"])
    s = torch.sigmoid(z)
    choice = s + correction
    allowed = torch.ones(E, dtype=torch.bool)
    margin = math.inf
    groups = router.get("groups")
    if groups and int(groups["count"]) > 1:
        n, keep = int(groups["count"]), int(groups["keep"])
        per = E // n
        score = torch.stack([torch.topk(choice[g * per:(g + 1) * per], min(2, per)).values.sum() for g in range(n)])
        order = torch.sort(score, descending=True).values
        if keep < n:
            margin = float(order[keep - 1] - order[keep])
        kept = torch.topk(score, keep).indices.tolist()
        allowed[:] = False
        for g in kept:
            allowed[g * per:(g + 1) * per] = True
    masked = torch.where(allowed, choice, torch.full_like(choice, -math.inf))
    ids = torch.topk(masked, top).indices
    order = torch.sort(masked, descending=True).values
    if top < E and order[top] > -math.inf:
        margin = min(margin, float(order[top - 1] - order[top]))
    return ids.tolist(), (s[ids] * float(router["scale"])).tolist(), margin


def mixture_of_experts(h: torch.Tensor, W: dict, mlp: dict, margins: list | None = None) -> torch.Tensor:
    """``margins`` (a list) receives, per token, how close the router's call was."""
    T = h.shape[0]
    router = mlp["router"]
    z = h @ W["router"].T
    out = torch.zeros_like(h)
    for t in range(T):
        ids, weights, margin = choose_experts(z[t], W["correction"], router)
        if margins is not None:
            margins.append(margin)
        for e, w in zip(ids, weights):
            out[t] = out[t] + w * gated_unit(h[t:t + 1], W, f"e{e}.")[0]
    if mlp.get("shared"):
        out = out + gated_unit(h, W, "shared.") * torch.sigmoid(h @ W["shared.sg"].T)
    return out


def token_side_input(x: torch.Tensor, W: dict, table: torch.Tensor, tokens, layer: int, dim: int, eps: float):
    """What a layer adds from the token itself, before the residual factor: ``e`` the layer's ``dim`` columns
    of the token's row of the side table, ``g = gelu_tanh(W_gate x) e``, ``y = W_proj g``, then ``y`` at unit
    RMS times a gain."""
    e = table[torch.as_tensor(tokens, dtype=torch.long)][:, layer * dim:(layer + 1) * dim].to(x.dtype)
    y = (gelu_tanh(x @ W["gate"].T) * e) @ W["proj"].T
    return rms_norm(y, W["norm"], eps)


# ------------------------------------------------------------------------------- the model


def part(state: dict, prefix: str) -> dict:
    return {k[len(prefix):]: v for k, v in state.items() if k.startswith(prefix)}


def ruburax_logits(state: dict, cfg: dict, tokens, dtype=torch.float64, streams: list | None = None,
                   margins: list | None = None) -> torch.Tensor:
    """Logits ``[T, vocab]`` of one sequence from position 0.  ``streams`` (a list) receives the residual
    stream after every layer, ``margins`` (a list) the routers' closest calls, layer by layer, token by token."""
    st = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in state.items()}
    eps, mult = float(cfg["norm"]["eps"]), float(cfg["residual_mult"])
    T = len(tokens)
    positions = list(range(T))
    x = st["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    kept: dict[int, tuple] = {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m, W = layer["mixer"], part(st, f"l{i}.mix.")
        if layer["type"] == "rglru":
            mixed = recurrent_unit(x, W, m)
        elif layer["type"] == "attention":
            other = kept[int(m["kv_from"])] if m.get("kv_from") is not None else None
            mixed, kept[i] = softmax_attention(x, W, positions, m, eps, biased=True, sink=True, keys_values=other)
        elif layer["type"] == "parallel":
            left, kept[i] = softmax_attention(x, part(W, "left."), positions, m["left"], eps, biased=False, sink=False)
            right = matrix_memory(x, part(W, "right."), m["right"], eps)
            mixed = float(m["left_scale"]) * left + float(m["right_scale"]) * right
        else:
            raise ValueError(layer["type"])
        x = x + mult * rms_norm(mixed, st[p + "norm1"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            W = part(st, p + "mlp.")
            f = gated_unit(x, W) if mlp["kind"] == "dense" else mixture_of_experts(x, W, mlp, margins)
            x = x + mult * rms_norm(f, st[p + "norm2"], eps)
        side = cfg.get("token_side")
        if side:
            x = x + mult * token_side_input(x, part(st, p + "side."), st["side.embed"], tokens, i, int(side["dim"]), eps)
        if streams is not None:
            streams.append(x.clone())
    z = rms_norm(x, st["final.norm"], eps)
    return (z @ st["embed"].T) * float(cfg["logit_scale"])
