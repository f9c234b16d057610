"""A plain, slow statement of the Tikizen decoder: one function per mechanism, whole sequences at once, on the CPU.

It shares no code with the package: it takes config.json as a dictionary and the tensors by their names, and works in
the dtype it is given (float32, or float64 to bound the float32 one).  A prompt is run whole; there is no cache and
no state that outlives a call, so it cannot have the faults that a cut prompt or a shared batch could bring.

Notation: T tokens, W width, H heads, D key size, E value size, N state size of the state-space mixer.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return rms_unit(x, eps) * w


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


# ---- positions ---------------------------------------------------------------------------------------------------
def rotary_frequencies(rot: dict, dtype) -> (torch.Tensor, float):
    """(frequency of every pair [dims/2], factor on cos and sin).  With ``scaling`` the slow pairs are divided by
    ``factor``, the fast ones stay, the ones between are blended along a ramp over the pair's index."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    mag = 1.0
    sc = rot.get("scaling")
    if sc:
        factor, original = float(sc["factor"]), float(sc["original"])

        def turn_dim(t):
            return dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(base))

        lo = max(math.floor(turn_dim(float(sc["fast"]))), 0)
        hi = min(math.ceil(turn_dim(float(sc["slow"]))), dims - 1)
        ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        f = f / factor * ramp + f * (1.0 - ramp)
        mag = 0.1 * math.log(factor) + 1.0
    return f.to(dtype), mag


def rotate(x: torch.Tensor, positions: torch.Tensor, rot: Optional[dict]) -> torch.Tensor:
    """x [T, H, D]: element i of the first ``dims`` turns with element i + dims/2 by the angle position * f_i."""
    if not rot:
        return x
    dims = int(rot["dims"])
    f, mag = rotary_frequencies(rot, x.dtype)
    a = positions.to(x.dtype)[:, None] * f[None, :]
    c, s = (torch.cos(a) * mag)[:, None, :], (torch.sin(a) * mag)[:, None, :]
    u, v = x[..., :dims // 2], x[..., dims // 2:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


# ---- mixers ------------------------------------------------------------------------------------------------------
def attention_keys_values(h, m: dict, w: Dict[str, torch.Tensor], p: str, eps: float):
    """Keys (rotated, then each head divided by its root mean square) and values of a layer that has projections."""
    T = h.shape[0]
    G, D, E = int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    pos = torch.arange(T)
    k = rms_unit(rotate((h @ w[f"{p}.k"].T).view(T, G, D), pos, m.get("rot")), eps)
    v = (h @ w[f"{p}.v"].T).view(T, G, E)
    return k, v


def attention(h, m: dict, w: Dict[str, torch.Tensor], p: str, eps: float, k, v) -> torch.Tensor:
    """Grouped-query attention with the visible keys cut into chunks counted from position 0."""
    T = h.shape[0]
    H, G, D, E = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    pos = torch.arange(T)
    q = rms_unit(rotate((h @ w[f"{p}.q"].T).view(T, H, D), pos, m.get("rot")), eps)
    see = pos[None, :] <= pos[:, None]
    if m.get("mask"):
        size = int(m["mask"]["size"])
        see = see & ((pos[None, :] // size) == (pos[:, None] // size))
    out = torch.zeros(T, H, E, dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * float(m["scale"])
        s = s.masked_fill(~see, float("-inf"))
        out[:, head] = torch.softmax(s, dim=-1) @ v[:, g]
    return out.reshape(T, H * E) @ w[f"{p}.o"].T


def retention(h, m: dict, w: Dict[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    """Linear attention with a fixed decay per head, walked token by token."""
    T = h.shape[0]
    H, D, E = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    pos = torch.arange(T)
    q = rotate((h @ w[f"{p}.q"].T).view(T, H, D), pos, m.get("rot"))
    k = rotate((h @ w[f"{p}.k"].T).view(T, H, D), pos, m.get("rot")) * D ** -0.5
    v = (h @ w[f"{p}.v"].T).view(T, H, E)
    decay = torch.tensor(m["decay"], dtype=h.dtype)
    S = torch.zeros(H, D, E, dtype=h.dtype)
    o = torch.zeros(T, H, E, dtype=h.dtype)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hde,hd->he", S, q[t])
    o = rms_unit(o, eps).reshape(T, H * E)
    return (o * silu(h @ w[f"{p}.g"].T)) @ w[f"{p}.o"].T


def mamba2(h, m: dict, w: Dict[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    """The state-space mixer: a short causal convolution, then per head a matrix state with a scalar decay."""
    T = h.shape[0]
    H, E, N, G = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"])
    taps, parts = int(m["conv"]), int(m["norm_groups"])
    inner = H * E
    proj = h @ w[f"{p}.in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    padded = torch.cat([torch.zeros(taps - 1, xbc.shape[1], dtype=h.dtype), xbc], dim=0)
    conv = w[f"{p}.conv.b"][None, :].clone().expand(T, -1).clone()
    for j in range(taps):        # tap j weighs the input taps - 1 - j tokens back, so the last tap weighs the token itself
        conv = conv + padded[j:j + T] * w[f"{p}.conv"][:, j][None, :]
    conv = silu(conv)
    x = conv[:, :inner].view(T, H, E)
    B = conv[:, inner:inner + G * N].view(T, G, N)
    C = conv[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + w[f"{p}.dt_bias"][None, :])
    rate = torch.exp(w[f"{p}.A_log"])
    S = torch.zeros(H, N, E, dtype=h.dtype)
    y = torch.zeros(T, H, E, dtype=h.dtype)
    group = torch.arange(H) // (H // G)
    for t in range(T):
        keep = torch.exp(-rate * dt[t])
        S = keep[:, None, None] * S + dt[t][:, None, None] * B[t][group][:, :, None] * x[t][:, None, :]
        y[t] = torch.einsum("hne,hn->he", S, C[t][group]) + w[f"{p}.D"][:, None] * x[t]
    y = y.reshape(T, inner) * silu(z)
    y = rms_unit(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w[f"{p}.norm"]
    return y @ w[f"{p}.o"].T


# ---- feed-forwards -----------------------------------------------------------------------------------------------
def dense_ff(h, mlp: dict, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    limit = float(mlp["limit"])
    g = torch.clamp(h @ w[f"{p}.gate"].T, max=limit)
    u = torch.clamp(h @ w[f"{p}.up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[f"{p}.down"].T


def expert(h, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return (silu(h @ w[f"{p}.gate"].T) * (h @ w[f"{p}.up"].T)) @ w[f"{p}.down"].T


def moe_ff(h, mlp: dict, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    n, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    logits = h @ w[f"{p}.router"].T + w[f"{p}.router.b"][None, :]
    best, chosen = torch.topk(logits, top, dim=-1)
    weight = torch.softmax(best, dim=-1)
    out = torch.zeros_like(h)
    for e in range(n):
        y = expert(h, w, f"{p}.e{e}")
        share = (weight * (chosen == e)).sum(dim=-1, keepdim=True)
        out = out + share * y
    if mlp.get("shared"):
        out = out + torch.sigmoid(h @ w[f"{p}.shared.sg"].T) * expert(h, w, f"{p}.shared")
    return out


# ---- the model ---------------------------------------------------------------------------------------------------
def forward(config: dict, weights: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float32,
            layer_outputs: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence.  ``layer_outputs``, if a list, receives the residual after each layer."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps, alpha = float(config["norm"]["eps"]), float(config["postln_alpha"])
    x = rms_norm(w["embed"][torch.tensor(tokens, dtype=torch.long)], w["embed.norm"], eps)
    kept = {}
    for i, layer in enumerate(config["layers"]):
        m, kind, p = layer["mixer"], layer["type"], f"l{i}.mix"
        if kind == "attention":
            src = m.get("kv_from")
            if src is None:
                kept[i] = attention_keys_values(x, m, w, p, eps)
            y = attention(x, m, w, p, eps, *kept[i if src is None else src])
        elif kind == "retention":
            y = retention(x, m, w, p, eps)
        elif kind == "mamba2":
            y = mamba2(x, m, w, p, eps)
        else:
            raise ValueError(f"layer {i}: no mixer '{kind}'")
        x = rms_norm(alpha * x + y, w[f"l{i}.norm1"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            y = dense_ff(x, mlp, w, f"l{i}.mlp") if mlp["kind"] == "dense" else moe_ff(x, mlp, w, f"l{i}.mlp")
            x = rms_norm(alpha * x + y, w[f"l{i}.norm2"], eps)
        elif f"l{i}.norm2" in w:       # no feed-forward, but the second norm is there: its sum is alpha x alone
            x = rms_norm(alpha * x, w[f"l{i}.norm2"], eps)
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T


def greedy(config: dict, weights: Dict[str, torch.Tensor], prompt: List[int], n_new: int, dtype=torch.float32) -> List[int]:
    """The tokens that always taking the largest logit gives (the whole sequence is run again for every token)."""
    toks, out = list(prompt), []
    for _ in range(n_new):
        nxt = int(torch.argmax(forward(config, weights, toks, dtype)[-1]))
        out.append(nxt)
        toks.append(nxt)
    return out
