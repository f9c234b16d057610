"""A plain, slow statement of the Vebonex design on the CPU: one function per mechanism, whole sequences, no cache.

The product path (``inferrs_b200/models/vebonex.py`` and the parts it names) shares no code with this file.
Everything runs in the dtype of the tensors it is given (float32 or float64).  Notation: ``T`` tokens, ``W`` model
width, ``H`` heads, ``D`` key size per head, ``E`` value size per head, ``R`` latent size.

A model is (config dict, weights dict); the config has the layout that ``config.json`` has.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def grouped_norm(x: torch.Tensor, w: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    """The last axis in ``groups`` equal consecutive parts, each brought to unit root mean square; then times w."""
    parts = x.reshape(x.shape[:-1] + (groups, x.shape[-1] // groups))
    return unit_rms(parts, eps).reshape(x.shape) * w


def poly_norm_act(z: torch.Tensor, coef: torch.Tensor, eps: float) -> torch.Tensor:
    """coef = (a, b, c, e):  a U(z) + b U(z^2) + c U(z^3) + e with U the unit-rms scaling over the last axis."""
    a, b, c, e = (coef[i] for i in range(4))
    return a * unit_rms(z, eps) + b * unit_rms(z * z, eps) + c * unit_rms(z * z * z, eps) + e


def dense_ffn(h: torch.Tensor, up: torch.Tensor, down: torch.Tensor, coef: torch.Tensor, eps: float) -> torch.Tensor:
    return poly_norm_act(h @ up.T, coef, eps) @ down.T


def gla_scan(q, k, v, alpha, S0=None):
    """q, k, alpha [T, H, D], v [T, H, E].  S_t = alpha_t[:, None] * S_{t-1} + k_t v_t^T;  o_t = S_t^T q_t.
    Returns (o [T, H, E], S_T [H, D, E])."""
    T, H, D = q.shape
    E = v.shape[-1]
    S = torch.zeros((H, D, E), dtype=q.dtype) if S0 is None else S0.clone()
    out = []
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hde,hd->he", S, q[t]))
    return torch.stack(out) if out else torch.zeros((0, H, E), dtype=q.dtype), S


def gla_mixer(h, w: Dict[str, torch.Tensor], heads: int, dim: int, vdim: int, tau: float, eps: float, S0=None):
    T = h.shape[0]
    q = (h @ w["q"].T).reshape(T, heads, dim) * dim ** -0.5
    k = (h @ w["k"].T).reshape(T, heads, dim)
    v = (h @ w["v"].T).reshape(T, heads, vdim)
    z = (h @ w["a1"].T) @ w["a2"].T + w["a2.b"]
    alpha = torch.sigmoid(z).pow(1.0 / tau).reshape(T, heads, dim)
    o, S = gla_scan(q, k, v, alpha, S0)
    o = unit_rms(o, eps) * w["norm"]                      # one weight of size E for every head
    gate = torch.nn.functional.silu(h @ w["g"].T)
    return (o.reshape(T, heads * vdim) * gate) @ w["o"].T, S


def soft_cap(x, cap: float):
    return cap * torch.tanh(x / cap)


def mlstm_scan(q, k, v, log_i, log_f, state=None):
    """q, k [T, H, D], v [T, H, E], log_i, log_f [T, H].  A matrix memory S, a vector n and a running maximum m:
        m_t = max(f_t + m_{t-1}, i_t)
        S_t = exp(f_t + m_{t-1} - m_t) S_{t-1} + exp(i_t - m_t) k_t v_t^T      (n_t the same with k_t alone)
        o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
    all of S, n, m start at zero."""
    T, H, D = q.shape
    E = v.shape[-1]
    if state is None:
        S, n, m = torch.zeros((H, D, E), dtype=q.dtype), torch.zeros((H, D), dtype=q.dtype), torch.zeros((H,), dtype=q.dtype)
    else:
        S, n, m = (s.clone() for s in state)
    out = []
    for t in range(T):
        m_new = torch.maximum(log_f[t] + m, log_i[t])
        keep = torch.exp(log_f[t] + m - m_new)
        take = torch.exp(log_i[t] - m_new)
        S = keep[:, None, None] * S + take[:, None, None] * (k[t][:, :, None] * v[t][:, None, :])
        n = keep[:, None] * n + take[:, None] * k[t]
        m = m_new
        num = torch.einsum("hde,hd->he", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        out.append(num / den[:, None])
    return torch.stack(out) if out else torch.zeros((0, H, E), dtype=q.dtype), (S, n, m)


def mlstm_mixer(h, w, heads: int, dim: int, vdim: int, gate_cap: float, eps: float, state=None):
    T = h.shape[0]
    q = (h @ w["q"].T).reshape(T, heads, dim) * dim ** -0.5
    k = (h @ w["k"].T).reshape(T, heads, dim)
    v = (h @ w["v"].T).reshape(T, heads, vdim)
    log_i = soft_cap(h @ w["i"].T + w["i.b"], gate_cap)
    log_f = torch.nn.functional.logsigmoid(soft_cap(h @ w["f"].T + w["f.b"], gate_cap))
    o, state = mlstm_scan(q, k, v, log_i, log_f, state)
    o = unit_rms(o, eps).reshape(T, heads * vdim) * w["norm"]      # a weight over all heads
    return (o * torch.sigmoid(h @ w["g"].T)) @ w["o"].T, state


def latent_of(h, w, eps: float):
    """The cached latent of a layer that has its own down-projection."""
    return unit_rms(h @ w["dkv"].T, eps) * w["dkv.norm"]


def latent_attention(h, c, w, heads: int, dim: int, vdim: int, scale: float, eps: float, start: int = 0,
                     window: Optional[int] = None):
    """h [T, W]: the rows of positions start .. start+T-1;  c [start+T, R]: the latents of positions 0 .. start+T-1.
    Keys and values are made from the latents per head; position i sees every j <= i (with a window: i - window < j);
    plain softmax."""
    T = h.shape[0]
    cq = unit_rms(h @ w["dq"].T, eps) * w["dq.norm"]
    q = (cq @ w["uq"].T).reshape(T, heads, dim)
    k = (c @ w["uk"].T).reshape(-1, heads, dim)
    v = (c @ w["uv"].T).reshape(-1, heads, vdim)
    score = torch.einsum("thd,jhd->htj", q, k) * scale
    i = torch.arange(start, start + T)[:, None]
    j = torch.arange(c.shape[0])[None, :]
    score = score.masked_fill(j > i, float("-inf"))
    if window is not None:
        score = score.masked_fill(j <= i - window, float("-inf"))
    p = torch.softmax(score, dim=-1)
    o = torch.einsum("htj,jhe->the", p, v).reshape(T, heads * vdim)
    return (o * torch.sigmoid(h @ w["g"].T)) @ w["o"].T


def sub(weights: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(config: dict, weights: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float32,
            layer_sums: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence from position 0.  ``layer_sums`` (a list) receives the sum of the
    streams after every layer."""
    wt = {k: v.to(dtype) for k, v in weights.items()}
    eps, groups = float(config["norm"]["eps"]), int(config["norm"]["groups"])
    hyper = config.get("streams") is not None          # without the key: the plain residual x <- x + y
    streams = int(config["streams"]) if hyper else 1
    T = len(tokens)
    x0 = wt["embed"][torch.tensor(tokens)] + wt["pos"][:T]
    xs = [x0.clone() for _ in range(streams)]
    latents: Dict[int, torch.Tensor] = {}
    for li, layer in enumerate(config["layers"]):
        p = f"l{li}."
        m = layer["mixer"]

        def mixer(h):
            w = sub(wt, p + "mix.")
            if layer["type"] == "gla":
                return gla_mixer(h, w, m["heads"], m["dim"], m["vdim"], float(m["tau"]), eps)[0]
            if layer["type"] == "mlstm":
                return mlstm_mixer(h, w, m["heads"], m["dim"], m["vdim"], float(m["gate_cap"]), eps)[0]
            if layer["type"] == "latent_attention":
                if m.get("kv_from") is None:
                    latents[li] = latent_of(h, w, eps)
                    c = latents[li]
                else:
                    c = latents[int(m["kv_from"])]
                return latent_attention(h, c, w, m["heads"], m["dim"], m["vdim"], float(m["scale"]), eps)
            raise ValueError(layer["type"])

        def ffn(h):
            w = sub(wt, p + "mlp.")
            return dense_ffn(h, w["up"], w["down"], w["act"], eps)

        for q, (fn, present) in enumerate(((mixer, True), (ffn, layer.get("mlp") is not None)), start=1):
            if not present:
                continue
            if not hyper:
                xs = [xs[0] + fn(grouped_norm(xs[0], wt[f"{p}norm{q}"], groups, eps))]
                continue
            hc = sub(wt, f"{p}hc{q}.")
            u = sum(hc["in"][s] * xs[s] for s in range(streams))
            y = fn(grouped_norm(u, wt[f"{p}norm{q}"], groups, eps))
            xs = [sum(hc["mix"][s, t] * xs[s] for s in range(streams)) + hc["out"][t] * y for t in range(streams)]
        if layer_sums is not None:
            layer_sums.append(sum(xs))
    x = sum(xs)
    return grouped_norm(x, wt["final.norm"], groups, eps) @ wt["head"].T


def greedy(config: dict, weights: Dict[str, torch.Tensor], prompt: List[int], n_new: int, dtype=torch.float32) -> List[int]:
    """The tokens that always taking the largest logit gives (the whole sequence is run again for every token)."""
    toks, out = list(prompt), []
    for _ in range(n_new):
        nxt = int(torch.argmax(forward(config, weights, toks, dtype)[-1]))
        out.append(nxt)
        toks.append(nxt)
    return out
