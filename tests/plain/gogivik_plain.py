"""Plain, slow, whole-sequence implementation of the Gogivik design (on the CPU, float64 or float32): the oracle
that the engine is compared with.

No cache, no batching, no kernels: one function per mechanism, token by token where the design is a recurrence.
It shares no code with the product package: it reads config.json keys and safetensors names itself.

The design in this file's notation (x: the stream [tokens, width]; unit(y) = y / sqrt(mean(y^2) + eps)):

    x        = embed[token]
    layer:     u = norm1(x);  u <- u + tapconv1(u);  x <- x + mixer(u)
               u = norm2(x);  u <- u + tapconv2(u);  x <- x + ff(u)             (no feed-forward: no second half)
    norm(x)  = unit(x) * (1 + w)
    tapconv  : per channel, over time, causal: out_t = sum_j w[:, j] * in_(t - taps + 1 + j), zeros before the start
    ff(u)    = W_down relu(W_up u)^2
    logits   = head norm_final(x) * logit_scale

mixers:

    attention         grouped-query softmax attention; queries and keys unit-normed per head (times a weight) and
                      rotated in halves with frequencies divided by a factor; values unit-normed per head and rotated by
                      their own position over their whole size, the summed output rotated back by the query's position;
                      a key is visible if it is not later and lies in the query's chunk of `mask.size` positions
    latent_attention  queries from a normed latent; keys and values from one normed latent per token plus one rotated
                      key part shared by the heads (interleaved pairs); a window of `mask.size` positions; the softmax's
                      denominator also holds exp(sink_h)
    mamba2            a state N x vdim per head: S <- exp(-exp(A_log) dt) S + dt B x^T, y = S^T C + D x; x, B, C pass a
                      short causal convolution and silu; y times silu(z), unit-normed in groups, times a weight
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch
import torch.nn.functional as F


def read_config(folder) -> dict:
    return json.loads((Path(folder) / "config.json").read_text())


def read_weights(folder, dtype=torch.float64) -> dict:
    from safetensors import safe_open

    out = {}
    for shard in sorted(Path(folder).glob("*.safetensors")):
        with safe_open(str(shard), framework="pt") as f:
            for key in f.keys():
                t = f.get_tensor(key)
                out[key] = t.to(dtype) if t.is_floating_point() else t
    return out


# ----------------------------------------------------------------------- small parts
def unit(y: torch.Tensor, eps: float) -> torch.Tensor:
    """y divided by its root mean square over the last axis, eps inside the root."""
    return y / torch.sqrt((y * y).mean(dim=-1, keepdim=True) + eps)


def offset_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The layers' norm: one is added to the stored weight."""
    return unit(x, eps) * (1.0 + w)


def tap_conv(u: torch.Tensor, w: torch.Tensor, bias=None) -> torch.Tensor:
    """Causal convolution over time on each channel: u [T, C], w [C, taps]; the last column weighs the current
    token, the one before it the token before, and so on; nothing before the sequence's start."""
    T, C = u.shape
    taps = w.shape[1]
    out = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += w[:, j] * u[s]
    if bias is not None:
        out = out + bias
    return out


def frequencies(base: float, dims: int, factor: float = 1.0, dtype=torch.float64) -> torch.Tensor:
    i = torch.arange(dims // 2, dtype=dtype)
    return base ** (-2.0 * i / dims) / factor


def rotate(y: torch.Tensor, pos: torch.Tensor, freq: torch.Tensor, layout: str, sign: float = 1.0) -> torch.Tensor:
    """Rotates the first 2 * len(freq) elements of the last axis of y [T, ..., D] by pos * freq; `halves` pairs
    element i with i + dims/2, `interleaved` pairs 2i with 2i + 1.  The rest passes unchanged."""
    half = freq.numel()
    dims = 2 * half
    shape = [y.shape[0]] + [1] * (y.dim() - 2) + [half]
    a = (pos.to(freq.dtype)[:, None] * freq[None, :]).reshape(shape) * sign
    cos, sin = torch.cos(a).to(y.dtype), torch.sin(a).to(y.dtype)
    out = y.clone()
    if layout == "halves":
        u, v = y[..., :half], y[..., half:dims]
        out[..., :half] = u * cos - v * sin
        out[..., half:dims] = v * cos + u * sin
    else:
        u, v = y[..., 0:dims:2], y[..., 1:dims:2]
        out[..., 0:dims:2] = u * cos - v * sin
        out[..., 1:dims:2] = v * cos + u * sin
    return out


def visible(T: int, window=None, chunk=None) -> torch.Tensor:
    """[T, T] boolean: query i (row) sees key j (column)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    m = j <= i
    if window is not None:
        m &= (i - j) < window
    if chunk is not None:
        m &= (i // chunk) == (j // chunk)
    return m


def softmax_attend(q, k, v, scale: float, mask: torch.Tensor, sink=None) -> torch.Tensor:
    """q [T, H, D], k [T, H, D], v [T, H, E] (keys and values already per query head) -> [T, H, E].  With `sink`
    [H] the denominator also holds exp(sink_h), which has no value."""
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    s = s.masked_fill(~mask[None], float("-inf"))
    if sink is None:
        p = torch.softmax(s, dim=-1)
    else:
        m = torch.maximum(s.max(dim=-1, keepdim=True).values, sink[:, None, None])
        e = torch.exp(s - m)
        p = e / (e.sum(dim=-1, keepdim=True) + torch.exp(sink[:, None, None] - m))
    return torch.einsum("hij,jhe->ihe", p, v)


# ----------------------------------------------------------------------------- mixers
def attention(u, w: dict, p: str, mx: dict, eps: float) -> torch.Tensor:
    T = u.shape[0]
    H, G, D, E = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    rot, chunk = mx["rot"], mx["mask"]["size"]
    pos = torch.arange(T)
    q = (u @ w[f"{p}.q"].T).view(T, H, D)
    k = (u @ w[f"{p}.k"].T).view(T, G, D)
    v = (u @ w[f"{p}.v"].T).view(T, G, E)
    q = unit(q, eps) * w[f"{p}.q.norm"]
    k = unit(k, eps) * w[f"{p}.k.norm"]
    factor = float(rot["scaling"]["factor"]) if rot.get("scaling") else 1.0
    fq = frequencies(float(rot["base"]), int(rot["dims"]), factor, u.dtype)
    q, k = rotate(q, pos, fq, "halves"), rotate(k, pos, fq, "halves")
    fv = frequencies(float(rot["base"]), E, 1.0, u.dtype)
    v = rotate(unit(v, eps), pos, fv, "halves")
    rep = H // G
    k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    o = softmax_attend(q, k, v, float(mx["scale"]), visible(T, chunk=chunk))
    o = rotate(o, pos, fv, "halves", sign=-1.0)
    return o.reshape(T, H * E) @ w[f"{p}.o"].T


def latent_attention(u, w: dict, p: str, mx: dict, eps: float) -> torch.Tensor:
    T = u.shape[0]
    H, D, R, E, C = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    rot = mx["rot"]
    pos = torch.arange(T)
    cq = unit(u @ w[f"{p}.dq"].T, eps) * w[f"{p}.dq.norm"]
    q = (cq @ w[f"{p}.uq"].T).view(T, H, D + R)
    dkv = u @ w[f"{p}.dkv"].T
    c = unit(dkv[:, :C], eps) * w[f"{p}.dkv.norm"]
    f = frequencies(float(rot["base"]), int(rot["dims"]), 1.0, u.dtype)
    kr = rotate(dkv[:, None, C:], pos, f, "interleaved")                       # [T, 1, R]
    qr = rotate(q[:, :, D:], pos, f, "interleaved")
    ku = (c @ w[f"{p}.uk"].T).view(T, H, D)
    v = (c @ w[f"{p}.uv"].T).view(T, H, E)
    qq = torch.cat([q[:, :, :D], qr], dim=-1)
    kk = torch.cat([ku, kr.expand(T, H, R)], dim=-1)
    o = softmax_attend(qq, kk, v, float(mx["scale"]), visible(T, window=mx["mask"]["size"]), sink=w[f"{p}.sink"])
    return o.reshape(T, H * E) @ w[f"{p}.o"].T


def mamba2(u, w: dict, p: str, mx: dict, eps: float) -> torch.Tensor:
    T = u.shape[0]
    H, E, N, G, NG = mx["heads"], mx["vdim"], mx["state"], mx["groups"], mx["norm_groups"]
    inner = H * E
    row = u @ w[f"{p}.in"].T
    z, xbc, dt = row[:, :inner], row[:, inner:2 * inner + 2 * G * N], row[:, 2 * inner + 2 * G * N:]
    xbc = F.silu(tap_conv(xbc, w[f"{p}.conv"], w[f"{p}.conv.b"]))
    x = xbc[:, :inner].view(T, H, E)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = F.softplus(dt + w[f"{p}.dt_bias"])                                    # [T, H]
    decay = torch.exp(-torch.exp(w[f"{p}.A_log"]) * dt)
    S = torch.zeros(H, N, E, dtype=u.dtype)
    y = torch.zeros(T, H, E, dtype=u.dtype)
    per = H // G
    for t in range(T):
        Bh, Ch = B[t].repeat_interleave(per, dim=0), C[t].repeat_interleave(per, dim=0)      # [H, N]
        S = decay[t][:, None, None] * S + dt[t][:, None, None] * Bh[:, :, None] * x[t][:, None, :]
        y[t] = torch.einsum("hne,hn->he", S, Ch) + w[f"{p}.D"][:, None] * x[t]
    y = y.reshape(T, inner) * F.silu(z)
    y = unit(y.view(T, NG, inner // NG), eps).reshape(T, inner) * w[f"{p}.norm"]
    return y @ w[f"{p}.o"].T


MIXERS = {"attention": attention, "latent_attention": latent_attention, "mamba2": mamba2}


def feed_forward(u, w: dict, p: str) -> torch.Tensor:
    return torch.relu(u @ w[f"{p}.up"].T) ** 2 @ w[f"{p}.down"].T


# ------------------------------------------------------------------------------ model
def forward(cfg: dict, w: dict, tokens, taps=None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence run whole.  `taps`, a list, receives the stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    for i, ly in enumerate(cfg["layers"]):
        p = f"l{i}"
        u = offset_norm(x, w[f"{p}.norm1"], eps)
        u = u + tap_conv(u, w[f"{p}.canon1"])
        x = x + MIXERS[ly["type"]](u, w, f"{p}.mix", ly["mixer"], eps)
        if ly.get("mlp") is not None:
            u = offset_norm(x, w[f"{p}.norm2"], eps)
            u = u + tap_conv(u, w[f"{p}.canon2"])
            x = x + feed_forward(u, w, f"{p}.mlp")
        if taps is not None:
            taps.append(x.clone())
    return offset_norm(x, w["final.norm"], eps) @ w["head"].T * float(cfg.get("logit_scale", 1.0))
