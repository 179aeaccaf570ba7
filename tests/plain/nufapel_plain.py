"""Plain, slow, whole-sequence implementation of the Nufapel design (on the CPU, float64 or float32): the
oracle that the engine is compared with.

No cache, no batching, no kernels: one function per mechanism, token by token where the design is a recurrence.
It shares no code with the product package: it reads config.json keys and safetensors names itself.

The design in this file's notation (x: the stream [tokens, width]; unit(y) = y / sqrt(mean(y^2) + eps)):

    x            = embed[token] + pos[position]
    loop:          layers start .. stop-1 run `times` times with the same weights, every pass with keys, values and
                   states of its own; right before pass t, x <- x + loop.step[t]
    dyt(x)       = tanh(alpha x) * w + b
    layer:   h   = dyt1(x);  x <- x + sigmoid(rg1 h + b1) * mixer(h)
             h   = dyt2(x);  x <- x + sigmoid(rg2 h + b2) * ff(h)            (no feed-forward: no second half)
    logits       = cap * tanh(head dyt_final(x) / cap)

mixers:

    general_delta   per head a matrix S (key channel x value channel), zero at the start;
                    S <- diag(w) S - (a u)(u^T S) + k v^T,  o = S^T r,  u = k / |k|
    parallel        half of unit(left) * w_left + unit(right) * w_right:
        left        causal softmax attention without rotation; score = q.k * scale * temp_h + rel[bucket(i - j), h];
                    the softmax's denominator also holds exp(sink_h); head h times sigmoid(g_h . h)
        right       matrix memory with exponential gates and a running maximum m for their scale

feed-forwards: W_down gelu(W_up h), or routed experts (sigmoid scores, groups scored by their two best).
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


def dyt(x, W, name):
    """Dynamic tanh: no mean, no variance."""
    return torch.tanh(W[f"{name}.alpha"] * x) * W[name] + W[f"{name}.b"]


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def run_order(cfg: dict):
    """[(layer, pass number or None if the layer starts no pass)] in the order in which the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if loop is None:
        return [(i, None) for i in range(n)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, None) for i in range(a)]
    for t in range(times):
        order += [(i, t if i == a else None) for i in range(a, b)]
    return order + [(i, None) for i in range(b, n)]


# -------------------------------------------------------------------- general_delta
def delta_scan(r, k, v, w, a, S=None):
    """The generalized delta rule over T tokens.  r, k, w, a [T, H, D], v [T, H, V]; S [H, D, V] (zero if None).
    Returns (o [T, H, V], the state after the last token)."""
    T, H, D = k.shape
    u = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    S = torch.zeros(H, D, v.shape[-1], dtype=k.dtype) if S is None else S.clone()
    o = torch.zeros(T, H, v.shape[-1], dtype=k.dtype)
    for t in range(T):
        uS = torch.einsum("hk,hkv->hv", u[t], S)                      # u^T S, the old state
        S = w[t][:, :, None] * S - (a[t] * u[t])[:, :, None] * uS[:, None, :] + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, r[t])
    return o, S


def delta_decay(z):
    """The decay per channel from its pre-activation (bias included)."""
    return torch.exp(-math.exp(-0.5) * torch.sigmoid(z))


def general_delta(h, W, p, mx, eps):
    """h [T, width] -> [T, width]; p the tensor prefix '<layer>.mix'."""
    H, D = int(mx["heads"]), int(mx["dim"])
    T = h.shape[0]
    r = (h @ W[f"{p}.r"].T).view(T, H, D)
    k = (h @ W[f"{p}.k"].T).view(T, H, D)
    v = (h @ W[f"{p}.v"].T).view(T, H, D)
    w = delta_decay(torch.tanh(h @ W[f"{p}.w1"].T) @ W[f"{p}.w2"].T + W[f"{p}.w0"]).view(T, H, D)
    a = torch.sigmoid(h @ W[f"{p}.a"].T + W[f"{p}.a.b"]).view(T, H, D)
    o, _ = delta_scan(r, k, v, w, a)
    o = unit(o, eps).reshape(T, H * D) * W[f"{p}.norm"]
    return (o * torch.sigmoid(h @ W[f"{p}.g"].T)) @ W[f"{p}.o"].T


# ------------------------------------------------------------------ parallel: left
def distance_bucket(n: int, B: int, D: int) -> int:
    half = B // 2
    if n < half:
        return n
    return min(B - 1, half + int(math.floor(math.log(n / half) / math.log(D / half) * (B - half))))


def biased_sink_attend(q, k, v, scale, temp, rel, bias_max, sink, first=0):
    """q [Tq, H, D] at positions first .. first + Tq - 1 against k [T, H, D], v [T, H, V] at positions 0 .. T - 1
    (causal).  score = q.k * scale * temp_h + rel[bucket(i - j), h]; the softmax's denominator also holds exp(sink_h),
    which has no value.  Returns [Tq, H, V]."""
    Tq, T, B = q.shape[0], k.shape[0], rel.shape[0]
    buckets = torch.tensor([[distance_bucket(first + i - j, B, bias_max) if j <= first + i else 0 for j in range(T)]
                            for i in range(Tq)])
    s = torch.einsum("ihd,jhd->hij", q, k) * scale * temp[:, None, None]
    s = s + rel[buckets].permute(2, 0, 1)
    hidden = torch.arange(T)[None, :] > (first + torch.arange(Tq))[:, None]
    s = s.masked_fill(hidden, -math.inf)
    sk = sink[:, None, None]
    m = torch.maximum(s.max(dim=-1, keepdim=True).values, sk)
    e = torch.exp(s - m)
    weights = e / (e.sum(-1, keepdim=True) + torch.exp(sk - m))
    return torch.einsum("hij,jhv->ihv", weights, v)


def sink_attention(h, W, p, mx):
    """Causal softmax attention with a learned distance bias, a temperature per head and a sink in the denominator;
    p the tensor prefix '<layer>.mix.left'.  Returns the projected output [T, width]."""
    H, G, D, V = int(mx["heads"]), int(mx["kv_heads"]), int(mx["dim"]), int(mx["vdim"])
    T = h.shape[0]
    q = (h @ W[f"{p}.q"].T).view(T, H, D)
    k = (h @ W[f"{p}.k"].T).view(T, G, D).repeat_interleave(H // G, dim=1)
    v = (h @ W[f"{p}.v"].T).view(T, G, V).repeat_interleave(H // G, dim=1)
    o = biased_sink_attend(q, k, v, float(mx["scale"]), W[f"{p}.temp"], W[f"{p}.rel"], int(mx["bias_max"]), W[f"{p}.sink"])
    o = o * torch.sigmoid(h @ W[f"{p}.g"].T)[:, :, None]
    return o.reshape(T, H * V) @ W[f"{p}.o"].T


# ----------------------------------------------------------------- parallel: right
def capped_gates(zi, zf, cap):
    """Log input gate and log forget gate from their pre-activations (biases included)."""
    return cap * torch.tanh(zi / cap), F.logsigmoid(cap * torch.tanh(zf / cap))


def memory_scan(q, k, v, gi, gf, state=None):
    """The matrix memory over T tokens.  q (already scaled), k [T, H, D], v [T, H, V], gi, gf [T, H] (log gates);
    state = (S [H, D, V], n [H, D], m [H]), all zero if None.  Returns (o [T, H, V], the state after the last token)."""
    T, H, D = k.shape
    V = v.shape[-1]
    if state is None:
        S, n, m = torch.zeros(H, D, V, dtype=k.dtype), torch.zeros(H, D, dtype=k.dtype), torch.zeros(H, dtype=k.dtype)
    else:
        S, n, m = (t.clone() for t in state)
    o = torch.zeros(T, H, V, dtype=k.dtype)
    for t in range(T):
        m_new = torch.maximum(gf[t] + m, gi[t])
        keep, take = torch.exp(gf[t] + m - m_new), torch.exp(gi[t] - m_new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[t]
        m = m_new
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        o[t] = torch.einsum("hkv,hk->hv", S, q[t]) / den[:, None]
    return o, (S, n, m)


def matrix_memory(h, W, p, mx, eps):
    """Matrix memory with exponential input gate and sigmoid forget gate in the log domain; p the tensor prefix
    '<layer>.mix.right'."""
    H, D, V, cap = int(mx["heads"]), int(mx["dim"]), int(mx["vdim"]), float(mx["gate_cap"])
    T = h.shape[0]
    q = (h @ W[f"{p}.q"].T).view(T, H, D) * D ** -0.5
    k = (h @ W[f"{p}.k"].T).view(T, H, D)
    v = (h @ W[f"{p}.v"].T).view(T, H, V)
    gi, gf = capped_gates(h @ W[f"{p}.i"].T + W[f"{p}.i.b"], h @ W[f"{p}.f"].T + W[f"{p}.f.b"], cap)
    o, _ = memory_scan(q, k, v, gi, gf)
    o = unit(o, eps).reshape(T, H * V) * W[f"{p}.norm"]
    return (o * torch.sigmoid(h @ W[f"{p}.g"].T)) @ W[f"{p}.o"].T


def parallel_mixer(h, W, p, mx, eps):
    left = sink_attention(h, W, f"{p}.left", mx["left"])
    right = matrix_memory(h, W, f"{p}.right", mx["right"], eps)
    return 0.5 * (unit(left, eps) * W[f"{p}.left.out"] + unit(right, eps) * W[f"{p}.right.out"])


# -------------------------------------------------------------------- feed-forwards
def dense_ff(h, W, p):
    return gelu_erf(h @ W[f"{p}.up"].T) @ W[f"{p}.down"].T


def route(z, top: int, groups: int, keep: int, scale: float, margins=None):
    """z [T, E] router logits -> (chosen experts [T, top], their weights [T, top]).  `margins`, a list, receives
    per token the smallest difference of scores on which a choice hangs (the last kept group against the best one
    dropped, the last chosen expert against the best one left)."""
    T, E = z.shape
    s = torch.sigmoid(z)
    per = E // groups
    gs = s.view(T, groups, per).topk(min(2, per), dim=-1).values.sum(-1)
    ranked = gs.topk(groups, dim=-1)
    kept = ranked.indices[:, :keep]
    allowed = torch.zeros(T, groups, dtype=torch.bool).scatter_(1, kept, True).repeat_interleave(per, dim=1)
    masked = torch.where(allowed, s, torch.full_like(s, -1.0))
    best = masked.topk(min(top + 1, keep * per), dim=-1)
    idx = best.indices[:, :top]
    chosen = s.gather(1, idx)
    if margins is not None:
        m = torch.full((T,), float("inf"), dtype=z.dtype)
        if keep < groups:
            m = torch.minimum(m, ranked.values[:, keep - 1] - ranked.values[:, keep])
        if best.values.shape[1] > top:
            m = torch.minimum(m, best.values[:, top - 1] - best.values[:, top])
        margins.append(m)
    return idx, chosen / (chosen.sum(-1, keepdim=True) + 1e-20) * scale


def expert(h, W, p, limit):
    g = torch.clamp(h @ W[f"{p}.gate"].T, max=limit)
    u = torch.clamp(h @ W[f"{p}.up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W[f"{p}.down"].T


def routed_ff(h, W, p, ml, margins=None):
    ro = ml["router"]
    z = h @ W[f"{p}.router"].T
    idx, wt = route(z, int(ro["top"]), int(ro["groups"]["count"]), int(ro["groups"]["keep"]), float(ro["scale"]), margins)
    out = torch.zeros_like(h)
    for e in range(int(ro["experts"])):
        hit = (idx == e)
        rows = hit.any(-1)
        if rows.any():
            y = expert(h[rows], W, f"{p}.e{e}", float(ml["expert"]["limit"]))
            out[rows] += y * (wt * hit)[rows].sum(-1, keepdim=True)
    return out


# ------------------------------------------------------------------------ the model
def forward(cfg: dict, W: dict, tokens, taps=None, margins=None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence run whole.  `taps`, a list, receives the stream after every layer run;
    `margins`, a list, one tensor [T] per routed feed-forward that ran (see `route`)."""
    eps = float(cfg["norm"]["eps"])
    T = len(tokens)
    x = W["embed"][torch.tensor(tokens)] + W["pos"][:T]
    for i, starts_pass in run_order(cfg):
        layer, p = cfg["layers"][i], f"l{i}"
        if starts_pass is not None:
            x = x + W["loop.step"][starts_pass]
        h = dyt(x, W, f"{p}.norm1")
        if layer["type"] == "general_delta":
            y = general_delta(h, W, f"{p}.mix", layer["mixer"], eps)
        elif layer["type"] == "parallel":
            y = parallel_mixer(h, W, f"{p}.mix", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + torch.sigmoid(h @ W[f"{p}.rg1"].T + W[f"{p}.rg1.b"]) * y
        ml = layer.get("mlp")
        if ml is not None:
            h = dyt(x, W, f"{p}.norm2")
            y = dense_ff(h, W, f"{p}.mlp") if ml["kind"] == "dense" else routed_ff(h, W, f"{p}.mlp", ml, margins)
            x = x + torch.sigmoid(h @ W[f"{p}.rg2"].T + W[f"{p}.rg2.b"]) * y
        if taps is not None:
            taps.append(x.clone())
    logits = dyt(x, W, "final.norm") @ W["head"].T
    cap = cfg.get("logit_softcap")
    return logits if cap is None else float(cap) * torch.tanh(logits / float(cap))
