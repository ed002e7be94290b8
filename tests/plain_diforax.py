"""A plain, slow Diforax in PyTorch on the CPU: one function per mechanism, written from the design's
equations, sharing no code with the engine.  Tests compare the engine's parts and whole models with it.

Notation: T tokens, W model width, H query heads, G key/value heads, d query/key size, e value size,
L taps, E routed experts, I identity experts.  Everything runs in the dtype of the tensors handed in
(the tests use float64).
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import torch
import torch.nn.functional as F


def same(value):
    return value


def bf16(value):
    """Round to bfloat16 and back: what a 16-bit engine loses where it stores 16 bits."""
    return value.to(torch.bfloat16).to(value.dtype)


def load_model_dir(path):
    """(config dict, name -> float64 tensor) of a model folder, read with this file's own reader."""
    path = Path(path)
    config = json.loads((path / "config.json").read_text())
    raw = (path / "model.safetensors").read_bytes()
    size = int.from_bytes(raw[:8], "little")
    header = json.loads(raw[8:8 + size])
    kinds = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "I32": torch.int32}
    weights = {}
    for name, entry in header.items():
        if name == "__metadata__":
            continue
        begin, end = entry["data_offsets"]
        flat = torch.frombuffer(bytearray(raw[8 + size + begin:8 + size + end]), dtype=kinds[entry["dtype"]])
        tensor = flat.reshape(entry["shape"])
        weights[name] = tensor.to(torch.float64) if tensor.is_floating_point() else tensor
    return config, weights


# ------------------------------------------------------------------ small functions
def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x, weight, eps):
    return rms_unit(x, eps) * weight


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


# ------------------------------------------------------------------ rotary positions
def rotate(x, positions, base, dims):
    """x: [T][heads][d].  Channel i < dims/2 pairs with channel i + dims/2; the pair turns by
    position * base^(-2i/dims).  Channels from ``dims`` on pass unchanged."""
    if dims == 0:
        return x
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    freq = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims)
    angle = positions.to(torch.float64)[:, None] * freq[None, :]
    cos, sin = torch.cos(angle).to(x.dtype)[:, None, :], torch.sin(angle).to(x.dtype)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, x[..., dims:]], dim=-1)


# ------------------------------------------------------------------ attention inside chunks
def chunk_visible(q_positions, k_positions, chunk):
    """[Tq][Tk] bool: key j is seen from i when j <= i and both lie in the same run of ``chunk``
    positions counted from position 0."""
    i, j = q_positions[:, None], k_positions[None, :]
    return (j <= i) & (torch.div(i, chunk, rounding_mode="floor") == torch.div(j, chunk, rounding_mode="floor"))


def attention_keys(h, positions, w_k, w_v, G, d, e, base, dims, eps, rnd=same):
    """What an attention layer caches for the rows ``h``: keys (turned, then brought to unit root
    mean square per head) [T][G][d] and values [T][G][e].  ``rnd`` rounds the projections' results."""
    T = h.shape[0]
    k = rms_unit(rotate(rnd(h @ w_k.T).view(T, G, d), positions, base, dims), eps)
    return k, rnd(h @ w_v.T).view(T, G, e)


def attention_queries(h, positions, w_q, H, d, base, dims, eps, rnd=same):
    T = h.shape[0]
    return rms_unit(rotate(rnd(h @ w_q.T).view(T, H, d), positions, base, dims), eps)


def chunked_attention(q, q_positions, k, v, k_positions, scale, chunk):
    """q [Tq][H][d], k [Tk][G][d], v [Tk][G][e] -> [Tq][H*e]; softmax over the visible keys."""
    H, G = q.shape[1], k.shape[1]
    per = H // G
    seen = chunk_visible(q_positions, k_positions, chunk)
    out = []
    for head in range(H):
        g = head // per
        s = (q[:, head, :] @ k[:, g, :].T) * scale
        s = s.masked_fill(~seen, float("-inf"))
        out.append(torch.softmax(s, dim=-1) @ v[:, g, :])
    return torch.cat(out, dim=-1)


# ------------------------------------------------------------------ gated delta rule
def short_conv(x, taps, history=None):
    """Causal convolution along time, one filter per channel.  x [T][C], taps [C][L] (the last tap
    multiplies the current token), ``history`` [L-1][C]: the inputs before this run (zeros at the start
    of a sequence).  Returns (y [T][C], the last L-1 inputs)."""
    T, C = x.shape
    L = taps.shape[1]
    if history is None:
        history = torch.zeros((L - 1, C), dtype=x.dtype)
    padded = torch.cat([history, x], dim=0)
    y = torch.zeros_like(x)
    for tap in range(L):
        y = y + padded[tap:tap + T] * taps[:, tap][None, :]
    return y, padded[T:]


def unit_vector(x):
    return x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + 1e-6)


def delta_rule_scan(q, k, v, beta, decay, S):
    """One head-group's recurrence over T tokens.  q, k [T][H][d] (already per query head), v [T][H][e],
    beta, decay [T][H], S [H][d][e].  Per token: S *= decay; u = beta (v - S^T k); S += k u^T; o = S^T q."""
    T = q.shape[0]
    out = []
    S = S.clone()
    for t in range(T):
        S = S * decay[t][:, None, None]
        u = beta[t][:, None] * (v[t] - torch.einsum("hde,hd->he", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        out.append(torch.einsum("hde,hd->he", S, q[t]))
    return torch.stack(out), S


def delta_mixer(h, w, H, G, d, e, eps, state=None, rnd=same):
    """The whole mixer on rows ``h`` [T][W].  ``w``: dict of the mixer's tensors by short name
    (q, q.conv, k, k.conv, v, v.conv, b, a, A_log, dt_bias, g, norm, o).  ``state``: None at the start of a
    sequence, else (S, conv history of q, of k, of v).  Returns (delta [T][W], new state)."""
    T = h.shape[0]
    S, hq, hk, hv = state if state is not None else (torch.zeros((H, d, e), dtype=h.dtype), None, None, None)
    q, hq = short_conv(h @ w["q"].T, w["q.conv"], hq)
    k, hk = short_conv(h @ w["k"].T, w["k.conv"], hk)
    v, hv = short_conv(h @ w["v"].T, w["v.conv"], hv)
    q = unit_vector(silu(q).view(T, G, d)) * d ** -0.5
    k = unit_vector(silu(k).view(T, G, d))
    v = silu(v).view(T, H, e)
    per = H // G
    q, k = q.repeat_interleave(per, dim=1), k.repeat_interleave(per, dim=1)
    beta = torch.sigmoid(h @ w["b"].T)
    decay = torch.exp(-torch.exp(w["A_log"]) * F.softplus(h @ w["a"].T + w["dt_bias"]))
    o, S = delta_rule_scan(q, k, v, beta, decay, S)
    o = rms_unit(o, eps) * w["norm"] * silu(h @ w["g"].T).view(T, H, e)
    return rnd(o.reshape(T, H * e)) @ w["o"].T, (S, hq, hk, hv)


# ------------------------------------------------------------------ feed-forwards
def gated_ff(h, gate, up, down, act, rnd=same):
    return rnd(act(h @ gate.T) * (h @ up.T)) @ down.T


def route(h, router, correction, n_groups, keep, top):
    """ids [T][top] and weights [T][top].  Scores are the softmax over all router outputs; the choice
    is made on score + correction, inside the ``keep`` groups (of neighbouring outputs) whose largest
    choice value is largest; the weights are the plain scores of the chosen, as they are."""
    s = torch.softmax(h @ router.T, dim=-1)
    choice = s + correction
    T, N = choice.shape
    per = N // n_groups
    best = choice.view(T, n_groups, per).max(dim=-1).values
    kept = torch.topk(best, keep, dim=-1).indices
    allowed = torch.zeros((T, n_groups), dtype=torch.bool)
    allowed.scatter_(1, kept, True)
    choice = choice.masked_fill(~allowed.repeat_interleave(per, dim=1), float("-inf"))
    ids = torch.topk(choice, top, dim=-1).indices
    return ids, torch.gather(s, 1, ids)


def moe(h, router, correction, experts, n_identity, n_groups, keep, top, rnd=same):
    """``experts``: list of (gate, up, down); router outputs behind them are identity experts, which
    hand the input itself on."""
    ids, weights = route(h, router, correction, n_groups, keep, top)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for slot in range(top):
            e = int(ids[t, slot])
            y = h[t] if e >= len(experts) else gated_ff(h[t:t + 1], *experts[e], silu, rnd)[0]
            out[t] += weights[t, slot] * y
    return out


# ------------------------------------------------------------------ the model
def _layer_tensors(weights, prefix):
    return {name[len(prefix):]: t for name, t in weights.items() if name.startswith(prefix)}


def forward(config, weights, tokens, dtype=torch.float64, keep_layers=False, rnd=same):
    """Logits [T][vocab] of one whole sequence (and the stream after every layer, if asked).
    ``config``: the dict of config.json; ``weights``: name -> tensor.  ``rnd=bf16`` rounds what a 16-bit
    engine keeps in 16 bits (the inputs of the products, cached keys and values, the mixers' outputs in
    front of their last product), not the stream, norms, router or recurrence: the difference to
    ``rnd=same`` is the error that rounding alone causes."""
    w = {name: (t.to(dtype) if t.is_floating_point() else t) for name, t in weights.items()}
    eps = float(config["norm"]["eps"])
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    T = tokens.numel()
    positions = torch.arange(T)
    x = w["embed"][tokens]
    cached = {}
    after = []
    for index, layer in enumerate(config["layers"]):
        p = f"l{index}."
        m = layer["mixer"]
        h = rnd(rms_norm(x, w[p + "norm1"], eps))
        mix = _layer_tensors(w, p + "mix.")
        if layer["type"] == "attention":
            if m.get("kv_from") is not None:
                # what a layer that reads another's keys leaves unsaid about them is the owner's
                m = {**{key: config["layers"][int(m["kv_from"])]["mixer"][key] for key in ("kv_heads", "dim", "vdim", "rot")
                        if key in config["layers"][int(m["kv_from"])]["mixer"]}, **m}
            H, G, d, e = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
            rot = m.get("rot") or {"base": 1.0, "dims": 0}            # no "rot": nothing turns
            base, dims = float(rot["base"]), int(rot["dims"])
            if m.get("kv_from") is not None:
                k, v = cached[int(m["kv_from"])]
            else:
                k, v = attention_keys(h, positions, mix["k"], mix["v"], G, d, e, base, dims, eps, rnd)
                k, v = rnd(k), rnd(v)
                cached[index] = (k, v)
            q = rnd(attention_queries(h, positions, mix["q"], H, d, base, dims, eps, rnd))
            chunk = int((m.get("mask") or {}).get("size") or T + 1)
            y = rnd(chunked_attention(q, positions, k, v, positions, float(m["scale"]), chunk)) @ mix["o"].T
        elif layer["type"] == "delta":
            y, _ = delta_mixer(h, mix, int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"]), eps,
                               rnd=rnd)
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(y, w[p + "norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = rnd(rms_norm(x, w[p + "norm2"], eps))
            if mlp["kind"] == "dense":
                y = gated_ff(h, w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"], gelu_tanh, rnd)
            else:
                r = mlp["router"]
                E, n_id = int(r["experts"]), int(r.get("identity", 0))
                experts = [(w[f"{p}mlp.e{j}.gate"], w[f"{p}mlp.e{j}.up"], w[f"{p}mlp.e{j}.down"]) for j in range(E)]
                groups = r.get("groups") or {}
                count = int(groups.get("count") or 1)
                y = moe(h, w[p + "mlp.router"], w[p + "mlp.correction"], experts, n_id,
                        count, int(groups.get("keep") or count), int(r["top"]), rnd)
            x = x + rms_norm(y, w[p + "norm2b"], eps)
        after.append(x)
    logits = rnd(rms_norm(x, w["final.norm"], eps)) @ w["head"].T
    return (logits, torch.stack(after)) if keep_layers else logits


def greedy_generate(config, weights, prompt, n_new):
    """``n_new`` tokens, each the largest logit at the last place (the whole sequence is run again for
    every token: slow and plain)."""
    tokens = list(prompt)
    for _ in range(n_new):
        tokens.append(int(torch.argmax(forward(config, weights, tokens)[-1])))
    return tokens[len(prompt):]
