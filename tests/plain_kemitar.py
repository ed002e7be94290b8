"""A plain, slow Kemitar forward pass in float64 torch: whole sequences, no cache, no batching,
one function for each mechanism.  It imports nothing from the ``flyweight_b200`` package and is
what the tests compare the engine with.

Kemitar in short (a decoder-only model):

* embedding: ``embed[t_n] * s`` plus one row of a hashed table of token pairs, row
  ``(t_{n-1} * a + t_n * b) mod B`` (row ``B``, the table's last, for a sequence's first token);
* every layer adds its sublayers' outputs *after* a norm: ``x += g1 * unit(mixer(shift(x)))`` and
  ``x += g2 * unit(ff(x))`` with ``unit(y) = y / sqrt(mean(y^2) + eps)`` and g a single number;
  the sublayers read the stream itself (no norm in front);
* token shift: the mixer reads ``x_n + (x_{n-1} - x_n) * mu`` (``x_{-1} = 0``), mu per channel;
* mixer: attention over a low-rank latent.  One projection gives per token a latent ``c`` (RMS-normed
  with a weight) and one rotated key part shared by every head; per head the unrotated key and the
  value are projections of ``c``; queries have an unrotated and a rotated part; causal softmax whose
  denominator also holds ``exp(sink_h)``; a layer may read an earlier layer's latent and rotated key;
* feed-forward: ``down(silu(gate x) * up x)``;
* output: ``g * unit(x)`` and the head.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

F64 = torch.float64


def same(value):
    return value


def bf16(value):
    """Round to bfloat16 and widen again: what a 16-bit engine does to the results of its products."""
    return value.to(torch.bfloat16).to(F64)


# ------------------------------------------------------------------ files
def read_safetensors(path) -> dict:
    """Every tensor of a safetensors file widened to float64 (8-byte length, JSON header, data)."""
    raw = np.fromfile(str(path), dtype=np.uint8)
    (header_len,) = struct.unpack("<Q", raw[:8].tobytes())
    header = json.loads(raw[8:8 + header_len].tobytes())
    base = 8 + header_len
    out = {}
    for name, entry in header.items():
        if name == "__metadata__":
            continue
        begin, end = entry["data_offsets"]
        blob = raw[base + begin:base + end]
        kind = entry["dtype"]
        if kind == "F32":
            tensor = torch.from_numpy(blob.view("<f4").copy())
        elif kind == "BF16":
            tensor = (torch.from_numpy(blob.view("<u2").astype(np.int32)) << 16).view(torch.float32)
        else:
            raise ValueError(f"plain reader: unsupported dtype {kind} for {name}")
        out[name] = tensor.to(F64).reshape(tuple(entry["shape"]))
    return out


def load_model_dir(path):
    path = Path(path)
    return json.loads((path / "config.json").read_text()), read_safetensors(path / "model.safetensors")


# ------------------------------------------------------------------ mechanisms
def unit_rms(y, eps):
    """y / sqrt(mean(y^2) + eps) over the last axis."""
    return y / torch.sqrt((y * y).mean(dim=-1, keepdim=True) + eps)


def hashed_pair_rows(tokens, buckets, mul_prev, mul_cur):
    """Row of the pair table for every token of one sequence."""
    rows = []
    for n, token in enumerate(tokens):
        rows.append(buckets if n == 0 else (int(tokens[n - 1]) * mul_prev + int(token) * mul_cur) % buckets)
    return rows


def embed(tokens, w, cfg):
    e = cfg["embedding"]
    x = w["embed"][list(tokens)] * float(e["scale"])
    pair = e.get("bigram")
    if pair is not None:
        x = x + w["bigram"][hashed_pair_rows(tokens, int(pair["buckets"]), int(pair["mul_prev"]),
                                             int(pair["mul_cur"]))]
    return x


def token_shift(x, mu):
    """x_n + (x_{n-1} - x_n) * mu, zeros in front of the first token."""
    before = torch.cat([torch.zeros_like(x[:1]), x[:-1]], dim=0)
    return x + (before - x) * mu


def rotate_half_split(v, positions, base, dims):
    """The first ``dims`` channels of the last axis turn: channel i pairs with i + dims/2, the pair
    (a, b) at position p becomes (a cos t - b sin t, b cos t + a sin t), t = p * base^(-2i/dims)."""
    half = dims // 2
    freq = torch.tensor(float(base), dtype=F64) ** (-2.0 * torch.arange(half, dtype=F64) / dims)
    angle = positions.to(F64)[:, None] * freq[None, :]
    cos, sin = torch.cos(angle), torch.sin(angle)
    while cos.dim() < v.dim():
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    a, b, rest = v[..., :half], v[..., half:dims], v[..., dims:]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, rest], dim=-1)


def latent_and_rotated_key(h, w, prefix, m, eps, rnd=same):
    """(latent [N][rank], rotated shared key part [N][rot_dim]) of the layer whose mixer is ``m``.
    ``rnd`` is applied to what a 16-bit engine would store in 16 bits (here and below)."""
    rank, rot_dim = int(m["kv_rank"]), int(m["rot_dim"])
    d = rnd(h @ w[prefix + "mix.dkv"].T)
    latent = rnd(unit_rms(d[:, :rank], eps) * w[prefix + "mix.dkv.norm"])
    positions = torch.arange(h.shape[0])
    key_rot = rnd(rotate_half_split(d[:, rank:rank + rot_dim], positions, m["rot"]["base"], int(m["rot"]["dims"])))
    return latent, key_rot


def softmax_with_sink(scores, sink):
    """Causal softmax over the last axis of [H][N][N] whose denominator also holds exp(sink_h)."""
    N = scores.shape[-1]
    mask = torch.ones(N, N, dtype=torch.bool).tril()
    scores = scores.masked_fill(~mask, -math.inf)
    top = torch.maximum(scores.max(dim=-1, keepdim=True).values, sink[:, None, None])
    weights = torch.exp(scores - top)
    return weights / (weights.sum(dim=-1, keepdim=True) + torch.exp(sink[:, None, None] - top))


def latent_attention(h, w, prefix, m, latent, key_rot, rnd=same):
    """The mixer of one layer over a whole sequence, keys and values from (latent, key_rot)."""
    H, dim, rot_dim, vdim, rank = (int(m[k]) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"))
    N = h.shape[0]
    q = rnd(h @ w[prefix + "mix.q"].T).reshape(N, H, dim + rot_dim)
    q_plain = q[..., :dim]
    q_rot = rnd(rotate_half_split(q[..., dim:], torch.arange(N), m["rot"]["base"], int(m["rot"]["dims"])))
    k_plain = rnd(latent @ w[prefix + "mix.uk"].T).reshape(N, H, dim)
    value = rnd(latent @ w[prefix + "mix.uv"].T).reshape(N, H, vdim)
    scores = (torch.einsum("nhd,mhd->hnm", q_plain, k_plain)
              + torch.einsum("nhr,mr->hnm", q_rot, key_rot)) * float(m["scale"])
    weights = softmax_with_sink(scores, w[prefix + "mix.sink"])
    out = rnd(torch.einsum("hnm,mhv->nhv", rnd(weights), value).reshape(N, H * vdim))
    return out @ w[prefix + "mix.o"].T


def gated_feed_forward(x, w, prefix, rnd=same):
    gate = x @ w[prefix + "mlp.gate"].T
    return rnd(gate * torch.sigmoid(gate) * (x @ w[prefix + "mlp.up"].T)) @ w[prefix + "mlp.down"].T


# ------------------------------------------------------------------ the model
def forward(cfg, w, tokens, return_layers: bool = False, rnd=same):
    """Logits [N][vocab] of one whole sequence (and the stream after every layer, if asked).
    ``rnd=bf16`` rounds what a 16-bit engine keeps in 16 bits (inputs and results of the products, not
    the stream, the norms or the softmax): the difference to ``rnd=same`` is the error that rounding
    alone causes, which the tests of the 16-bit path take their bound from."""
    eps = float(cfg["norm"]["eps"])
    x = embed(tokens, w, cfg)
    kept = {}                     # layer index -> (latent, rotated key part)
    after = []
    for index, layer in enumerate(cfg["layers"]):
        prefix = f"l{index}."
        if layer["type"] != "latent_attention":
            raise ValueError(f"plain Kemitar: unknown layer type {layer['type']!r}")
        m = layer["mixer"]
        h = rnd(token_shift(x, w[prefix + "shift"]))
        source = m.get("kv_from")
        if source is None:
            kept[index] = latent_and_rotated_key(h, w, prefix, m, eps, rnd)
            source = index
        x = x + unit_rms(latent_attention(h, w, prefix, m, *kept[int(source)], rnd=rnd), eps) * w[prefix + "norm1"]
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(f"plain Kemitar: unknown feed-forward {layer['mlp']['kind']!r}")
            x = x + unit_rms(gated_feed_forward(rnd(x), w, prefix, rnd), eps) * w[prefix + "norm2"]
        after.append(x.clone())
    logits = rnd(unit_rms(x, eps) * w["final.norm"]) @ w["head"].T
    return (logits, torch.stack(after)) if return_layers else logits


def greedy_generate(cfg, w, prompt, count):
    """Greedy continuation by re-running whole sequences (the lowest id among equal logits)."""
    tokens, out = list(prompt), []
    for _ in range(count):
        row = forward(cfg, w, tokens)[-1].numpy()
        nxt = int(np.lexsort((np.arange(row.size), -row))[0])
        out.append(nxt)
        tokens.append(nxt)
    return out
