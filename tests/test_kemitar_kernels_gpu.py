"""The mechanisms Kemitar brought to the engine, each alone: the kernel (or the part) against the
function of ``plain_kemitar`` that states the same mechanism, on hand-made batches whose segments
start at position 0, in the middle of a sequence and on single tokens, over shuffled pages."""
import math

import numpy as np
import pytest
import torch

import plain_kemitar as P

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)
F64 = torch.float64


def dev(t, dtype=None):
    return t.to(device=DEV, dtype=dtype or t.dtype).contiguous()


def close(got, want, rel, what=""):
    got, want = got.detach().cpu().to(F64), want.detach().cpu().to(F64)
    assert got.shape == want.shape, f"{what}: {tuple(got.shape)} vs {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite"
    scale = max(1.0, float(want.abs().max()))
    worst = float((got - want).abs().max())
    assert worst <= rel * scale, f"{what}: max|delta| {worst:.3e} > {rel:.1e} * {scale:.3g}"


def bf16_round(t):
    return t.to(torch.bfloat16).to(F64)


def make_batch(cached, new, tokens=None, table=None, slots=None):
    """Segment s holds cached[s] tokens after the step, the last new[s] brought by it, in state slot
    ``slots[s]`` (default: ``len - 1 - s``, so that slots and segments differ)."""
    from flyweight_b200.engine import Segment, StepBatch
    S = len(cached)
    segments = []
    for s, (n, m) in enumerate(zip(cached, new)):
        ids = [0] * m if tokens is None else tokens[s][n - m:n]
        segments.append(Segment(f"s{s}", S - 1 - s if slots is None else slots[s], n - m, list(ids), []))
    tables = [table.tolist()] if table is not None else [[[0]] * S]
    return StepBatch(segments, tables, DEV)


# ------------------------------------------------------------------ embedding with hashed pairs
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("buckets,mul_prev,mul_cur", [(97, 31, 5), (1, 1, 1), (300, 65537, 40009)])
def test_hashed_pair_embedding(dtype, buckets, mul_prev, mul_cur):
    from flyweight_b200.kernels import latent
    g = torch.Generator().manual_seed(1)
    V, W, scale = 301, 72, 2.5
    table = torch.randn(V, W, generator=g, dtype=F64)
    pairs = torch.randn(buckets + 1, W, generator=g, dtype=F64)
    if dtype == torch.bfloat16:
        table, pairs = bf16_round(table), bf16_round(pairs)
    cfg = {"embedding": {"scale": scale, "bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}}}
    seqs = [[int(t) for t in torch.randint(0, V, (n,), generator=g)] for n in (9, 6, 1, 4)]
    want = [P.embed(seq, {"embed": table, "bigram": pairs}, cfg) for seq in seqs]
    state = torch.full((4, 1), -7, dtype=torch.int32, device=DEV)
    # step 1: a whole short sequence, the head of the others; step 2: the rest (one a single token)
    first = [5, 2, 1, 3]
    for cached, new in ((first, first), ([9, 6, 1, 4], [4, 4, 0, 1])):
        keep = [s for s in range(4) if new[s] > 0]
        batch = make_batch([cached[s] for s in keep], [new[s] for s in keep], [seqs[s] for s in keep],
                           slots=[3 - s for s in keep])
        out = latent.embed_pair_hash(dev(table, dtype), dev(pairs, dtype), batch, state, buckets, mul_prev,
                                     mul_cur, None, scale)
        at = 0
        for s in keep:
            n, m = cached[s], new[s]
            close(out[at:at + m], want[s][n - m:n], 1e-6, f"sequence {s}")
            at += m
            assert int(state[3 - s]) == seqs[s][n - 1]


def test_hashed_pair_rows_with_large_multipliers():
    """The row index is computed without overflow: products near 2^47."""
    from flyweight_b200.kernels import latent
    V, W, buckets, mul_prev, mul_cur = 2 ** 20, 8, 521, 2 ** 27 - 39, 2 ** 26 + 15
    seq = [V - 1, V - 2, 12345, V - 1, 0, 7]
    table = torch.zeros(V, W, dtype=torch.float32)
    pairs = torch.arange(buckets + 1, dtype=torch.float32)[:, None].expand(buckets + 1, W).contiguous()
    batch = make_batch([len(seq)], [len(seq)], [seq])
    state = torch.zeros((1, 1), dtype=torch.int32, device=DEV)
    out = latent.embed_pair_hash(dev(table), dev(pairs), batch, state, buckets, mul_prev, mul_cur, None, 1.0)
    assert out[:, 0].cpu().tolist() == [float(r) for r in P.hashed_pair_rows(seq, buckets, mul_prev, mul_cur)]


# ------------------------------------------------------------------ token shift
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W", [80, 82, 1030])
def test_token_shift_over_portions(out_dtype, W):
    from flyweight_b200.kernels import latent
    g = torch.Generator().manual_seed(2)
    mu = torch.rand(W, generator=g, dtype=F64) * 1.4 - 0.2
    seqs = [torch.randn(n, W, generator=g, dtype=F64).to(torch.float32).to(F64) for n in (7, 2, 1, 5)]
    want = [P.token_shift(x, mu.to(torch.float32).to(F64)) for x in seqs]
    state = torch.full((4, W), float("nan"), dtype=torch.float32, device=DEV)    # position 0 must not read it
    rel = 1e-6 if out_dtype == torch.float32 else 2.0 ** -8
    for cached, new in (([3, 1, 1, 2], [3, 1, 1, 2]), ([5, 2, 1, 4], [2, 1, 0, 2]), ([7, 2, 1, 5], [2, 0, 0, 1])):
        keep = [s for s in range(4) if new[s] > 0]
        batch = make_batch([cached[s] for s in keep], [new[s] for s in keep], slots=[3 - s for s in keep])
        x = torch.cat([seqs[s][cached[s] - new[s]:cached[s]] for s in keep]).to(torch.float32)
        out = latent.token_shift(dev(x), dev(mu, torch.float32), state, batch, out_dtype)
        at = 0
        for s in keep:
            n, m = cached[s], new[s]
            close(out[at:at + m], want[s][n - m:n], rel, f"sequence {s} rows {n - m}..{n}")
            at += m
            close(state[3 - s], seqs[s][n - 1], 0.0, "the kept row")


# ------------------------------------------------------------------ x += g * unit(y)
@pytest.mark.parametrize("W", [80, 82, 3000])
def test_gain_only_norm_adds_into_the_stream(W):
    from flyweight_b200.kernels import latent
    g = torch.Generator().manual_seed(3)
    x = torch.randn(5, W, generator=g, dtype=torch.float32)
    y = torch.randn(5, W, generator=g, dtype=torch.float32) * torch.tensor([1e-3, 1.0, 50.0, 0.0, 1.0])[:, None]
    gain, eps = torch.tensor([1.7], dtype=torch.float32), 1e-5
    want = x.to(F64) + P.unit_rms(y.to(F64), eps) * float(gain)
    xd = dev(x)
    copy = latent.unit_rms_gain_add_(xd, dev(y), dev(gain), eps, torch.bfloat16)
    close(xd, want, 1e-6, "the stream")
    close(copy, want, 2.0 ** -8, "its rounded copy")
    assert latent.unit_rms_gain_add_(dev(x), dev(y), dev(gain), eps, None) is None


# ------------------------------------------------------------------ latent attention, the part
def latent_spec(heads, dim, rot, vdim, rank, base, scale, hidden, shares=False, sink=True):
    from flyweight_b200.config.spec import PartSpec
    tensors = {"q": "q", "uk": "uk", "uv": "uv", "o": "o", "sink": "sink"}
    if not shares:
        tensors.update({"dkv": "dkv", "dkv_norm": "dkv.norm"})
    return PartSpec("latent_attention",
                    {"hidden_size": hidden, "num_heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim,
                     "kv_rank": rank, "scale": scale, "eps": 1e-5, "sink": sink, "shares_cache": shares,
                     "position": PartSpec("rope", {"theta": base, "rotary_dim": rot, "pairing": "half_split"})},
                    tensors)


def plain_names(w):
    """The plain implementation's names for a part's tensors (layer 0)."""
    return {"l0.mix." + name: value for name, value in w.items()}


def run_mixer(spec, w, dtype, h_seqs, cuts, n_pages=12, shuffle_seed=0):
    """The part over several sequences, fed in the portions ``cuts`` (a list of steps, each a list of
    (sequence, new tokens) pairs), pages handed out in a shuffled order.  Returns outputs by sequence."""
    from flyweight_b200.engine import Segment, StepBatch, StepContext
    from flyweight_b200.parts import Precision, build_mixer
    name = "float32" if dtype == torch.float32 else "bfloat16"
    precision = Precision(name)
    part = build_mixer(spec)
    part.bind(lambda n: w[n].to(dtype), precision, DEV)
    part.prepare(1024, DEV)
    kv = part.state_spec()
    pool = torch.full((n_pages, 1, 64, kv.head_dim), float("nan"), dtype=precision.cache_dtype, device=DEV)
    order = torch.randperm(n_pages, generator=torch.Generator().manual_seed(shuffle_seed)).tolist()
    pages = {s: [] for s in range(len(h_seqs))}
    done = {s: 0 for s in range(len(h_seqs))}
    outs = {s: [] for s in range(len(h_seqs))}
    cache = type("Cache", (), {})()
    cache.k_pool, cache.v_pool, cache.group, cache.state = pool, None, 0, None
    for step in cuts:
        segments, rows = [], []
        for s, m in step:
            while len(pages[s]) * 64 < done[s] + m:
                pages[s].append(order.pop())
            segments.append(Segment(f"s{s}", s, done[s], [0] * m, []))
        width = max(len(pages[s]) for s, _ in step)
        table = [pages[s] + [-1] * (width - len(pages[s])) for s, _ in step]
        batch = StepBatch(segments, [table], DEV)
        h = torch.cat([h_seqs[s][done[s]:done[s] + m] for s, m in step]).to(precision.act_dtype)
        out = part.forward(StepContext(batch, precision, DEV), dev(h), cache)
        at = 0
        for s, m in step:
            outs[s].append(out[at:at + m].float().cpu())
            at += m
            done[s] += m
    return {s: torch.cat(parts) for s, parts in outs.items() if parts}, pool, pages


def mixer_weights(heads, dim, rot, vdim, rank, hidden, seed, dtype):
    g = torch.Generator().manual_seed(seed)

    def matrix(rows, cols):
        return torch.randn(rows, cols, generator=g, dtype=F64) / math.sqrt(cols)

    w = {"q": matrix(heads * (dim + rot), hidden), "dkv": matrix(rank + rot, hidden),
         "dkv.norm": 1.0 + 0.1 * torch.randn(rank, generator=g, dtype=F64),
         "uk": matrix(heads * dim, rank), "uv": matrix(heads * vdim, rank), "o": matrix(hidden, heads * vdim),
         "sink": 2.0 * torch.randn(heads, generator=g, dtype=F64)}
    if dtype == torch.bfloat16:
        w = {k: bf16_round(v) for k, v in w.items()}
    return w


SHAPES = [  # heads, dim, rot, vdim, rank, hidden
    (3, 24, 8, 16, 40, 80),
    (1, 10, 6, 12, 37, 82),
    (20, 16, 16, 8, 48, 96),
    (6, 32, 32, 48, 88, 128),
    (4, 16, 32, 16, 144, 64),
]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_attention_whole_cut_and_one_by_one(shape, dtype):
    heads, dim, rot, vdim, rank, hidden = shape
    base, scale = 500.0, 1.0 / math.sqrt(dim + rot)
    w = mixer_weights(heads, dim, rot, vdim, rank, hidden, seed=sum(shape), dtype=dtype)
    m = {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": rank, "scale": scale,
         "rot": {"base": base, "dims": rot}}
    g = torch.Generator().manual_seed(7)
    lengths = (150, 67, 1)
    h_seqs = [torch.randn(n, hidden, generator=g, dtype=F64) for n in lengths]
    if dtype == torch.bfloat16:
        h_seqs = [bf16_round(h) for h in h_seqs]
    pw = plain_names(w)
    want = []
    for h in h_seqs:
        latent, key_rot = P.latent_and_rotated_key(h, pw, "l0.", m, 1e-5)
        want.append(P.latent_attention(h, pw, "l0.", m, latent, key_rot))
    spec = latent_spec(heads, dim, rot, vdim, rank, base, scale, hidden)
    rel = 2e-5 if dtype == torch.float32 else 12 * 2.0 ** -9
    whole = [[(0, 150), (1, 67), (2, 1)]]
    cut = [[(0, 63)], [(0, 2), (1, 64)], [(1, 1), (0, 62)], [(0, 1), (1, 2), (2, 1)], [(0, 22)]]
    single = [[(1, 1)] for _ in range(67)]
    for what, cuts in (("whole", whole), ("cut", cut), ("one by one", single)):
        got, pool, pages = run_mixer(spec, w, dtype, h_seqs, cuts, shuffle_seed=len(cuts))
        for s, out in got.items():
            close(out, want[s][:out.shape[0]], rel, f"{what}: sequence {s}")
    # what the cache holds: the normed latent and the turned key part, nothing per head
    latent, key_rot = P.latent_and_rotated_key(h_seqs[1], pw, "l0.", m, 1e-5)
    rows = torch.cat([pool[p, 0] for p in pages[1]])[:67].float().cpu()
    close(rows[:, :rank], latent, 1e-5 if dtype == torch.float32 else 2.0 ** -7, "cached latent")
    close(rows[:, rank:rank + rot], key_rot, 1e-5 if dtype == torch.float32 else 2.0 ** -7, "cached key part")
    assert float(rows[:, rank + rot:].abs().sum()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_layer_that_reads_another_layers_rows(dtype):
    """Own queries and per-head projections over rows that another layer's projection wrote."""
    heads, dim, rot, vdim, rank, hidden = 5, 16, 8, 24, 40, 80
    base, scale = 1000.0, 0.2
    own = mixer_weights(3, 24, rot, 16, rank, hidden, seed=1, dtype=dtype)
    other = mixer_weights(heads, dim, rot, vdim, rank, hidden, seed=2, dtype=dtype)
    g = torch.Generator().manual_seed(9)
    h0 = torch.randn(90, hidden, generator=g, dtype=F64)
    h1 = torch.randn(90, hidden, generator=g, dtype=F64)
    if dtype == torch.bfloat16:
        h0, h1 = bf16_round(h0), bf16_round(h1)
    m0 = {"heads": 3, "dim": 24, "rot_dim": rot, "vdim": 16, "kv_rank": rank, "scale": scale,
          "rot": {"base": base, "dims": rot}}
    m1 = dict(m0, heads=heads, dim=dim, vdim=vdim)
    latent, key_rot = P.latent_and_rotated_key(h0, plain_names(own), "l0.", m0, 1e-5)
    want = P.latent_attention(h1, plain_names(other), "l0.", m1, latent, key_rot)
    from flyweight_b200.engine import Segment, StepBatch, StepContext
    from flyweight_b200.parts import Precision, build_mixer
    precision = Precision("float32" if dtype == torch.float32 else "bfloat16")
    writer = build_mixer(latent_spec(3, 24, rot, 16, rank, base, scale, hidden))
    reader = build_mixer(latent_spec(heads, dim, rot, vdim, rank, base, scale, hidden, shares=True))
    assert reader.state_spec() is None and "dkv" not in reader.declare()
    writer.bind(lambda n: own[n].to(dtype), precision, DEV)
    reader.bind(lambda n: other[n].to(dtype), precision, DEV)
    writer.prepare(256, DEV)
    reader.prepare(256, DEV)
    cache = type("Cache", (), {})()
    cache.k_pool = torch.full((4, 1, 64, writer.state_spec().head_dim), float("nan"), dtype=precision.cache_dtype,
                              device=DEV)
    cache.v_pool, cache.group, cache.state = None, 0, None
    outs, done = [], 0
    for n in (70, 1, 19):
        batch = StepBatch([Segment("a", 0, done, [0] * n, [])], [[[2, 0]]], DEV)
        ctx = StepContext(batch, precision, DEV)
        writer.forward(ctx, dev(h0[done:done + n], precision.act_dtype), cache)
        outs.append(reader.forward(ctx, dev(h1[done:done + n], precision.act_dtype), cache).float().cpu())
        done += n
    close(torch.cat(outs), want, 2e-5 if dtype == torch.float32 else 12 * 2.0 ** -9, "reader")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("far,n", [(0, 600), (1, 600), (63, 600), (64, 600), (65, 600), (127, 600), (128, 600),
                                   (300, 600), (511, 600), (512, 600), (599, 600), (0, 1), (0, 2), (1, 2), (62, 63),
                                   (63, 64), (0, 64), (63, 65), (64, 65), (127, 128), (128, 129), (64, 129)])
def test_one_key_that_stands_out_is_found_wherever_it_lies(dtype, far, n):
    """Random scores hide a lost key among hundreds: here the query at the end matches one key far
    more than any other, so the output is that key's value unless the key was skipped -- at a page's
    first and last row, in the first page, in the last, for a prompt and for a decoded token."""
    from flyweight_b200.kernels import latent
    heads, rank, rot, row = 6, 48, 16, 64
    g = torch.Generator().manual_seed(far + n)
    keys = torch.randn(n, row, generator=g, dtype=F64) * 0.3
    keys[:, rank + rot:] = 0
    query = torch.randn(heads, row, generator=g, dtype=F64) * 0.3
    query[:, rank + rot:] = 0
    keys[far, :rank + rot] = 4.0 * query[2, :rank + rot] / query[2, :rank + rot].norm()   # head 2 looks for `far`
    query[2] *= 6.0 / query[2].norm()
    if dtype == torch.bfloat16:
        keys, query = bf16_round(keys), bf16_round(query)
    sink = torch.tensor([0.5, -1.0, 0.0, 3.0, -4.0, 1.0], dtype=F64)
    scale = 1.0
    scores = (query @ keys.T) * scale                                   # [heads][n]
    top = torch.maximum(scores.max(dim=1).values, sink)
    p = torch.exp(scores - top[:, None])
    want = (p @ keys[:, :rank]) / (p.sum(dim=1) + torch.exp(sink - top))[:, None]
    assert float((want[2] - keys[far, :rank]).abs().max()) < 0.05 * float(keys[far, :rank].abs().max())
    order = torch.randperm(12, generator=g).tolist()
    pages = order[:10]
    pool = torch.full((12, 1, 64, row), float("nan"), dtype=F64)
    for i, page in enumerate(pages):
        chunk = keys[i * 64:(i + 1) * 64]
        pool[page, 0, :chunk.shape[0]] = chunk
    table = torch.tensor([pages[:max(1, -(-n // 64))]], dtype=torch.int32)
    rel = 1e-5 if dtype == torch.float32 else 2.0 ** -7
    for new in sorted({1, min(40, n)}):   # the last token alone (decoding), and as the last of a portion
        batch = make_batch([n], [new], table=table)
        qa = torch.zeros(new, heads, row, dtype=F64)
        qa[-1] = query
        out = latent.latent_attention(dev(qa, dtype), dev(pool, dtype), dev(sink, torch.float32), batch,
                                      batch.block_tables[0], rank, rank + rot, scale)
        close(out.view(new, heads, -1)[-1, :, :rank], want, rel, f"key {far}, {new} new tokens")
        if dtype == torch.bfloat16:
            # the same through the paged attention kernels (the row is key and value at once)
            from flyweight_b200.engine import StepContext
            from flyweight_b200.kernels import attention
            cache = type("Cache", (), {})()
            cache.k_pool, cache.v_pool = dev(pool, dtype), None
            for tiled in (False, True):
                attention.force_tiled(tiled)
                try:
                    out = attention.paged_attention(StepContext(batch, None, DEV), dev(qa, dtype).view(new, -1), cache,
                                                    batch.block_tables[0], heads, 0, scale, dtype,
                                                    sink=dev(sink, torch.float32))
                finally:
                    attention.force_tiled(False)
                close(out.view(new, heads, -1)[-1, :, :rank], want, rel, f"key {far}, {new} new tokens, paged")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_sink_counts_once_and_is_not_scaled(dtype):
    """A single key: the weight is exp(s) / (exp(s) + exp(sink)) with s scaled and the sink not."""
    from flyweight_b200.kernels import latent
    heads, rank, rot, row = 3, 16, 0, 16
    key = torch.ones(1, row, dtype=F64)
    query = torch.stack([torch.full((row,), v, dtype=F64) for v in (0.25, -0.5, 1.0)])
    sink = torch.tensor([2.0, -1.0, 30.0], dtype=F64)
    scale = 0.125
    s = (query @ key.T)[:, 0] * scale
    weight = torch.exp(s) / (torch.exp(s) + torch.exp(sink))
    pool = torch.zeros(2, 1, 64, row, dtype=F64)
    pool[1, 0, 0] = key
    batch = make_batch([1], [1], table=torch.tensor([[1]], dtype=torch.int32))
    out = latent.latent_attention(dev(query[None], dtype), dev(pool, dtype), dev(sink, torch.float32), batch,
                                  batch.block_tables[0], rank, rank + rot, scale)
    close(out.view(heads, -1)[:, :rank], weight[:, None].expand(heads, rank), 1e-6 if dtype == torch.float32 else 2.0 ** -8)
    none = latent.latent_attention(dev(query[None], dtype), dev(pool, dtype), None, batch,
                                   batch.block_tables[0], rank, rank + rot, scale)
    close(none.view(heads, -1)[:, :rank], torch.ones(heads, rank, dtype=F64), 1e-6 if dtype == torch.float32 else 2.0 ** -8)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,heads,N,K", [(1, 3, 40, 24), (70, 20, 48, 16), (5, 1, 37, 10), (130, 8, 96, 32),
                                         (9, 4, 16, 144)])
def test_per_head_products(dtype, T, heads, N, K):
    from flyweight_b200.kernels import latent
    g = torch.Generator().manual_seed(T)
    x_head, y_head, x_col, y_col = K + 6, N + 2, 4, 2
    x = torch.randn(T, x_col + heads * x_head, generator=g, dtype=F64)
    w = torch.randn(heads, N, K, generator=g, dtype=F64) / math.sqrt(K)
    if dtype == torch.bfloat16:
        x, w = bf16_round(x), bf16_round(w)
    y = torch.full((T, y_col + heads * y_head + 3), 7.0, dtype=dtype, device=DEV)
    latent.head_linear(dev(x, dtype), x_col, x_head, K, dev(w, dtype), y, y_col, y_head)
    xs = x[:, x_col:].reshape(T, heads, x_head)[:, :, :K]
    want = torch.einsum("thk,hnk->thn", xs, w)
    got = y[:, y_col:y_col + heads * y_head].reshape(T, heads, y_head).float().cpu()
    close(got[:, :, :N], want, 1e-5 if dtype == torch.float32 else 2.0 ** -7, "products")
    assert float((got[:, :, N:] - 7.0).abs().max()) == 0.0 and float((y[:, :y_col].float() - 7.0).abs().max()) == 0.0


@pytest.mark.parametrize("heads,row", [(8, 128), (20, 64), (17, 48), (40, 128), (128, 64), (12, 96), (6, 80)])
@pytest.mark.parametrize("new", [1, 3, 70, 200])
def test_paged_attention_with_a_sink_and_one_shared_pool_head(heads, row, new):
    """Many query heads over one pool head whose rows are keys and values, with a sink per head: the
    tensor-core kernels (decode, tiled, tcgen05 -- whichever the step's shape selects) against the
    softmax written out."""
    from flyweight_b200.engine import StepContext
    from flyweight_b200.kernels import attention
    g = torch.Generator().manual_seed(heads + new)
    cached = [330, new, 129 + new]
    news = [new, new, 1]
    scale = 0.3
    seqs = [bf16_round(torch.randn(n, row, generator=g, dtype=F64) * 0.7) for n in cached]
    sink = torch.randn(heads, generator=g, dtype=F64) * 2.0
    order = torch.randperm(20, generator=g).tolist()
    pool = torch.full((20, 1, 64, row), float("nan"), dtype=F64)
    table = torch.full((3, 6), -1, dtype=torch.int32)
    for s, keys in enumerate(seqs):
        for i in range(-(-keys.shape[0] // 64)):
            page = order.pop()
            table[s, i] = page
            chunk = keys[i * 64:(i + 1) * 64]
            pool[page, 0, :chunk.shape[0]] = chunk
    # single tokens lead the batch, as the scheduler orders a mixed step
    idx = [2, 0, 1]
    batch = make_batch([cached[i] for i in idx], [news[i] for i in idx], table=table[idx])
    q = bf16_round(torch.randn(sum(news), heads, row, generator=g, dtype=F64))
    cache = type("Cache", (), {})()
    cache.k_pool, cache.v_pool = dev(pool, torch.bfloat16), None
    out = attention.paged_attention(StepContext(batch, None, DEV), dev(q, torch.bfloat16).view(sum(news), -1), cache,
                                    batch.block_tables[0], heads, 0, scale, torch.bfloat16,
                                    sink=dev(sink, torch.float32)).view(sum(news), heads, row).float().cpu().to(F64)
    at = 0
    for i in idx:
        keys, n, m = seqs[i], cached[i], news[i]
        for j in range(m):
            pos = n - m + j
            scores = (q[at + j] @ keys[:pos + 1].T) * scale                 # [heads][pos + 1]
            top = torch.maximum(scores.max(dim=1).values, sink)
            p = torch.exp(scores - top[:, None])
            want = (p @ keys[:pos + 1]) / (p.sum(dim=1) + torch.exp(sink - top))[:, None]
            close(out[at + j], want, 2.0 ** -7, f"sequence {i} position {pos}")
        at += m


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("at", [0, 5, 62, 63, 64, 100])
def test_a_key_behind_the_query_is_not_seen(dtype, at):
    """Inside one portion the query of token ``at`` matches the key of token ``at + 1`` far more than any
    other: a kernel that let it look ahead would return that key's value."""
    from flyweight_b200.engine import StepContext
    from flyweight_b200.kernels import attention, latent
    heads, rank, rot, row, n = 4, 48, 16, 64, 130
    g = torch.Generator().manual_seed(at)
    keys = torch.randn(n, row, generator=g, dtype=F64) * 0.3
    keys[:, rank + rot:] = 0
    query = torch.randn(heads, row, generator=g, dtype=F64) * 0.3
    query[:, rank + rot:] = 0
    query[1] *= 6.0 / query[1].norm()
    keys[at + 1, :rank + rot] = 4.0 * query[1, :rank + rot] / query[1, :rank + rot].norm()
    if dtype == torch.bfloat16:
        keys, query = bf16_round(keys), bf16_round(query)
    sink = torch.tensor([0.0, -2.0, 1.0, 0.5], dtype=F64)
    scores = query @ keys[:at + 1].T
    top = torch.maximum(scores.max(dim=1).values, sink)
    p = torch.exp(scores - top[:, None])
    want = (p @ keys[:at + 1, :rank]) / (p.sum(dim=1) + torch.exp(sink - top))[:, None]
    pool = torch.full((4, 1, 64, row), float("nan"), dtype=F64)
    for i, page in enumerate((2, 0, 3)):
        chunk = keys[i * 64:(i + 1) * 64]
        pool[page, 0, :chunk.shape[0]] = chunk
    batch = make_batch([n], [n], table=torch.tensor([[2, 0, 3]], dtype=torch.int32))
    qa = torch.zeros(n, heads, row, dtype=F64)
    qa[at] = query
    rel = 1e-5 if dtype == torch.float32 else 2.0 ** -7
    out = latent.latent_attention(dev(qa, dtype), dev(pool, dtype), dev(sink, torch.float32), batch,
                                  batch.block_tables[0], rank, rank + rot, 1.0)
    close(out.view(n, heads, -1)[at, :, :rank], want, rel, f"query {at}")
    if dtype == torch.bfloat16:
        cache = type("Cache", (), {})()
        cache.k_pool, cache.v_pool = dev(pool, dtype), None
        for tiled in (False, True):
            attention.force_tiled(tiled)
            try:
                out = attention.paged_attention(StepContext(batch, None, DEV), dev(qa, dtype).view(n, -1), cache,
                                                batch.block_tables[0], heads, 0, 1.0, dtype,
                                                sink=dev(sink, torch.float32))
            finally:
                attention.force_tiled(False)
            close(out.view(n, heads, -1)[at, :, :rank], want, rel, f"query {at}, paged")


@pytest.mark.parametrize("heads,row,n", [(8, 128, 9000), (20, 64, 12000)])
def test_a_long_context_cut_into_more_slices_than_a_cluster_holds(heads, row, n):
    """One decoded token over thousands of rows: the context is cut into more than eight slices, which are
    merged by the kernel of their own; the sink must still count once."""
    from flyweight_b200.engine import StepContext
    from flyweight_b200.kernels import attention
    g = torch.Generator().manual_seed(n)
    keys = bf16_round(torch.randn(n, row, generator=g, dtype=F64) * 0.5)
    q = bf16_round(torch.randn(1, heads, row, generator=g, dtype=F64))
    sink = torch.randn(heads, generator=g, dtype=F64) * 3.0 + 4.0      # heavy sinks: counted twice, they would show
    n_pages = -(-n // 64)
    order = torch.randperm(n_pages + 3, generator=g).tolist()[:n_pages]
    pool = torch.full((n_pages + 3, 1, 64, row), float("nan"), dtype=F64)
    for i, page in enumerate(order):
        chunk = keys[i * 64:(i + 1) * 64]
        pool[page, 0, :chunk.shape[0]] = chunk
    batch = make_batch([n], [1], table=torch.tensor([order], dtype=torch.int32))
    groups = attention.head_groups(heads, 1)
    splits, _, in_cluster = attention.decode_splits(1, groups, n_pages, row)
    assert splits > 8 and not in_cluster
    cache = type("Cache", (), {})()
    cache.k_pool, cache.v_pool = dev(pool, torch.bfloat16), None
    scale = 0.2
    out = attention.paged_attention(StepContext(batch, None, DEV), dev(q, torch.bfloat16).view(1, -1), cache,
                                    batch.block_tables[0], heads, 0, scale, torch.bfloat16,
                                    sink=dev(sink, torch.float32)).view(heads, row).float().cpu().to(F64)
    scores = (q[0] @ keys.T) * scale
    top = torch.maximum(scores.max(dim=1).values, sink)
    p = torch.exp(scores - top[:, None])
    want = (p @ keys) / (p.sum(dim=1) + torch.exp(sink - top))[:, None]
    close(out, want, 2.0 ** -7, "one token over a long context")
