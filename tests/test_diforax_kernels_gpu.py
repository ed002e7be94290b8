"""The mechanisms Diforax brought to the engine, each alone: the kernel (or the part) against the
function of ``plain_diforax`` that states the same mechanism, on hand-made batches whose segments start
at position 0, in the middle of a sequence and on single tokens, over shuffled pages and slots."""
import math

import pytest
import torch

import plain_diforax as P

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)
F64 = torch.float64
BOTH = [torch.float32, torch.bfloat16]


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


def matrix(g, rows, cols, dtype):
    m = torch.randn(rows, cols, generator=g, dtype=F64) / math.sqrt(cols)
    return bf16_round(m) if dtype == torch.bfloat16 else m.to(torch.float32).to(F64)


def precision_of(dtype):
    from flyweight_b200.parts import Precision
    return Precision("float32" if dtype == torch.float32 else "bfloat16")


class Feeder:
    """Feeds sequences to a part in steps of (sequence, new tokens) pairs: hands out pages in a shuffled
    order, keeps block tables and positions, and gives every sequence a state slot of its own."""

    def __init__(self, n_seqs, n_pages=24, seed=0, slots=None):
        self.order = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
        self.pages = {s: [] for s in range(n_seqs)}
        self.done = {s: 0 for s in range(n_seqs)}
        self.slots = slots or {s: n_seqs - 1 - s for s in range(n_seqs)}

    def batch(self, step):
        from flyweight_b200.engine import Segment, StepBatch
        segments = []
        for s, m in step:
            while len(self.pages[s]) * 64 < self.done[s] + m:
                self.pages[s].append(self.order.pop())
            segments.append(Segment(f"s{s}", self.slots[s], self.done[s], [0] * m, []))
        width = max(1, max(len(self.pages[s]) for s, _ in step))
        table = [self.pages[s] + [-1] * (width - len(self.pages[s])) for s, _ in step]
        return StepBatch(segments, [table], DEV)

    def advance(self, step):
        for s, m in step:
            self.done[s] += m


def run_part(part, precision, h_seqs, steps, cache, feeder=None, feed_forward=False):
    """Outputs by sequence of a mixer (or feed-forward) over ``steps``."""
    from flyweight_b200.engine import StepContext
    feeder = feeder or Feeder(len(h_seqs))
    outs = {s: [] for s in range(len(h_seqs))}
    for step in steps:
        batch = feeder.batch(step)
        h = torch.cat([h_seqs[s][feeder.done[s]:feeder.done[s] + m] for s, m in step]).to(precision.act_dtype)
        ctx = StepContext(batch, precision, DEV)
        out = part.forward(ctx, dev(h)) if feed_forward else part.forward(ctx, dev(h), cache)
        at = 0
        for s, m in step:
            outs[s].append(out[at:at + m].float().cpu())
            at += m
        feeder.advance(step)
    return {s: torch.cat(parts) for s, parts in outs.items() if parts}


def cuts_of(lengths, sizes):
    """Steps that feed sequences of the given lengths side by side in portions of ``sizes`` (cycled)."""
    done = [0] * len(lengths)
    steps, i = [], 0
    while any(d < n for d, n in zip(done, lengths)):
        step = []
        for s, n in enumerate(lengths):
            if done[s] < n:
                m = min(sizes[(i + s) % len(sizes)], n - done[s])
                step.append((s, m))
                done[s] += m
        steps.append(step)
        i += 1
    return steps


# ------------------------------------------------------------------ x += w * unit(y), and the next norm
@pytest.mark.parametrize("W", [80, 82, 3000])
@pytest.mark.parametrize("next_dtype", [None, torch.float32, torch.bfloat16])
def test_output_norm_adds_into_the_stream(W, next_dtype):
    from flyweight_b200.kernels import ops
    g = torch.Generator().manual_seed(W)
    x = torch.randn(7, W, generator=g, dtype=torch.float32)
    y = torch.randn(7, W, generator=g, dtype=torch.float32) * 3
    w = 1 + 0.1 * torch.randn(W, generator=g, dtype=torch.float32)
    w2 = 1 + 0.1 * torch.randn(W, generator=g, dtype=torch.float32)
    want_x = x.to(F64) + P.rms_norm(y.to(F64), w.to(F64), 1e-5)
    xd = dev(x)
    h = ops.rmsnorm_add_(xd, dev(y), dev(w), 1e-5, *(() if next_dtype is None else (dev(w2), 1e-6, next_dtype)))
    close(xd, want_x, 1e-6, "the stream")
    if next_dtype is None:
        assert h is None
    else:
        assert h.dtype == next_dtype
        close(h, P.rms_norm(want_x, w2.to(F64), 1e-6), 1e-6 if next_dtype == torch.float32 else 2.0 ** -8, "the next norm")


# ------------------------------------------------------------------ the gate's activation
@pytest.mark.parametrize("T", [1, 9, 70, 300])
def test_gelu_on_the_gate(T):
    from flyweight_b200.kernels import ops, tensorcore
    g = torch.Generator().manual_seed(T)
    F, K = 192, 128
    x = bf16_round(torch.randn(T, K, generator=g, dtype=F64))
    w = bf16_round(torch.randn(2 * F, K, generator=g, dtype=F64) / math.sqrt(K) * 3)
    gu = x @ w.T
    want = P.gelu_tanh(gu[:, :F]) * gu[:, F:]
    close(ops.gate_act_mul(dev(gu, torch.float32), torch.float32, "gelu_tanh"), want, 1e-6, "unfused")
    close(ops.gate_act_mul(dev(gu, torch.float32), torch.float32, "silu"), P.silu(gu[:, :F]) * gu[:, F:], 1e-6, "silu")
    fused = tensorcore.swiglu_gate_up(dev(x, torch.bfloat16), dev(w, torch.bfloat16), activation="gelu_tanh")
    close(fused, want, 2.0 ** -7, "in the product's epilogue")
    assert tensorcore.status() == 0


# ------------------------------------------------------------------ rotation, then unit root mean square
@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("heads,kv,dim,D,rot", [(6, 3, 32, 32, 16), (4, 1, 16, 48, 16), (2, 2, 64, 64, 32),
                                                (8, 2, 128, 128, 64), (3, 1, 24, 32, 0), (5, 5, 20, 32, 6)])
def test_rotation_then_unit_rms(dtype, heads, kv, dim, D, rot):
    """Heads of ``dim`` channels sit in rows of ``D`` (zero padding behind them): the mean of squares goes
    over ``dim``; queries, the key rows in their pages and the untouched value rows are checked."""
    from flyweight_b200.kernels import ops
    from flyweight_b200.parts.rope import Rope
    from flyweight_b200.config.spec import PartSpec
    g = torch.Generator().manual_seed(dim + rot)
    eps, T, pos0 = 1e-5, 9, 59
    raw = torch.randn(T, heads + 2 * kv, dim, generator=g, dtype=F64) * 2
    raw = bf16_round(raw) if dtype == torch.bfloat16 else raw.to(torch.float32).to(F64)
    positions = torch.arange(pos0, pos0 + T)
    want_q = P.rms_unit(P.rotate(raw[:, :heads], positions, 777.0, rot), eps)
    want_k = P.rms_unit(P.rotate(raw[:, heads:heads + kv], positions, 777.0, rot), eps)
    padded = torch.zeros(T, heads + 2 * kv, D, dtype=F64)
    padded[..., :dim] = raw
    table = Rope(PartSpec("rope", {"theta": 777.0, "rotary_dim": max(rot, 2)})).table(128, DEV) if rot else \
        torch.zeros((1, 1, 2), dtype=torch.float32, device=DEV)
    feeder = Feeder(1, n_pages=4, seed=dim)
    feeder.done[0] = pos0
    batch = feeder.batch([(0, T)])
    k_pool = torch.full((4, kv, 64, D), float("nan"), dtype=dtype, device=DEV)
    v_pool = torch.full_like(k_pool, float("nan"))
    q = ops.qk_norm_rope(dev(padded.view(T, -1), dtype), None, None, table, batch.positions, batch.tok_seg,
                         batch.block_tables[0], k_pool, v_pool, heads, kv, D, rot, eps, dtype,
                         unit_rms_after=True, norm_dim=dim)
    rel = 2e-6 if dtype == torch.float32 else 2.0 ** -8
    close(q.view(T, heads, D)[..., :dim], want_q, rel, "queries")
    assert float(q.view(T, heads, D)[..., dim:].float().abs().max() if D > dim else 0.0) == 0.0
    for i in range(T):
        page, row = feeder.pages[0][(pos0 + i) // 64], (pos0 + i) % 64
        close(k_pool[page, :, row, :dim], want_k[i], rel, f"key row of position {pos0 + i}")
        close(v_pool[page, :, row, :dim], raw[i, heads + kv:], 0.0 if dtype == torch.float32 else rel, "value row")


# ------------------------------------------------------------------ attention inside chunks: the part
def attention_spec(heads, kv, dim, vdim, chunk, rot, scale, hidden, shares=False):
    from flyweight_b200.config.spec import PartSpec
    tensors = {"q": "q", "o": "o"}
    if not shares:
        tensors.update({"k": "k", "v": "v"})
    position = PartSpec("rope", {"theta": 5000.0, "rotary_dim": rot}) if rot else PartSpec("no_position")
    return PartSpec("gqa_attention", {"hidden_size": hidden, "num_heads": heads, "num_kv_heads": kv, "head_dim": dim,
                                      "value_dim": vdim, "scale": scale, "qk_norm_eps": None, "qk_unit_rms_eps": 1e-5,
                                      "chunk": chunk, "shares_cache": shares, "position": position}, tensors)


def build_attention(spec, w, dtype, n_pages=24):
    from flyweight_b200.parts import build_mixer
    precision = precision_of(dtype)
    part = build_mixer(spec)
    part.bind(lambda n: w[n].to(dtype), precision, DEV)
    part.prepare(2048, DEV)
    cache = type("Cache", (), {})()
    kv = part.state_spec()
    cache.group, cache.state = 0, None
    if kv is not None:
        cache.k_pool = torch.full((n_pages, kv.n_kv_heads, 64, kv.head_dim), float("nan"), dtype=precision.cache_dtype, device=DEV)
        cache.v_pool = torch.full_like(cache.k_pool, float("nan"))
    return part, precision, cache


def plain_attention(h, w, heads, kv, dim, vdim, chunk, rot, scale, keys=None):
    positions = torch.arange(h.shape[0])
    if keys is None:
        keys = P.attention_keys(h, positions, w["k"], w["v"], kv, dim, vdim, 5000.0, rot, 1e-5)
    q = P.attention_queries(h, positions, w["q"], heads, dim, 5000.0, rot, 1e-5)
    return P.chunked_attention(q, positions, keys[0], keys[1], positions, scale, chunk) @ w["o"].T, keys


ATTENTION_SHAPES = [  # heads, kv, dim, vdim, chunk, rot, hidden
    (6, 3, 32, 16, 48, 16, 80), (4, 1, 16, 48, 64, 16, 96), (2, 2, 64, 64, 100, 32, 96),
    (8, 2, 128, 128, 130, 64, 128), (16, 4, 64, 64, 70, 64, 128), (3, 1, 24, 8, 5, 0, 72), (2, 1, 32, 32, 1, 32, 64),
]


@pytest.mark.parametrize("shape", ATTENTION_SHAPES)
@pytest.mark.parametrize("dtype", BOTH)
def test_chunked_attention_whole_cut_and_one_by_one(shape, dtype):
    heads, kv, dim, vdim, chunk, rot, hidden = shape
    g = torch.Generator().manual_seed(sum(shape))
    w = {"q": matrix(g, heads * dim, hidden, dtype), "k": matrix(g, kv * dim, hidden, dtype),
         "v": matrix(g, kv * vdim, hidden, dtype), "o": matrix(g, hidden, heads * vdim, dtype)}
    lengths = [300, 131, 1, 67]
    h_seqs = [torch.randn(n, hidden, generator=g, dtype=F64) for n in lengths]
    if dtype == torch.bfloat16:
        h_seqs = [bf16_round(h) for h in h_seqs]
    want = [plain_attention(h, w, heads, kv, dim, vdim, chunk, rot, 0.3)[0] for h in h_seqs]
    rel = 2e-5 if dtype == torch.float32 else 3 * 2.0 ** -7
    spec = attention_spec(heads, kv, dim, vdim, chunk, rot, 0.3, hidden)
    for name, sizes in (("whole", [1000]), ("cut", [3, 2, 64, 1, 33, 7, 128, 2]), ("one by one", [1])):
        if name == "one by one":
            lengths_now, seqs_now, want_now = lengths[1:], h_seqs[1:], want[1:]
        else:
            lengths_now, seqs_now, want_now = lengths, h_seqs, want
        part, precision, cache = build_attention(spec, w, dtype)
        got = run_part(part, precision, seqs_now, cuts_of(lengths_now, sizes), cache, Feeder(len(seqs_now), seed=len(name)))
        for s, wanted in enumerate(want_now):
            close(got[s], wanted, rel, f"{name}, sequence {s}")


@pytest.mark.parametrize("dtype", BOTH)
def test_a_layer_that_reads_another_layers_keys_under_its_own_chunk(dtype):
    heads, kv, dim, vdim, hidden = 6, 3, 32, 16, 80
    g = torch.Generator().manual_seed(5)
    w = {"q": matrix(g, heads * dim, hidden, dtype), "k": matrix(g, kv * dim, hidden, dtype),
         "v": matrix(g, kv * vdim, hidden, dtype), "o": matrix(g, hidden, heads * vdim, dtype)}
    w2 = {"q": matrix(g, heads * dim, hidden, dtype), "o": matrix(g, hidden, heads * vdim, dtype)}
    h1, h2 = (torch.randn(150, hidden, generator=g, dtype=F64) for _ in range(2))
    if dtype == torch.bfloat16:
        h1, h2 = bf16_round(h1), bf16_round(h2)
    _, keys = plain_attention(h1, w, heads, kv, dim, vdim, 48, 16, 0.2)
    want, _ = plain_attention(h2, w2, heads, kv, dim, vdim, 37, 16, 0.3, keys=keys)
    owner, precision, cache = build_attention(attention_spec(heads, kv, dim, vdim, 48, 16, 0.2, hidden), w, dtype)
    reader, _, _ = build_attention(attention_spec(heads, kv, dim, vdim, 37, 16, 0.3, hidden, shares=True), w2, dtype)
    assert reader.state_spec() is None and "k" not in reader.names
    feeder = Feeder(1)
    from flyweight_b200.engine import StepContext
    outs = []
    for m in (70, 1, 1, 50, 28):
        batch = feeder.batch([(0, m)])
        ctx = StepContext(batch, precision, DEV)
        at = feeder.done[0]
        owner.forward(ctx, dev(h1[at:at + m], precision.act_dtype), cache)
        outs.append(reader.forward(ctx, dev(h2[at:at + m], precision.act_dtype), cache).float().cpu())
        feeder.advance([(0, m)])
    close(torch.cat(outs), want, 2e-5 if dtype == torch.float32 else 3 * 2.0 ** -7, "the reading layer")


# ------------------------------------------------------------------ one key that stands out, at every edge
def edge_cases():
    cases = []
    for chunk in (50, 64, 100, 130):
        for n in (chunk * 2 + 1, chunk * 3, 257, 450):
            first = (n - 1) // chunk * chunk              # the first position the last query sees
            for far in {first, first + 1, n - 1, first - 1, first - 2, 0, 63, 64, (first // 64) * 64 - 1}:
                if 0 <= far < n:
                    cases.append((chunk, n, far))
    return sorted(set(cases))


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("chunk,n,far", edge_cases())
def test_one_key_that_stands_out_at_a_chunks_and_a_pages_edges(dtype, chunk, n, far):
    """Random scores hide a lost or a wrongly seen key among hundreds.  Here the last query matches the
    key at ``far`` far more than any other: if it lies inside the query's chunk the output is its value,
    if it lies just outside the output must not show it -- for a decoded token and for the last token of
    a portion, through every attention kernel."""
    from flyweight_b200.engine import StepContext
    from flyweight_b200.kernels import attention, ops
    heads, kv, hd = 12, 3, 64
    g = torch.Generator().manual_seed(chunk + n + far)
    keys = torch.randn(n, kv, hd, generator=g, dtype=F64) * 0.3
    values = torch.randn(n, kv, hd, generator=g, dtype=F64)
    query = torch.randn(heads, hd, generator=g, dtype=F64) * 0.3
    keys[far, 1] = 5.0 * query[5] / query[5].norm()          # head 5 (of key head 1) looks for `far`
    query[5] *= 6.0 / query[5].norm()
    if dtype == torch.bfloat16:
        keys, values, query = bf16_round(keys), bf16_round(values), bf16_round(query)
    seen = far >= (n - 1) // chunk * chunk
    positions = torch.arange(n)
    want = P.chunked_attention(query[None], positions[-1:], keys, values, positions, 1.0, chunk).view(heads, hd)
    if seen:
        assert float((want[5] - values[far, 1]).abs().max()) < 0.05 * float(values[far, 1].abs().max())
    else:
        assert float((want[5] - values[far, 1]).abs().max()) > 0.2
    feeder = Feeder(1, n_pages=12, seed=far)
    feeder.batch([(0, n)])                                    # hands out the pages
    k_pool = torch.full((12, kv, 64, hd), float("nan"), dtype=F64)
    v_pool = torch.full((12, kv, 64, hd), float("nan"), dtype=F64)
    for i, page in enumerate(feeder.pages[0]):
        rows = keys[i * 64:(i + 1) * 64]
        k_pool[page, :, :rows.shape[0]] = rows.transpose(0, 1)
        v_pool[page, :, :rows.shape[0]] = values[i * 64:(i + 1) * 64].transpose(0, 1)
    cache = type("Cache", (), {})()
    cache.k_pool, cache.v_pool = dev(k_pool, dtype), dev(v_pool, dtype)
    rel = 1e-5 if dtype == torch.float32 else 2.0 ** -7
    for new in sorted({1, min(40, n), min(130, n)}):
        feeder.done[0] = n - new
        batch = feeder.batch([(0, new)])
        qa = torch.zeros(new, heads, hd, dtype=F64)
        qa[-1] = query
        ctx = StepContext(batch, None, DEV)
        ways = [("tiled", True)] if dtype == torch.bfloat16 else []
        for name, tiled in [("default", False)] + ways:
            attention.force_tiled(tiled)
            try:
                out = attention.paged_attention(ctx, dev(qa, dtype).view(new, -1), cache, batch.block_tables[0],
                                                heads, -chunk, 1.0, dtype)
            finally:
                attention.force_tiled(False)
            close(out.view(new, heads, hd)[-1], want, rel, f"{name} kernel, {new} new tokens")
    assert ops is not None


# ------------------------------------------------------------------ the gated delta rule
def delta_spec(heads, kv, dim, vdim, taps, hidden):
    from flyweight_b200.config.spec import PartSpec
    names = ("q", "k", "v", "q_conv", "k_conv", "v_conv", "b", "a", "a_log", "dt_bias", "gate", "norm", "o")
    return PartSpec("gated_delta_rule", {"hidden_size": hidden, "num_heads": heads, "num_kv_heads": kv, "dim": dim,
                                         "vdim": vdim, "taps": taps, "eps": 1e-5}, {n: n for n in names})


def delta_weights(g, heads, kv, dim, vdim, taps, hidden, dtype):
    def vector(n, scale, shift=0.0):
        v = shift + scale * torch.randn(n, generator=g, dtype=F64)
        return bf16_round(v) if dtype == torch.bfloat16 else v.to(torch.float32).to(F64)
    w = {"q": matrix(g, kv * dim, hidden, dtype), "k": matrix(g, kv * dim, hidden, dtype),
         "v": matrix(g, heads * vdim, hidden, dtype), "gate": matrix(g, heads * vdim, hidden, dtype),
         "b": matrix(g, heads, hidden, dtype), "a": matrix(g, heads, hidden, dtype),
         "o": matrix(g, hidden, heads * vdim, dtype), "a_log": vector(heads, 0.5, -1.0), "dt_bias": vector(heads, 0.5),
         "norm": vector(vdim, 0.1, 1.0)}
    for name, rows in (("q_conv", kv * dim), ("k_conv", kv * dim), ("v_conv", heads * vdim)):
        w[name] = vector(rows * taps, 0.6).view(rows, taps)
    return w


def plain_delta(h, w, heads, kv, dim, vdim):
    names = {"q.conv": "q_conv", "k.conv": "k_conv", "v.conv": "v_conv", "A_log": "a_log", "g": "gate"}
    plain = {**w, **{theirs: w[ours] for theirs, ours in names.items()}}
    return P.delta_mixer(h, plain, heads, kv, dim, vdim, 1e-5)[0]


DELTA_SHAPES = [  # heads, kv, dim, vdim, taps, hidden
    (4, 2, 16, 24, 4, 80), (3, 1, 40, 20, 3, 96), (2, 2, 8, 8, 2, 64), (4, 2, 64, 128, 4, 128), (1, 1, 128, 64, 1, 72),
    (2, 1, 256, 40, 2, 64),
]


@pytest.mark.parametrize("shape", DELTA_SHAPES)
@pytest.mark.parametrize("dtype", BOTH)
def test_delta_rule_whole_cut_and_one_by_one(shape, dtype):
    """The state and the convolution's last inputs are carried through a slot: whole sequences, portions
    down to one and two tokens, four sequences side by side in slots that are not their batch places."""
    from flyweight_b200.kernels.recurrent import delta_state_size
    from flyweight_b200.parts import build_mixer
    heads, kv, dim, vdim, taps, hidden = shape
    g = torch.Generator().manual_seed(sum(shape))
    w = delta_weights(g, heads, kv, dim, vdim, taps, hidden, dtype)
    lengths = [210, 70, 1, 33]
    h_seqs = [torch.randn(n, hidden, generator=g, dtype=F64) for n in lengths]
    if dtype == torch.bfloat16:
        h_seqs = [bf16_round(h) for h in h_seqs]
    want = [plain_delta(h, w, heads, kv, dim, vdim) for h in h_seqs]
    precision = precision_of(dtype)
    part = build_mixer(delta_spec(heads, kv, dim, vdim, taps, hidden))
    part.bind(lambda n: w[n].to(dtype), precision, DEV)
    assert part.state_spec().shape == (delta_state_size(heads, kv, dim, vdim, taps),)
    rel = 2e-5 if dtype == torch.float32 else 3 * 2.0 ** -7
    cache = type("Cache", (), {})()
    for name, sizes in (("whole", [1000]), ("cut", [3, 2, 64, 1, 33, 7, 2]), ("one by one", [1])):
        cache.state = torch.zeros((6, part.state_spec().shape[0]), dtype=torch.float32, device=DEV)
        cache.state[0].fill_(float("nan"))          # nobody's slot: never read
        slots = {0: 4, 1: 2, 2: 5, 3: 1}
        got = run_part(part, precision, h_seqs, cuts_of(lengths, sizes), cache, Feeder(4, slots=slots))
        for s, wanted in enumerate(want):
            close(got[s], wanted, rel, f"{name}, sequence {s}")
        assert torch.isnan(cache.state[0]).all() and float(cache.state[3].abs().max()) == 0.0


def test_the_delta_state_remembers_a_write_from_hundreds_of_tokens_ago():
    """One early token writes a value under a key that no later token touches (later keys are orthogonal
    to it and decay is switched off): a query for that key, 400 tokens and several steps later, reads the
    value back.  A state that was dropped, reset or shifted between steps would not."""
    from flyweight_b200.kernels import recurrent
    H, G, d, e, L, n = 2, 1, 16, 8, 1, 400
    C = 2 * G * d + H * e
    p = torch.zeros(n, C + H * e + 2 * H, dtype=F64)
    g = torch.Generator().manual_seed(9)
    big = 20.0                                          # silu(20) ~ 20; unit vectors forget the length
    p[:, G * d + 1] = big                               # every key: axis 1
    p[:, 0 * d + 2] = big                               # every query: axis 2 (reads nothing)
    p[7, G * d:2 * G * d] = 0
    p[7, G * d + 0] = big                               # token 7 writes under axis 0
    v7 = torch.randn(H * e, generator=g, dtype=F64).abs() + 1.0
    p[:, 2 * G * d:C] = torch.randn(n, H * e, generator=g, dtype=F64)
    p[7, 2 * G * d:C] = v7
    p[:, C + H * e:C + H * e + H] = 30.0                # beta = 1
    p[:, C + H * e + H:] = -30.0                        # softplus -> 0: decay 1
    p[n - 1, 0:G * d] = 0
    p[n - 1, 0] = big                                   # the last query asks for axis 0
    taps = torch.ones(C, 1, dtype=torch.float32)
    zeros = torch.zeros(H, dtype=torch.float32)
    state = torch.zeros((2, recurrent.delta_state_size(H, G, d, e, L)), dtype=torch.float32, device=DEV)
    feeder = Feeder(1, slots={0: 1})
    outs = []
    for step in cuts_of([n], [5, 64, 1, 1, 130, 2]):
        batch = feeder.batch(step)
        at, m = feeder.done[0], step[0][1]
        outs.append(recurrent.delta_rule(dev(p[at:at + m], torch.float32), dev(taps), dev(zeros), dev(zeros), state,
                                         batch, H, G, d, e).cpu())
        feeder.advance(step)
    out = torch.cat(outs).view(n, H * e)
    want = P.silu(v7) * d ** -0.5
    close(out[n - 1], want, 1e-4, "the value written 392 tokens before")
    assert float(out[n - 2].abs().max()) < 1e-3 * float(want.abs().max())


def test_gated_head_norm():
    from flyweight_b200.kernels import recurrent
    g = torch.Generator().manual_seed(4)
    T, H, e = 9, 3, 20
    o = torch.randn(T, H, e, generator=g, dtype=torch.float32) * 4
    wide = torch.randn(T, 100 + H * e, generator=g, dtype=torch.float32)
    weight = 1 + 0.1 * torch.randn(e, generator=g, dtype=torch.float32)
    gate = wide[:, 40:40 + H * e]
    want = (P.rms_unit(o.to(F64), 1e-5) * weight.to(F64) * P.silu(gate.to(F64)).view(T, H, e)).view(T, H * e)
    for dtype in BOTH:
        out = recurrent.gated_head_norm(dev(o), dev(wide)[:, 40:40 + H * e], dev(weight), 1e-5, dtype)
        close(out, want, 1e-6 if dtype == torch.float32 else 2.0 ** -8, str(dtype))


# ------------------------------------------------------------------ the router and the experts
ROUTERS = [  # outputs, groups, keep, top
    (8, 4, 2, 3), (5, 1, 1, 1), (6, 3, 2, 4), (8, 2, 1, 2), (20, 5, 2, 6), (64, 8, 3, 8), (7, 7, 7, 7), (33, 1, 1, 5),
]


@pytest.mark.parametrize("W", [512, 520, 2112])
@pytest.mark.parametrize("N,groups,keep,top", [(8, 4, 2, 3), (33, 1, 1, 5), (20, 5, 2, 6)])
@pytest.mark.parametrize("dtype", BOTH)
def test_router_over_wide_rows(W, N, groups, keep, top, dtype):
    """Few tokens with rows of 512 entries and more take the kernel's other way through the products (K cut
    over the warps): whole turns of all warps, a last turn that only some warps take part in, a last piece."""
    from flyweight_b200.kernels import experts
    g = torch.Generator().manual_seed(N + W)
    T = 40
    h = torch.randn(T, W, generator=g, dtype=F64)
    h = bf16_round(h) if dtype == torch.bfloat16 else h.to(torch.float32).to(F64)
    router = (torch.randn(N, W, generator=g, dtype=F64) / math.sqrt(W) * 2).to(torch.float32)
    correction = (torch.randn(N, generator=g, dtype=F64) * 0.15).to(torch.float32)
    ids, weights = experts.route(dev(h, dtype), dev(router), dev(correction), groups, keep, top)
    want_ids, want_w = P.route(h, router.to(F64), correction.to(F64), groups, keep, top)
    same = (ids.cpu().long() == want_ids).all(dim=1)
    assert same.float().mean() > 0.95, f"{int((~same).sum())} of {T} tokens choose differently"
    close(weights.cpu()[same], want_w[same], 1e-5, "weights")


@pytest.mark.parametrize("N,groups,keep,top", ROUTERS)
@pytest.mark.parametrize("dtype", BOTH)
def test_router(N, groups, keep, top, dtype):
    """Chosen outputs and weights against the plain router on the same inputs.  Corrections are large
    enough to change the choice (so that a choice made on the plain scores would show) and negative for
    some outputs (so that a group counted as 0 instead of minus infinity would show)."""
    from flyweight_b200.kernels import experts
    g = torch.Generator().manual_seed(N * top)
    T, W = 300, 72
    h = torch.randn(T, W, generator=g, dtype=F64)
    h = bf16_round(h) if dtype == torch.bfloat16 else h.to(torch.float32).to(F64)
    router = (torch.randn(N, W, generator=g, dtype=F64) / math.sqrt(W) * 2).to(torch.float32)
    correction = (torch.randn(N, generator=g, dtype=F64) * 0.15 - 0.3).to(torch.float32)
    ids, weights = experts.route(dev(h, dtype), dev(router), dev(correction), groups, keep, top)
    want_ids, want_w = P.route(h, router.to(F64), correction.to(F64), groups, keep, top)
    same = (ids.cpu().long() == want_ids).all(dim=1)
    assert same.float().mean() > 0.99, f"{int((~same).sum())} of {T} tokens choose differently"
    close(weights.cpu()[same], want_w[same], 1e-5, "weights")
    plain_choice = torch.topk(torch.softmax(h @ router.to(F64).T, dim=-1), top, dim=-1).indices
    if N > top and (groups > keep or N > 8):
        assert not (plain_choice == want_ids).all(), "this case does not tell a choice without correction apart"


def experts_spec(hidden, ff, n_experts, identity, top, groups, keep):
    from flyweight_b200.config.spec import PartSpec
    tensors = {"router": "router", "correction": "correction"}
    for j in range(n_experts):
        tensors.update({f"gate{j}": f"e{j}.gate", f"up{j}": f"e{j}.up", f"down{j}": f"e{j}.down"})
    return PartSpec("routed_experts", {"hidden_size": hidden, "ffn_dim": ff, "experts": n_experts, "identity": identity,
                                       "top": top, "groups": groups, "keep_groups": keep}, tensors)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("hidden,ff,n_experts,identity,top,groups,keep",
                         [(80, 48, 6, 2, 3, 4, 2), (96, 40, 5, 0, 1, 1, 1), (96, 24, 3, 3, 4, 3, 2),
                          (128, 64, 8, 0, 2, 2, 1), (64, 70, 1, 1, 2, 1, 1), (72, 16, 0, 4, 2, 2, 2)])
@pytest.mark.parametrize("T", [1, 5, 300])
def test_routed_experts(dtype, hidden, ff, n_experts, identity, top, groups, keep, T):
    """The feed-forward part against the plain one: experts that get no token, experts that get more
    than a tile of them, identity experts, a router with identity experts only.  In bfloat16 the
    corrections are far apart, so that the choice does not hang on the rounding of the scores."""
    from flyweight_b200.parts import build_feed_forward
    g = torch.Generator().manual_seed(hidden + ff + T)
    N = n_experts + identity
    w = {"router": matrix(g, N, hidden, dtype) * 3, "correction": torch.randn(N, generator=g, dtype=F64) * 0.1}
    if dtype == torch.bfloat16:
        w["correction"] = torch.randperm(N, generator=g).to(F64) * 4.0
    for j in range(n_experts):
        w[f"e{j}.gate"], w[f"e{j}.up"] = matrix(g, ff, hidden, dtype), matrix(g, ff, hidden, dtype)
        w[f"e{j}.down"] = matrix(g, hidden, ff, dtype)
    h = torch.randn(T, hidden, generator=g, dtype=F64)
    h = bf16_round(h) if dtype == torch.bfloat16 else h.to(torch.float32).to(F64)
    precision = precision_of(dtype)
    part = build_feed_forward(experts_spec(hidden, ff, n_experts, identity, top, groups, keep))
    part.bind(lambda n: w[n].to(dtype), precision, DEV)
    got = run_part(part, precision, [h], [[(0, T)]], None, feed_forward=True)[0]
    if dtype == torch.bfloat16:
        # the grouped tensor-core product (the default where the sizes allow it) beside the fp32-FMA kernel
        from flyweight_b200.kernels import experts as expert_kernels, tensorcore
        expert_kernels.set_tensor_cores(False)
        try:
            plain_way = run_part(part, precision, [h], [[(0, T)]], None, feed_forward=True)[0]
        finally:
            expert_kernels.set_tensor_cores(True)
        close(plain_way, got, 2.0 ** -7, "the two kernels of the experts' products")
        assert tensorcore.status() == 0
    plain_experts = [(w[f"e{j}.gate"], w[f"e{j}.up"], w[f"e{j}.down"]) for j in range(n_experts)]
    want = P.moe(h, w["router"], w["correction"], plain_experts, identity, groups, keep, top)
    close(got, want, 2e-5 if dtype == torch.float32 else 3 * 2.0 ** -7, "experts")
    # the same with the output norm and the residual sum in the part's last kernel
    from flyweight_b200.engine import StepContext
    x = torch.randn(T, hidden, generator=g, dtype=torch.float32)
    w_norm = 1 + 0.1 * torch.randn(hidden, generator=g, dtype=torch.float32)
    xd = dev(x)
    part.forward_add_normed(StepContext(Feeder(1).batch([(0, T)]), precision, DEV), dev(h, precision.act_dtype), xd,
                            dev(w_norm), 1e-5)
    close(xd, x.to(F64) + P.rms_norm(want, w_norm.to(F64), 1e-5), 2e-5 if dtype == torch.float32 else 3 * 2.0 ** -7,
          "normed and added")
    # a token's result does not depend on what else is in the step
    if T > 5:
        alone = run_part(part, precision, [h[:3]], [[(0, 3)]], None, feed_forward=True)[0]
        close(alone, got[:3], 0.0 if dtype == torch.float32 else 2.0 ** -8, "three tokens alone")
