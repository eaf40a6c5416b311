"""Kesedra on the GPU against the plain statement: each mechanism alone, then the model through the
step function, the cache, the state slots and the generation loop, cut into steps and batches in every
way."""

import math

import pytest
import torch

import plain_kesedra as plain
from gpu_helpers import DTYPES, FP32_TOL
from tiny import random_prompt
from tiny_kesedra import TINY_K, make_kesedra_folder

pytestmark = pytest.mark.gpu

CONFIGS = ["KA", "KB", "KC"]
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}
F = torch.float64
_cases, _runners = {}, {}


def case(tmp_path_factory, name, seed=1):
    if (name, seed) not in _cases:
        folder = make_kesedra_folder(tmp_path_factory.mktemp(f"k{name}{seed}"), name, seed=seed)
        _cases[(name, seed)] = (folder,) + plain.read_model_folder(folder)
    return _cases[(name, seed)]


def runner_for(tmp_path_factory, name, dtype, max_tokens=64 * 40):
    from starter_b200.engine import ModelRunner, load_model

    if (name, dtype) not in _runners:
        folder, _, _ = case(tmp_path_factory, name)
        _runners[(name, dtype)] = ModelRunner(load_model(folder, dtype), max_tokens=max_tokens, max_sequences=12)
    return _runners[(name, dtype)]


def close(got, want, dtype, what, fp32=2e-5, bf16=2e-2):
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    tol = (fp32 if dtype in ("float32", torch.float32) else bf16) * float(want.abs().max())
    err = (got - want).abs()
    assert float(err.max()) <= tol, f"{what}: off by {float(err.max()):.3e} (allowed {tol:.3e}) at {tuple(int(i) for i in (err == err.max()).nonzero()[0])}"


# Bounds of the model-level comparisons, relative to the largest logit of the case and fixed from
# measurements.  float32: as for the other designs (measured here: at most 2.1e-6).  bfloat16 against the
# float64 statement: this design norms every sublayer's output to unit size before it is added, so a
# sublayer's rounding is never small beside its result; measured on these configurations, prompts and
# decoded tails alike: mean error 5.5e-3 to 5.9e-3, largest row 1.6e-2 to 3.9e-2.  The worst-conditioned
# row is a sequence's first token behind a recurrent layer: its state is empty, so the head's output is
# c * v / rms(c * v) with the scalar c = sum_i r_i u_i k_i, of which only the sign survives the unit norm.
# A lost state, a key that is one off or a skipped layer moves rows by 1e-1 and more, and the float32 runs
# of the same kernels hold every row to 2e-5.
BF16_ROW_TOL = 6e-2
BF16_MEAN_TOL = 1e-2


def assert_close(got, want, dtype, what=""):
    """Fails with the first wrong row named: its place is the clue (a prompt's end, the first
    single-token step, a page boundary, a window's edge)."""
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    scale = float(want.abs().max())
    tol = (FP32_TOL if dtype == "float32" else BF16_ROW_TOL) * scale
    err = (got - want).abs().reshape(want.shape[0], -1).max(dim=1).values
    bad = (~(err <= tol)).nonzero().flatten().tolist()
    assert not bad, (f"{what}: {len(bad)} of {len(err)} rows off by more than {tol:.2e}; first wrong row {bad[0]} "
                     f"(error {err[bad[0]].item():.3e}), largest error {err.max().item():.3e}")
    if dtype != "float32":
        mean = (got - want).abs().mean().item()
        assert mean <= BF16_MEAN_TOL * scale, f"{what}: mean error {mean:.3e} above {BF16_MEAN_TOL * scale:.3e}"


def dev(v, ty=torch.float32):
    return v.to("cuda", ty).contiguous()


class Routed:
    """Runs steps and notes, per request, which experts every routed layer chose for each of its tokens.
    The 32-bit comparisons do not use the notes (there the choice itself is held to the plain statement);
    the bfloat16 comparisons hand them to the plain statement, because a near-tie between two experts may
    fall either way once the router's input is rounded to 8 bits, and that is no fault."""

    def __init__(self, runner):
        self.runner = runner
        self.layers = [i for i, b in enumerate(runner.model.blocks)
                       if getattr(b, "feed_forward", None) is not None and hasattr(b.feed_forward, "last_ids")]
        self.notes = {}

    def step(self, entries, keys):
        out = self.runner.step(entries)
        at = 0
        for entry, key in zip(entries, keys):
            n = len(entry.tokens)
            for layer in self.layers:
                ids = self.runner.model.blocks[layer].feed_forward.last_ids[at:at + n].cpu()
                self.notes.setdefault(key, {}).setdefault(layer, []).append(ids)
            at += n
        return out

    def routes(self, key, dtype):
        if dtype == "float32" or not self.layers:
            return None
        return {layer: torch.cat(parts) for layer, parts in self.notes[key].items()}


# ------------------------------------------------------------------------------ mechanisms alone

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [40, 37, 600, 13000])
def test_residual_sum_and_both_norms_alone(hidden, dtype):
    from starter_b200 import ops

    t = TORCH[dtype]
    g = torch.Generator().manual_seed(hidden)
    x = torch.randn(7, hidden, generator=g, dtype=F) * 3
    y = torch.randn(7, hidden, generator=g, dtype=F) * 5
    post, nxt, bias = (torch.randn(hidden, generator=g, dtype=F) for _ in range(3))
    xd, yd = dev(x), dev(y, t)
    y64 = yd.double().cpu()
    # a sublayer's output with a bias left over, normed, added, and the next norm of the sum
    out = ops.residual_norm(xd, t, 1e-5, (yd, dev(post), dev(bias), 1e-3), dev(nxt))
    want_x = x + plain.rms(y64 + bias, 1e-3) * post
    close(xd, want_x, "float32", "the sum, in place", fp32=3e-6)
    close(out, plain.rms(want_x, 1e-5) * nxt, dtype, "the next norm")
    # selected rows, nothing written back; no pending output
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device="cuda")
    before = xd.clone()
    out = ops.residual_norm(xd, t, 1e-5, (yd, dev(post), None, 1e-5), dev(nxt), rows=rows)
    assert torch.equal(xd, before)
    again = want_x + plain.rms(y64, 1e-5) * post
    close(out, (plain.rms(again, 1e-5) * nxt)[[5, 0, 5]], dtype, "selected rows")
    close(ops.residual_norm(xd, t, 1e-5, None, dev(nxt)), plain.rms(want_x, 1e-5) * nxt, dtype, "norm alone")
    assert ops.residual_norm(xd, t, 1e-5, (yd, None, None, 0.0), None) is None
    close(xd, want_x + y64, "float32", "a plain sum", fp32=3e-6)


@pytest.mark.parametrize("dtype", DTYPES)
def test_scaled_embedding_and_bias_activation(dtype):
    from starter_b200 import ops

    t = TORCH[dtype]
    g = torch.Generator().manual_seed(1)
    table = dev(torch.randn(50, 72, generator=g), t)
    tokens = torch.tensor([3, 49, 0, 3], dtype=torch.int32, device="cuda")
    out = ops.embedding32(tokens, table, 6.5)
    assert out.dtype == torch.float32
    assert torch.equal(out, table.float()[tokens.long()] * 6.5)
    x = dev(torch.randn(9, 44, generator=g) * 2, t)
    b = dev(torch.randn(44, generator=g))
    xb = x.double().cpu() + b.double().cpu()
    close(ops.bias_act(x, b, "relu2"), torch.relu(xb) ** 2, dtype, "squared relu")
    close(ops.bias_act(x, None, "tanh"), torch.tanh(x.double().cpu()), dtype, "tanh")
    close(ops.bias_act(x, b, None), xb, dtype, "bias alone")


def wkv_inputs(heads, dim, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    n = sum(lengths)
    hd = heads * dim
    r, k, v, gate = (torch.randn(n, hd, generator=g, dtype=F) for _ in range(4))
    x_decay = torch.randn(n, hd, generator=g, dtype=F) * 0.5
    w0 = torch.linspace(-6.0, 0.5, hd, dtype=F)        # from channels that keep almost everything to ones that forget
    u = torch.randn(heads, dim, generator=g, dtype=F)
    gain = 1 + 0.1 * torch.randn(hd, generator=g, dtype=F)
    return r, k, v, gate, x_decay, w0, u, gain


def plain_wkv(r, k, v, gate, x_decay, w0, u, gain, heads, dim, eps):
    n = r.shape[0]
    decay = torch.exp(-torch.exp(x_decay + w0)).reshape(n, heads, dim)
    o = plain.wkv_recurrence(r.reshape(n, heads, dim), k.reshape(n, heads, dim), v.reshape(n, heads, dim), decay, u)
    return plain.rms(o, eps).reshape(n, heads * dim) * gain * (gate * torch.sigmoid(gate))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, dim", [(2, 16), (3, 24), (1, 64), (2, 128), (1, 40), (5, 8), (1, 256), (2, 2)])
def test_recurrence_alone_whole_in_portions_and_token_by_token(heads, dim, dtype):
    """Three sequences of unequal lengths in one step; then the same sequences in portions (down to one
    token, across the kernel's chunks of 16) from the state the portions before left in their slots, in
    slots that another sequence used before."""
    from starter_b200 import ops

    t = TORCH[dtype]
    lengths = [37, 1, 70] if dim < 256 else [19, 1, 6]
    width = 24
    r, k, v, gate, x_decay, w0, u, gain = wkv_inputs(heads, dim, lengths, 7)
    rd, kd, vd, gd = (dev(a, t) for a in (r, k, v, gate))
    r, k, v, gate = (a.double().cpu() for a in (rd, kd, vd, gd))
    xdd, ud, gaind = ops.bias_act(dev(x_decay), dev(w0), "decay"), dev(u), dev(gain)
    h = dev(torch.randn(sum(lengths), width, generator=torch.Generator().manual_seed(2)), t)
    starts = [0, lengths[0], lengths[0] + lengths[1]]
    want = torch.cat([plain_wkv(*(a[s:s + n] for a in (r, k, v, gate, x_decay)), w0, u, gain, heads, dim, 1e-5)
                      for s, n in zip(starts, lengths)])
    state = torch.full((6, width + heads * dim * dim), 3.0, device="cuda")     # what another sequence left
    slots = [4, 1, 2]
    state[slots] = 0.0
    ints = lambda a: torch.tensor(a, dtype=torch.int32, device="cuda")  # noqa: E731
    out = ops.wkv_scan(rd, kd, vd, xdd, ud, gd, gaind, state, h, ints(slots), ints(starts), ints(lengths),
                       heads, dim, 1e-5)
    close(out, want, dtype, f"whole, heads {heads} x {dim}", fp32=5e-5)
    for i, slot in enumerate(slots):       # the last mixer input of every sequence is in its slot
        assert torch.equal(state[slot, :width], h[starts[i] + lengths[i] - 1].float())
    assert bool((state[[0, 3, 5]] == 3.0).all())
    whole_state = state.clone()
    # the same in portions: every sequence cut its own way, the portions of a step packed together
    state[slots] = 0.0
    cuts = [[16, 1, 15, 5], [1], [2, 33, 32, 3]] if dim < 256 else [[16, 3], [1], [1, 5]]
    got = [[None] * len(c) for c in cuts]
    done = [0, 0, 0]
    for step in range(max(len(c) for c in cuts)):
        live = [i for i in range(3) if step < len(cuts[i])]
        idx = torch.cat([torch.arange(starts[i] + done[i], starts[i] + done[i] + cuts[i][step]) for i in live]).cuda()
        sizes = [cuts[i][step] for i in live]
        offs = [sum(sizes[:j]) for j in range(len(live))]
        out = ops.wkv_scan(rd[idx].contiguous(), kd[idx].contiguous(), vd[idx].contiguous(), xdd[idx].contiguous(),
                           ud, gd[idx].contiguous(), gaind, state, h[idx].contiguous(), ints([slots[i] for i in live]),
                           ints(offs), ints(sizes), heads, dim, 1e-5)
        for j, i in enumerate(live):
            got[i][step] = out[offs[j]:offs[j] + sizes[j]]
            done[i] += sizes[j]
    close(torch.cat([torch.cat(g) for g in got]), want, dtype, f"in portions, heads {heads} x {dim}", fp32=5e-5)
    close(state[slots], whole_state[slots], "float32", "the state the portions leave", fp32=5e-5)


@pytest.mark.parametrize("dtype", DTYPES)
def test_recurrence_keeps_what_a_far_token_wrote(dtype):
    """One token far back writes a large k v^T into a channel that hardly decays; 300 tokens on, through
    19 chunks and two steps, a receptance that reads only that channel must still find it."""
    from starter_b200 import ops

    t = TORCH[dtype]
    heads, dim, n = 1, 16, 330
    r = torch.zeros(n, dim, dtype=F)
    k = torch.randn(n, dim, generator=torch.Generator().manual_seed(1), dtype=F) * 0.01
    v = torch.randn(n, dim, generator=torch.Generator().manual_seed(2), dtype=F) * 0.01
    k[20, 3], v[20, 5] = 4.0, 8.0
    r[:, 3] = 1.0
    gate = torch.full((n, dim), 2.0, dtype=F)
    x_decay = torch.zeros(n, dim, dtype=F)
    w0 = torch.full((dim,), 0.0, dtype=F)
    w0[3] = -9.0                                   # decay exp(-exp(-9)) = 0.99988 a step
    u, gain = torch.zeros(1, dim, dtype=F), torch.ones(dim, dtype=F)
    want_o = plain.wkv_recurrence(r.reshape(n, 1, dim), k.reshape(n, 1, dim), v.reshape(n, 1, dim),
                                  torch.exp(-torch.exp(x_decay + w0)).reshape(n, 1, dim), u)
    assert abs(want_o[320, 0, 5].item()) > 25.0 and abs(want_o[19, 0, 5].item()) < 0.01
    rd, kd, vd, gd = (dev(a, t) for a in (r, k, v, gate))
    want = plain_wkv(*(a.double().cpu() for a in (rd, kd, vd, gd)), x_decay, w0, u, gain, 1, dim, 1e-5)
    state = torch.zeros(2, 8 + dim * dim, device="cuda")
    h = torch.zeros(n, 8, device="cuda", dtype=t)
    ints = lambda a: torch.tensor(a, dtype=torch.int32, device="cuda")  # noqa: E731
    parts = []
    for lo, hi in ((0, 250), (250, 330)):
        parts.append(ops.wkv_scan(rd[lo:hi].contiguous(), kd[lo:hi].contiguous(), vd[lo:hi].contiguous(),
                                  ops.bias_act(dev(x_decay[lo:hi]), dev(w0), "decay"), dev(u), gd[lo:hi].contiguous(), dev(gain), state,
                                  h[lo:hi].contiguous(), ints([1]), ints([0]), ints([hi - lo]), 1, dim, 1e-5))
    close(torch.cat(parts), want, dtype, "a far token in a slow channel", fp32=5e-5)


@pytest.mark.parametrize("dtype", DTYPES)
def test_token_shift_alone(dtype):
    """The first row a sequence brings is mixed with what its slot holds; every other row with the row before."""
    from starter_b200 import ops

    t = TORCH[dtype]
    g = torch.Generator().manual_seed(4)
    h = dev(torch.randn(9, 20, generator=g), t)
    mu = torch.rand(5, 20, generator=g, dtype=F)
    state = torch.zeros(4, 20 + 7, device="cuda")
    state[2, :20] = torch.randn(20, generator=g)
    slots = torch.tensor([2, 2, 2, 0, 3, 3, 3, 3, 1], dtype=torch.int32, device="cuda")
    out = ops.token_shift(h, state, dev(mu), slots)
    h64 = h.double().cpu()
    prev = torch.cat([state[2, :20].double().cpu()[None], h64[:-1]])
    prev[3] = 0.0
    prev[4] = 0.0
    prev[8] = 0.0
    want = torch.stack([h64 + (prev - h64) * mu[s] for s in range(5)])
    close(out, want, dtype, "token shift")


def latent_case(heads, rank, rot, lengths, seed, window):
    g = torch.Generator().manual_seed(seed)
    n = sum(lengths)
    qa = torch.randn(n, heads, rank + rot, generator=g, dtype=F)
    rows = torch.randn(n, rank + rot, generator=g, dtype=F)
    return qa, rows


def plain_latent(qa, rows, rank, scale, window):
    """One sequence: scores against the rows as they are, the window, softmax, the sum of the rows' first
    ``rank`` entries."""
    n = qa.shape[0]
    s = torch.einsum("thd,sd->hts", qa, rows) * scale
    i, j = torch.arange(n)[:, None], torch.arange(n)[None, :]
    seen = (i - j >= 0) & ((i - j < window) if window else (i >= j))
    p = torch.softmax(s.masked_fill(~seen[None], -math.inf), dim=-1)
    return torch.einsum("hts,sd->thd", p, rows[:, :rank])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, rank, rot, window", [(3, 32, 8, 10), (1, 48, 16, 3), (4, 64, 32, 65), (4, 64, 32, 64),
                                                      (2, 20, 6, 0), (5, 16, 4, 500), (2, 512, 64, 100), (3, 24, 8, 1),
                                                      (5, 96, 16, 0), (70, 32, 16, 40), (16, 128, 32, 33)])
def test_latent_attention_alone_with_one_key_that_stands_out(heads, rank, rot, window, dtype):
    """Queries late in a sequence of 200 (pages 0 to 3, scattered) score one key far above the rest: the
    key just inside the window, just outside it, on either side of a page border, the query's own place
    and a key far back; the answer must be that key's latent, or must not contain it."""
    from starter_b200 import ops

    t = TORCH[dtype]
    n = 200
    qa, rows = latent_case(heads, rank, rot, [n], heads * 100 + rank, window)
    probes = {}                                     # query position -> the key made to stand out
    w = window if window else n
    for q_pos, back in ((150, w - 1), (151, w), (130, 2), (129, 1), (199, 0), (180, 170), (128, 64), (191, 63)):
        if q_pos - back >= 0 and q_pos not in probes:
            probes[q_pos] = q_pos - back
    for q_pos, key in probes.items():
        direction = rows[key] / rows[key].norm()
        qa[q_pos, :, :] = direction * 60.0          # a score of 60 |row| * scale against about +-8 for the rest
    qd, rd = dev(qa, t), dev(rows, t)
    want = plain_latent(qd.double().cpu(), rd.double().cpu(), rank, 0.11, window)
    for q_pos, key in probes.items():               # the plain statement itself shows the probe
        picked = (want[q_pos, 0] - rd.double().cpu()[key, :rank]).abs().max().item() < 0.05
        assert picked == (q_pos - key < w), (q_pos, key)
    pages = [5, 2, 7, 0]
    table = torch.zeros(3, 6, dtype=torch.int32, device="cuda")
    table[1, :4] = torch.tensor(pages, dtype=torch.int32)
    store = torch.zeros(8, 1, 64, rank + rot, dtype=t, device="cuda")
    for i, page in enumerate(pages):
        chunk = rd[64 * i:64 * (i + 1)]
        store[page, 0, :chunk.shape[0]] = chunk
    pos = torch.arange(n, dtype=torch.int32, device="cuda")
    slot = torch.ones(n, dtype=torch.int32, device="cuda")
    out = ops.latent_attention(qd, store, table, slot, pos, heads, rank, rot, 0.11, window or None)
    close(out, want, dtype, f"window {window}", bf16=1.5e-2)
    # the last 40 as single tokens of a step of their own (what decoding asks)
    tail = torch.arange(160, 200, device="cuda")
    out = ops.latent_attention(qd[tail].contiguous(), store, table, slot[tail].contiguous(), pos[tail].contiguous(),
                               heads, rank, rot, 0.11, window or None)
    close(out, want[160:], dtype, f"window {window}, single tokens", bf16=1.5e-2)
    if not ops.latent_tc_takes(t, rank, rot):
        return
    # the tensor-core kernel: the whole sequence as one step (four tiles of 64 tokens), then its last 40
    # tokens as a later portion, then the last token alone with its keys cut into 1, 3 and 7 parts
    ints = lambda a: torch.tensor(a, dtype=torch.int32, device="cuda")  # noqa: E731
    out = ops.latent_attention_tc(qd, store, table, ints([1]), ints([0]), ints([n]), ints([n]), ints([0, 0, 0, 0]),
                                  ints([128, 0, 192, 64]), heads, rank, rot, 0.11, window or None)
    close(out, want, dtype, f"tensor cores, window {window}", bf16=1.5e-2)
    out = ops.latent_attention_tc(qd[tail].contiguous(), store, table, ints([1]), ints([0]), ints([40]), ints([n]),
                                  ints([0]), ints([0]), heads, rank, rot, 0.11, window or None)
    close(out, want[160:], dtype, f"tensor cores, window {window}, a portion", bf16=1.5e-2)
    for parts in (1, 3, 7):
        out = ops.latent_attention_tc(qd[199:].contiguous(), store, table, ints([1]), ints([0]), ints([1]), ints([n]),
                                      ints([0]), ints([0]), heads, rank, rot, 0.11, window or None, n_splits=parts)
        close(out, want[199:], dtype, f"tensor cores, window {window}, one token in {parts} parts", bf16=1.5e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("dims", [8, 4])
def test_latent_prepare_and_query_rotation_alone(dims, dtype):
    """Norms, the rotation of the shared key part (all of it, or its first half) and where the row is
    filed: positions on both sides of a page border, two sequences."""
    from starter_b200 import ops
    from starter_b200.config import InterleavedRopeSpec
    from starter_b200.parts import InterleavedRotaryTable

    t = TORCH[dtype]
    q_rank, rank, rot, heads, dim = 12, 20, 8, 3, 6
    g = torch.Generator().manual_seed(dims)
    pos_list, slot_list = [62, 63, 64, 65, 0, 1], [1, 1, 1, 1, 0, 0]
    n = len(pos_list)
    proj = dev(torch.randn(n, q_rank + rank + rot, generator=g) * 3, t)
    qg, kg = torch.randn(q_rank, generator=g, dtype=F), torch.randn(rank, generator=g, dtype=F)
    tables = InterleavedRotaryTable(InterleavedRopeSpec(dims=dims, base=77.0), t)
    tables.ensure(100)
    rotation = tables.rotation()
    cos, sin = ops.latent_tables(rotation, dims)
    table = torch.tensor([[3, 0], [1, 2]], dtype=torch.int32, device="cuda")
    store = torch.zeros(4, 1, 64, rank + rot, dtype=t, device="cuda")
    pos = torch.tensor(pos_list, dtype=torch.int32, device="cuda")
    slot = torch.tensor(slot_list, dtype=torch.int32, device="cuda")
    cq = ops.latent_prepare(proj, dev(qg), dev(kg), 1e-4, cos, sin, pos, slot, table, store, q_rank, rank, rot, dims)
    p64 = proj.double().cpu()
    close(cq, plain.norm_plain_gain(p64[:, :q_rank], qg, 1e-4), dtype, "query latent")
    want_c = plain.norm_plain_gain(p64[:, q_rank:q_rank + rank], kg, 1e-4)
    want_s = plain.rotate_interleaved(p64[:, q_rank + rank:], torch.tensor(pos_list), 77.0, dims)
    for i, (p, s) in enumerate(zip(pos_list, slot_list)):
        row = store[int(table[s, p // 64]), 0, p % 64]
        close(row[:rank], want_c[i], dtype, f"latent of token {i}")
        close(row[rank:], want_s[i], dtype, f"shared key part of token {i}")
    assert int((store.float().abs().sum(dim=-1) > 0).sum()) == n        # nothing else was written
    only_q = ops.latent_prepare(proj[:, :q_rank].contiguous(), dev(qg), None, 1e-4, cos, sin, pos, slot, table, None,
                                q_rank, rank, rot, dims, write_cache=False)
    assert torch.equal(only_q, cq)
    q = dev(torch.randn(n, heads * (dim + rot), generator=g), t)
    qa = torch.zeros(n, heads, rank + rot, dtype=t, device="cuda")
    ops.latent_rotate_q(q, qa, cos, sin, pos, heads, dim, rot, dims, rank)
    want_q = plain.rotate_interleaved(q.double().cpu().reshape(n, heads, dim + rot)[:, :, dim:], torch.tensor(pos_list), 77.0, dims)
    close(qa[:, :, rank:], want_q, dtype, "rotated query part")
    assert float(qa[:, :, :rank].abs().max()) == 0.0


@pytest.mark.parametrize("experts, top", [(5, 2), (3, 1), (3, 3), (12, 4), (64, 8)])
def test_router_alone(experts, top):
    from starter_b200 import ops

    g = torch.Generator().manual_seed(experts)
    h = dev(torch.randn(50, 72, generator=g))
    router, bias = torch.randn(experts, 72, generator=g, dtype=F), torch.randn(experts, generator=g, dtype=F)
    w = {"router": router, "router.b": bias}
    ids, weights = ops.moe_route(h, dev(router), dev(bias), top)
    want_ids, want_w = plain.route(h.double().cpu(), w, "", top)
    assert torch.equal(ids.cpu().long(), want_ids)
    close(weights, want_w, "float32", "softmax over the chosen")
    # equal logits: the lower index first
    ids, weights = ops.moe_route(torch.zeros(2, 72, device="cuda"), dev(router), torch.zeros(experts, device="cuda"), top)
    assert ids.cpu().tolist() == [list(range(top))] * 2 and torch.allclose(weights.cpu(), torch.full((2, top), 1.0 / top))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows", [1, 5, 70, 300])
@pytest.mark.parametrize("experts, top, width, inner", [(5, 2, 64, 24), (3, 3, 96, 16), (8, 2, 128, 64), (6, 1, 40, 36)])
def test_experts_alone(experts, top, width, inner, rows, dtype):
    """Every row's chosen experts, clamps reached on both sides, against the plain experts one by one;
    widths that are and are not multiples of 16 (tensor-core tiles and the plain tiles)."""
    from starter_b200 import ops

    t = TORCH[dtype]
    g = torch.Generator().manual_seed(rows + experts)
    h = dev(torch.randn(rows, width, generator=g), t)
    gate_up = dev(torch.randn(experts, 2 * inner, width, generator=g) * 0.3, t)
    down = dev(torch.randn(experts, width, inner, generator=g) * 0.2, t)
    ids = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(rows)]).to(torch.int32).cuda()
    weights = torch.softmax(torch.randn(rows, top, generator=g), dim=-1).cuda()
    out = ops.moe_experts(h, ids, weights, gate_up, down, 1.25)
    w = {}
    for e in range(experts):
        w[f"e{e}.gate"], w[f"e{e}.up"] = gate_up[e, :inner].double().cpu(), gate_up[e, inner:].double().cpu()
        w[f"e{e}.down"] = down[e].double().cpu()
    h64 = h.double().cpu()
    want = torch.zeros(rows, width, dtype=F)
    reached = 0
    for r in range(rows):
        for c in range(top):
            e = int(ids[r, c])
            want[r] += weights[r, c].double().cpu() * plain.expert(h64[r:r + 1], w, f"e{e}.", 1.25)[0]
            reached += int(((h64[r] @ w[f"e{e}.gate"].T) > 1.25).any())
    assert reached > 0
    close(out, want, dtype, f"{rows} rows, {experts} experts")


@pytest.mark.parametrize("experts, top, width, inner", [(3, 2, 144, 80), (4, 1, 256, 128)])
def test_experts_on_every_tile_kind(experts, top, width, inner):
    """600 rows, so that the step chooses the tiles of 128 rows: those, the tiles of 64 and the plain tiles
    against the plain experts, with sizes that end inside a k-slice and inside a tile's outputs."""
    from starter_b200 import ops

    rows = 600
    g = torch.Generator().manual_seed(experts + width)
    h = dev(torch.randn(rows, width, generator=g), torch.bfloat16)
    gate_up = dev(torch.randn(experts, 2 * inner, width, generator=g) * 0.3, torch.bfloat16)
    down = dev(torch.randn(experts, width, inner, generator=g) * 0.2, torch.bfloat16)
    ids = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(rows)]).to(torch.int32)
    weights = torch.softmax(torch.randn(rows, top, generator=g), dim=-1)
    h64 = h.double().cpu()
    want = torch.zeros(rows, width, dtype=F)
    for e in range(experts):
        w = {"e.gate": gate_up[e, :inner].double().cpu(), "e.up": gate_up[e, inner:].double().cpu(),
             "e.down": down[e].double().cpu()}
        share = (weights * (ids == e)).sum(dim=1).double()
        used = share > 0
        want[used] += share[used, None] * plain.expert(h64[used], w, "e.", 1.25)
    assert ops._lib("moe").sb_moe_tile_rows_for(1, width, inner, rows * top, experts) in (128, 256)
    for tile_rows in (None, 4, 32, 64, 128, 256):
        out = ops.moe_experts(h, ids.cuda(), weights.cuda(), gate_up, down, 1.25, tile_rows=tile_rows)
        close(out, want, "bfloat16", f"tiles of {tile_rows or 'the chosen'} rows")


# ------------------------------------------------------------------------------ the model

def all_places(n):
    return list(range(n))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", CONFIGS)
def test_each_request_alone_and_whole(tmp_path_factory, name, dtype):
    from starter_b200.engine import StepEntry

    _, cfg, w = case(tmp_path_factory, name)
    routed = Routed(runner_for(tmp_path_factory, name, dtype))
    runner = routed.runner
    for length, seed in ((1, 1), (2, 2), (9, 3), (64, 4), (65, 5), (200, 6)):
        prompt = random_prompt(length, cfg["vocab"], seed)
        slot = runner.open_sequence()
        got = routed.step([StepEntry(slot, prompt, all_places(length))], [length])
        runner.close_sequence(slot)
        want = plain.forward(cfg, w, prompt, routes=routed.routes(length, dtype))
        assert_close(got, want, dtype, f"{name} whole, length {length}")
        assert_close(got[:3], want[:3], dtype, f"{name}: the first tokens of a sequence")
    runner.check_status()
    runner.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", CONFIGS)
def test_every_layer_against_the_plain_layers(tmp_path_factory, name, dtype):
    """The residual stream after each layer, which names the first layer that differs."""
    from starter_b200 import ops
    from starter_b200.engine import StepEntry

    _, cfg, w = case(tmp_path_factory, name)
    runner = runner_for(tmp_path_factory, name, dtype)
    model = runner.model
    prompt = random_prompt(90, cfg["vocab"], 8)
    slot = runner.open_sequence()
    ctx = runner.make_context([StepEntry(slot, prompt, [])])
    residual = ops.embedding32(ctx.tokens, model.embed, model.spec.embedding_scale, ctx.status)
    pending, got, routes = None, [], {}
    for i, entry in enumerate(model.spec.schedule):
        residual, pending = model.blocks[entry.layer](residual, pending, ctx, entry.cache, entry.writes_cache)
        after = residual.clone()
        ops.residual_norm(after, model.dtype, 0.0, pending.for_kernel(), None)
        got.append(after)
        ids = getattr(getattr(model.blocks[entry.layer], "feed_forward", None), "last_ids", None)
        if ids is not None:
            routes[i] = ids.cpu()
    runner.close_sequence(slot)
    want = []
    plain.forward(cfg, w, prompt, layers_out=want, routes=None if dtype == "float32" else routes)
    for i in range(len(want)):
        close(got[i], want[i], dtype, f"{name} after layer {i}", fp32=2e-5, bf16=2.5e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", CONFIGS)
def test_prompt_then_tokens_one_by_one(tmp_path_factory, name, dtype):
    """Windows of 3, 10, 64 and 65 pass over decoded tokens, and a page border is crossed while decoding."""
    from starter_b200.engine import StepEntry

    _, cfg, w = case(tmp_path_factory, name)
    routed = Routed(runner_for(tmp_path_factory, name, dtype))
    runner = routed.runner
    for length, tail in ((40, 39), (100, 45), (150, 90)):
        # (seeds chosen so that no first token lands on the ill-conditioned case described at BF16_ROW_TOL:
        # with seed 50 the scalar of KB's recurrent layer is 0.2% of its terms and bfloat16 cannot tell its sign)
        prompt = random_prompt(length, cfg["vocab"], 20 + length)
        slot = runner.open_sequence()
        head = length - tail
        rows = [routed.step([StepEntry(slot, prompt[:head], all_places(head))], [length])]
        for tok in prompt[head:]:
            rows.append(routed.step([StepEntry(slot, [tok], [0])], [length]))
        runner.close_sequence(slot)
        got = torch.cat(rows)
        want = plain.forward(cfg, w, prompt, routes=routed.routes(length, dtype))
        assert_close(got, want, dtype, f"{name} last {tail} one by one, length {length}")
        assert_close(got[head:head + 1], want[head:head + 1], dtype, "the first single-token step")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["KA", "KC"])
def test_long_decoding_over_many_pages(tmp_path_factory, name, dtype):
    """Two requests of unequal lengths decoded together for 300 steps, the longer one over six pages; the
    shorter one ends on the way; every logit is held to the plain statement."""
    from starter_b200.engine import StepEntry

    _, cfg, w = case(tmp_path_factory, name)
    routed = Routed(runner_for(tmp_path_factory, name, dtype))
    runner = routed.runner
    lengths, heads = (380, 150), (80, 3)
    prompts = [random_prompt(n, cfg["vocab"], 300 + n) for n in lengths]
    slots = [runner.open_sequence() for _ in prompts]
    first = routed.step([StepEntry(s, p[:h], all_places(h)) for s, p, h in zip(slots, prompts, heads)], [0, 1])
    got = [[first[:heads[0]]], [first[heads[0]:]]]
    at = list(heads)
    while at[0] < lengths[0]:
        live = [i for i in range(2) if at[i] < lengths[i]]
        rows = routed.step([StepEntry(slots[i], [prompts[i][at[i]]], [0]) for i in live], live)
        for k, i in enumerate(live):
            got[i].append(rows[k:k + 1])
            at[i] += 1
            if at[i] == lengths[i]:
                runner.close_sequence(slots[i])
    for i in range(2):
        want = plain.forward(cfg, w, prompts[i], routes=routed.routes(i, dtype))
        assert_close(torch.cat(got[i]), want, dtype, f"{name} request {i} decoded to {lengths[i]}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", CONFIGS)
def test_portions_of_several_sizes(tmp_path_factory, name, dtype):
    from starter_b200.engine import StepEntry

    _, cfg, w = case(tmp_path_factory, name)
    prompt = random_prompt(171, cfg["vocab"], 77)
    for sizes in ((2, 2, 3, 57, 64, 1, 40, 2), (63, 2, 63, 43), (5, 128, 38)):
        routed = Routed(runner_for(tmp_path_factory, name, dtype))
        runner = routed.runner
        slot = runner.open_sequence()
        rows, at = [], 0
        for n in sizes:
            rows.append(routed.step([StepEntry(slot, prompt[at:at + n], all_places(n))], [0]))
            at += n
        assert at == len(prompt)
        runner.close_sequence(slot)
        want = plain.forward(cfg, w, prompt, routes=routed.routes(0, dtype))
        assert_close(torch.cat(rows), want, dtype, f"{name} portions {sizes}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", CONFIGS)
def test_unequal_batches_with_slots_pages_and_states_used_again(tmp_path_factory, name, dtype):
    from starter_b200.engine import StepEntry

    _, cfg, w = case(tmp_path_factory, name)
    runner = runner_for(tmp_path_factory, name, dtype)
    vocab = cfg["vocab"]
    batches = [[(70, 9), (5, 3), (33, 12), (1, 6)], [(2, 40), (129, 2), (64, 5)], [(17, 0), (63, 3)]]
    seed = 300
    for batch in batches:
        routed = Routed(runner)
        seqs, slots, got = [], [], []
        for plen, extra in batch:
            seed += 1
            seqs.append(random_prompt(plen + extra, vocab, seed))
            slots.append(runner.open_sequence())
            got.append([])
        first = routed.step([StepEntry(slots[i], seqs[i][:plen], all_places(plen)) for i, (plen, _) in enumerate(batch)],
                            list(range(len(batch))))
        offset = 0
        for i, (plen, _) in enumerate(batch):
            got[i].append(first[offset:offset + plen])
            offset += plen
        live = [i for i, (_, extra) in enumerate(batch) if extra > 0]
        for i, (_, extra) in enumerate(batch):
            if extra == 0:
                runner.close_sequence(slots[i])
        step = 0
        while live:
            out = routed.step([StepEntry(slots[i], [seqs[i][batch[i][0] + step]], [0]) for i in live], live)
            for row, i in enumerate(live):
                got[i].append(out[row:row + 1])
            step += 1
            for i in [i for i in live if batch[i][1] == step]:
                runner.close_sequence(slots[i])
            live = [i for i in live if batch[i][1] > step]
        for i, seq in enumerate(seqs):
            want = plain.forward(cfg, w, seq, routes=routed.routes(i, dtype))
            assert_close(torch.cat(got[i]), want, dtype, f"{name} batch {batch}, request {i}")
        runner.cache.check()
    assert runner.cache.slots.held_count == 0 and runner.cache.pages.held_count == 0


@pytest.mark.parametrize("name", CONFIGS)
def test_greedy_generation_through_the_entry_point(tmp_path_factory, name):
    """Unequal prompts through ``Engine.generate`` (the scheduler, the captured single-token step with its
    saved and restored recurrent state, the sampler): 70 tokens each, past a page border and past every
    window, equal to the plain statement's greedy continuation."""
    from starter_b200 import Engine

    folder, cfg, w = case(tmp_path_factory, name)
    engine = Engine(folder, dtype="float32", max_batch=4)
    prompts = [random_prompt(n, cfg["vocab"], 900 + n) for n in (50, 3, 21)]
    steps = list(engine.generate(prompts, 70))
    assert len(steps) == 70
    for i, prompt in enumerate(prompts):
        assert [s[i] for s in steps] == plain.generate(cfg, w, prompt, 70), f"request {i}"


def test_random_weights_from_the_library_run_in_bfloat16():
    """``random_model`` places every tensor as the loader would, and sampling with temperature runs."""
    from starter_b200 import Engine
    from starter_b200.config import config_from_dict
    from starter_b200.engine.runner import random_model

    model = random_model(config_from_dict(TINY_K["KC"]), seed=5, dtype="bfloat16")
    engine = Engine.from_model(model, max_batch=2)
    out = engine.complete([[1, 2, 3], [4]], 12, temperature=0.8, seed=3)
    assert [len(c.tokens) for c in out] == [12, 12]
    assert all(0 <= t < 257 for c in out for t in c.tokens)


# ------------------------------------------------------------------------------ the programs

def test_command_line_and_trace_replay(tmp_path_factory, tmp_path):
    """``python -m starter_b200 generate`` and ``bin/trace_run`` pick the design by its config.json (this
    folder's config leaves the decay rank to the checkpoint)."""
    import json
    import os
    import subprocess
    import sys

    import numpy as np

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    folder, cfg, w = case(tmp_path_factory, "KB")
    prompts = [random_prompt(5, cfg["vocab"], 1), random_prompt(19, cfg["vocab"], 2)]
    text = ";".join(",".join(str(t) for t in p) for p in prompts)
    out = subprocess.run([sys.executable, "-m", "starter_b200", "generate", "--model-path", folder, "--input-ids", text,
                          "--max-new-tokens", "6", "--dtype", "float32"], cwd=root, capture_output=True, text=True,
                         timeout=600)
    assert out.returncode == 0, out.stderr
    lines = [json.loads(line) for line in out.stdout.splitlines() if line.startswith("{")]
    assert [line["tokens"] for line in lines] == [plain.generate(cfg, w, p, 6) for p in prompts]

    # a trace: two unequal requests start together, are decoded together, the shorter one ends first
    a, b = random_prompt(140, cfg["vocab"], 5), random_prompt(70, cfg["vocab"], 6)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:130], "want": [0, 129]},
                                     {"id": "b", "tokens": b[:66], "want": [65]}], "end": []}]
    for i in range(10):
        entries = [{"id": "a", "tokens": [a[130 + i]], "want": [0]}]
        if i < 4:
            entries.append({"id": "b", "tokens": [b[66 + i]], "want": [0] if i % 2 else []})
        steps.append({"step": 1 + i, "entries": entries, "end": (["b"] if i == 3 else []) + (["a"] if i == 9 else [])})
    out_dir = str(tmp_path / "float32")
    proc = subprocess.Popen([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
                             "--out", out_dir, "--max-tokens", "210"], stdin=subprocess.PIPE, stdout=subprocess.PIPE,
                            text=True)
    for record in steps:
        proc.stdin.write(json.dumps(record) + "\n")
        proc.stdin.flush()
        assert proc.stdout.readline().strip() == f"done {record['step']}"
    proc.stdin.close()
    assert proc.wait(timeout=120) == 0
    want_a, want_b = plain.forward(cfg, w, a), plain.forward(cfg, w, b)
    read = lambda s: torch.from_numpy(np.fromfile(os.path.join(out_dir, f"{s}.f32"), dtype="<f4").reshape(-1, cfg["vocab"]))  # noqa: E731
    assert_close(read(0), torch.stack([want_a[0], want_a[129], want_b[65]]), "float32", "the first step")
    for i in range(10):
        rows = [want_a[130 + i]] + ([want_b[66 + i]] if i < 4 and i % 2 else [])
        assert_close(read(1 + i), torch.stack(rows), "float32", f"step {1 + i}")
