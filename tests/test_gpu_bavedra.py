"""Bavedra on the GPU against the plain statement: each mechanism alone, then the model through the step
function, the cache, the state slots and the generation loop, cut into steps and batches in every way."""

import pytest
import torch

import plain_bavedra as plain
from gpu_helpers import DTYPES, FP32_TOL
from tiny import random_prompt
from tiny_bavedra import TINY_B, make_bavedra_folder

pytestmark = pytest.mark.gpu

CONFIGS = ["BA", "BB", "BC"]
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}
F = torch.float64
_cases, _runners = {}, {}


def case(tmp_path_factory, name, seed=1):
    if (name, seed) not in _cases:
        folder = make_bavedra_folder(tmp_path_factory.mktemp(f"b{name}{seed}"), name, seed=seed)
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


# Bounds of the model-level comparisons, relative to the largest logit of the case.  float32: as for the other
# designs.  bfloat16 against the float64 statement: a row may be off by 6e-2 and the mean over a comparison by
# 1e-2 of the largest logit (measured on these configurations: rows up to 3e-2, means about 4e-3); a lost state, a
# key that is one off or a skipped layer moves rows by 1e-1 and more, and the float32 runs of the same kernels
# hold every row to 2e-5.
BF16_ROW_TOL = 6e-2
BF16_MEAN_TOL = 1e-2


def assert_close(got, want, dtype, what=""):
    """Fails with the first wrong row named: its place is the clue (a prompt's end, the first single-token
    step, a page boundary, a window's edge)."""
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


def ints(a):
    return torch.tensor(a, dtype=torch.int32, device="cuda")


def packed(lengths, slots):
    """(seq_slot, seq_q_start, seq_q_len) on the device for sequences packed one after another."""
    starts = [sum(lengths[:i]) for i in range(len(lengths))]
    return ints(slots), ints(starts), ints(lengths)


class Routed:
    """Runs steps and notes, per request, which experts every routed layer chose for each of its tokens.
    The 32-bit comparisons do not use the notes (there the choice itself is held to the plain statement);
    the bfloat16 comparisons hand them to the plain statement, because a near-tie between two experts may
    fall either way once the router's input is rounded to 8 bits, and that is no fault."""

    def __init__(self, runner):
        self.runner = runner
        model = runner.model
        # per run of a layer (a layer may run several times): the place in the run order and its block
        self.runs = [(i, model.blocks[e.layer]) for i, e in enumerate(model.spec.schedule)
                     if hasattr(getattr(model.blocks[e.layer], "feed_forward", None), "last_ids")]
        self.shared = len({id(b) for _, b in self.runs}) < len(self.runs)
        self.notes = {}

    def step(self, entries, keys):
        if not self.shared:
            out = self.runner.step(entries)
            self._note(entries, keys, {i: b.feed_forward.last_ids for i, b in self.runs})
            return out
        # a routed layer that runs twice overwrites its note: catch each run's choice as it is made
        caught = {}
        order = iter([i for i, _ in self.runs])
        cls = type(self.runs[0][1].feed_forward)
        old = cls.__call__

        def wrapped(ff, x, ctx=None):
            out = old(ff, x, ctx)
            caught[next(order)] = ff.last_ids
            return out

        cls.__call__ = wrapped
        try:
            out = self.runner.step(entries)
        finally:
            cls.__call__ = old
        self._note(entries, keys, caught)
        return out

    def _note(self, entries, keys, ids_of):
        at = 0
        for entry, key in zip(entries, keys):
            n = len(entry.tokens)
            for place, ids in ids_of.items():
                self.notes.setdefault(key, {}).setdefault(place, []).append(ids[at:at + n].cpu())
            at += n

    def routes(self, key, dtype):
        if dtype == "float32" or not self.runs:
            return None
        return {place: torch.cat(parts) for place, parts in self.notes[key].items()}


# ------------------------------------------------------------------------------ mechanisms alone

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("channels, taps, col, act", [(40, 4, 8, "silu"), (33, 2, 0, None), (130, 3, 5, "silu"), (16, 1, 3, None),
                                                       (24, 8, 0, "silu")])
def test_short_convolution_alone(channels, taps, col, act, dtype):
    """Three sequences whole in one step, then cut into portions down to one token over several steps with the
    last inputs carried in their slots, a portion shorter than the filter among them; the channels are a slice
    of wider rows; a slot used before is zeroed as the cache does."""
    from starter_b200 import ops

    t = TORCH[dtype]
    g = torch.Generator().manual_seed(channels + taps)
    lengths, slots = [150, 1, 37], [3, 0, 2]
    total, ld = sum(lengths), col + channels + 3
    x = dev(torch.randn(total, ld, generator=g, dtype=F), t)
    w = torch.randn(channels, taps, generator=g, dtype=F)
    bias = torch.randn(channels, generator=g, dtype=F)
    in_bias = torch.randn(channels, generator=g, dtype=F) if col else None
    xs = x.double().cpu()[:, col:col + channels] + (in_bias if in_bias is not None else 0.0)
    want, at = [], 0
    for n in lengths:
        y = plain.short_convolution(xs[at:at + n], w, bias)
        want.append(plain.silu(y) if act else y)
        at += n
    want = torch.cat(want)
    state_at = 7
    state = torch.full((5, state_at + (taps - 1) * channels + 2), 9.0, device="cuda")
    state[:, state_at:state_at + (taps - 1) * channels] = 0.0
    args = (dev(w), dev(bias), dev(in_bias) if in_bias is not None else None, state, state_at)
    out = ops.short_conv(x, col, channels, *args, *packed(lengths, slots), max(lengths), act)
    close(out, want, dtype, "whole")
    assert float(state[:, :state_at].min()) == 9.0 and float(state[:, -2:].min()) == 9.0       # nothing beside it is touched
    state[:, state_at:state_at + (taps - 1) * channels] = 0.0
    got = [[], [], []]
    done = [0, 0, 0]
    bases = [0, 150, 151]
    for sizes in ([2, 1, 1], [1, 0, 2], [64, 0, 1], [3, 0, 33], [80, 0, 0]):
        live = [i for i in range(3) if sizes[i]]
        rows = torch.cat([x[bases[i] + done[i]:bases[i] + done[i] + sizes[i]] for i in live])
        out = ops.short_conv(rows.contiguous(), col, channels, *args, *packed([sizes[i] for i in live], [slots[i] for i in live]),
                             max(sizes), act)
        at = 0
        for i in live:
            got[i].append(out[at:at + sizes[i]])
            at += sizes[i]
            done[i] += sizes[i]
    assert done == lengths
    close(torch.cat([torch.cat(p) for p in got]), want, dtype, "in portions")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("channels, blocks", [(96, 3), (40, 1), (256, 4), (7, 7)])
def test_gated_linear_recurrence_alone(channels, blocks, dtype):
    """A sequence of 700 tokens (cut into segments that run side by side and are chained) next to short ones, then
    the same in portions down to one token; the channels' memory spreads from one token to thousands, and what the
    first token wrote is still read at the end."""
    from starter_b200 import ops

    t = TORCH[dtype]
    g = torch.Generator().manual_seed(channels)
    lengths, slots = [700, 2, 45], [1, 4, 0]
    total, bs = sum(lengths), channels // blocks
    u = dev(torch.randn(total, channels, generator=g, dtype=F), t)
    u[0] = 30.0                                                      # a first token that stands out
    gates = dev(torch.randn(blocks, total, 2 * bs, generator=g, dtype=F) * 2.0)
    rb, ib = torch.randn(channels, generator=g, dtype=F), torch.randn(channels, generator=g, dtype=F)
    lam = torch.linspace(-9.0, 2.0, channels, dtype=F)
    yb = torch.randn(channels, generator=g, dtype=F)
    proj = dev(torch.randn(total, channels + 5, generator=g, dtype=F), t)
    zr = gates.double().cpu()[:, :, :bs].permute(1, 0, 2).reshape(total, channels)
    zi = gates.double().cpu()[:, :, bs:].permute(1, 0, 2).reshape(total, channels)
    r, i = torch.sigmoid(zr + rb), torch.sigmoid(zi + ib)
    y = plain.gelu_tanh(proj.double().cpu()[:, 5:] + yb)
    want, at = [], 0
    for n in lengths:
        part = slice(at, at + n)
        want.append(plain.gated_linear_recurrence(u.double().cpu()[part], r[part], i[part], lam) * y[part])
        at += n
    want = torch.cat(want)
    # the long-memory channels still hold the first token at the end
    without = u.double().cpu()[:700].clone()
    without[0] = 0.0
    forgot = plain.gated_linear_recurrence(without, r[:700], i[:700], lam) * y[:700]
    assert float((forgot[699] - want[699]).abs().max()) > 0.02
    state = torch.zeros(6, 3 + channels, device="cuda")
    consts = (dev(rb), dev(ib), dev(lam), 8.0)
    out = ops.glru_scan(u, gates, *consts, proj, 5, dev(yb), state, 3, *packed(lengths, slots), max(lengths))
    close(out, want, dtype, "whole", fp32=3e-5)
    state.zero_()
    got, done, bases = [[], [], []], [0, 0, 0], [0, 700, 702]
    for sizes in ([1, 1, 2], [2, 1, 1], [300, 0, 40], [17, 0, 2], [380, 0, 0]):
        live = [k for k in range(3) if sizes[k]]
        rows = torch.cat([torch.arange(bases[k] + done[k], bases[k] + done[k] + sizes[k]) for k in live]).cuda()
        out = ops.glru_scan(u[rows].contiguous(), gates[:, rows].contiguous(), *consts, proj[rows].contiguous(), 5, dev(yb),
                            state, 3, *packed([sizes[k] for k in live], [slots[k] for k in live]), max(sizes))
        at = 0
        for k in live:
            got[k].append(out[at:at + sizes[k]])
            at += sizes[k]
            done[k] += sizes[k]
    close(torch.cat([torch.cat(p) for p in got]), want, dtype, "in portions", fp32=3e-5)


def scan_inputs(heads, groups, n, v, lengths, seed, t):
    g = torch.Generator().manual_seed(seed)
    total = sum(lengths)
    q = dev(torch.randn(total, groups * n + 3, generator=g, dtype=F), t)
    k = dev(torch.randn(total, 2 + groups * n, generator=g, dtype=F), t)
    val = dev(torch.randn(total, heads * v, generator=g, dtype=F), t)
    raw = dev(torch.randn(total, 2 * heads + 1, generator=g, dtype=F), t)       # [b | a | unused]
    A_log = torch.linspace(-7.0, 0.5, heads, dtype=F)
    dt_bias = torch.randn(heads, generator=g, dtype=F) * 0.5
    return q, k, val, raw, A_log, dt_bias


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, groups, n, v", [(3, 1, 12, 8), (2, 2, 33, 20), (4, 2, 64, 32), (2, 1, 128, 64), (1, 1, 256, 100),
                                                 (6, 3, 5, 48), (2, 2, 40, 24), (1, 1, 1, 1)])
@pytest.mark.parametrize("mode", ["state_space", "gated_delta"])
def test_matrix_state_recurrences_alone(mode, heads, groups, n, v, dtype):
    """Both recurrences whole, then in portions down to one token across the kernel's chunks of 16 with the state
    carried in the slots; the first head hardly decays, and the first token's key and value are made large, so that
    300 tokens later the read-out still shows whether the state was kept."""
    from starter_b200 import ops

    t = TORCH[dtype]
    lengths, slots = [300, 1, 18], [2, 0, 3]
    q, k, val, raw, A_log, dt_bias = scan_inputs(heads, groups, n, v, lengths, heads * 1000 + n, t)
    k[0] *= 4.0
    val[0] *= 4.0
    skip = torch.linspace(-1.0, 2.0, heads, dtype=F)
    qq = q.double().cpu()[:, :groups * n].reshape(-1, groups, n)
    kk = k.double().cpu()[:, 2:].reshape(-1, groups, n)
    vv = val.double().cpu().reshape(-1, heads, v)
    a_raw, b_raw = raw.double().cpu()[:, heads:2 * heads], raw.double().cpu()[:, :heads]
    dt = plain.softplus(a_raw + dt_bias)
    want, at = [], 0
    for length in lengths:
        part = slice(at, at + length)
        if mode == "state_space":
            want.append(plain.state_space_recurrence(vv[part], kk[part], qq[part], dt[part], A_log, skip))
        else:
            decay = torch.exp(-torch.exp(A_log) * dt[part])
            want.append(plain.delta_recurrence(plain.unit(qq[part]) * n ** -0.5, plain.unit(kk[part]), vv[part],
                                               torch.sigmoid(b_raw[part]), decay))
        at += length
    want = torch.cat(want).reshape(-1, heads * v)
    state_at = 5
    state = torch.zeros(4, state_at + heads * n * v + 1, device="cuda")
    consts = (dev(A_log), dev(dt_bias), dev(skip) if mode == "state_space" else None, state, state_at)
    b_pair = None if mode == "state_space" else lambda r: (r, 0)

    def run(rows, lens, sl):
        pick = (lambda x: x) if rows is None else (lambda x: x[rows].contiguous())
        rr = pick(raw)
        return ops.state_scan(mode, (pick(q), 0), (pick(k), 2), (pick(val), 0), (rr, heads), None if b_pair is None else b_pair(rr),
                              *consts, *packed(lens, sl), heads, groups, n, v)

    out = run(None, lengths, slots)
    # the float bound: sums of up to 256 products in another order than the statement's
    close(out, want, dtype, "whole", fp32=5e-5, bf16=2e-2)
    state.zero_()
    got, done, bases = [[], [], []], [0, 0, 0], [0, 300, 301]
    for sizes in ([1, 1, 1], [2, 0, 1], [16, 0, 15], [33, 0, 1], [248, 0, 0]):
        live = [i for i in range(3) if sizes[i]]
        rows = torch.cat([torch.arange(bases[i] + done[i], bases[i] + done[i] + sizes[i]) for i in live]).cuda()
        out = run(rows, [sizes[i] for i in live], [slots[i] for i in live])
        at = 0
        for i in live:
            got[i].append(out[at:at + sizes[i]])
            at += sizes[i]
            done[i] += sizes[i]
    close(torch.cat([torch.cat(p) for p in got]), want, dtype, "in portions", fp32=5e-5, bf16=2e-2)
    assert float(want[299].abs().max()) > 1e-3


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_in_parts_with_a_gate_and_mean_of_two_normed_rows(dtype):
    from starter_b200 import ops

    t = TORCH[dtype]
    g = torch.Generator().manual_seed(3)
    for parts, psize, shared in ((1, 40, False), (3, 8, False), (4, 64, True), (5, 7, True), (2, 600, False)):
        o = dev(torch.randn(6, parts * psize, generator=g, dtype=F) * 3.0)
        z = dev(torch.randn(6, parts * psize + 4, generator=g, dtype=F), t)
        w = torch.randn(psize if shared else parts * psize, generator=g, dtype=F)
        zz, oo = z.double().cpu()[:, 4:], o.double().cpu()
        full = w.repeat(parts) if shared else w
        first = plain.rms((oo * plain.silu(zz)).reshape(6, parts, psize), 1e-5).reshape(6, -1) * full
        second = plain.rms(oo.reshape(6, parts, psize), 1e-5).reshape(6, -1) * full * plain.silu(zz)
        close(ops.group_norm_gate(o, z, 4, dev(w), parts, 1e-5, True, t), first, dtype, f"gate first, {parts} x {psize}")
        close(ops.group_norm_gate(o, z, 4, dev(w), parts, 1e-5, False, t), second, dtype, f"norm first, {parts} x {psize}")
    for width in (37, 64, 1000, 5000):
        a = dev(torch.randn(5, width, generator=g, dtype=F) * 2.0, t)
        b = dev(torch.randn(5, width, generator=g, dtype=F) * 0.1, t)
        wa, wb = torch.randn(width, generator=g, dtype=F), torch.randn(width, generator=g, dtype=F)
        want = 0.5 * (plain.norm(a.double().cpu(), wa, 1e-6) + plain.norm(b.double().cpu(), wb, 1e-6))
        close(ops.norm_pair_mean(a, b, dev(wa), dev(wb), 1e-6), want, dtype, f"pair of width {width}")


def tables(base, dims, length):
    i = torch.arange(dims // 2, dtype=F)
    angle = torch.outer(torch.arange(length, dtype=F), base ** (-2.0 * i / dims))
    return dev(angle.cos()), dev(angle.sin())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv_heads, dim, rot, window", [(4, 2, 16, 8, 10), (1, 1, 24, 24, 3), (8, 2, 64, 32, 65), (4, 4, 32, 0, 64),
                                                               (2, 1, 128, 2, 130), (3, 3, 10, 4, None)])
def test_rotated_window_attention_with_a_sink_alone(heads, kv_heads, dim, rot, window, dtype):
    """A sequence of 300 over five scattered pages, filed by the rotating prepare kernel (keys turned, values the
    keys as projected), queries turned in place; queries late in the sequence aim at one key: the first key inside
    their window, the one just outside it, keys on either side of a page border, their own place; the answer holds
    that key's value or, outside the window, falls to the sink.  Plain and tensor-core kernels, whole, as a later
    portion and as the last token alone in 1, 3 and 7 parts."""
    from starter_b200 import ops

    t = TORCH[dtype]
    n, scale, base = 300, 0.25, 1000.0
    g = torch.Generator().manual_seed(heads * 100 + dim)
    group = heads // kv_heads
    q = torch.randn(n, heads, dim, generator=g, dtype=F)
    k = torch.randn(n, kv_heads, dim, generator=g, dtype=F)
    pos = torch.arange(n)
    turn = (lambda x: plain.rotate_pairs(x, pos, base, rot)) if rot else (lambda x: x)
    span = window or n
    probes = {}
    for q_pos in (299, 290, 257, 200, 193, 130, 129, 70):
        first = max(q_pos - span + 1, 0)
        probes[q_pos] = first                           # the oldest key it still sees
        if first >= 1:
            probes[q_pos - 1] = first - 1               # the query before it: its own oldest key
            probes[q_pos - 2] = first - 3 if first >= 3 else 0      # and one aimed at a key just behind its window
    probes[280], probes[191] = 280, max(128, 191 - span + 1)
    outside = {}
    for q_pos in (295, 260, 135):
        if q_pos - span >= 0:
            outside[q_pos] = q_pos - span               # the key just outside the window
    for table_ in (probes, outside):
        for q_pos, key in table_.items():
            for h in range(heads):
                # aim in rotated space: the query that, once turned to q_pos, lines up with the key turned to its place
                target = turn(k)[key, h // group]
                aimed = target / target.norm() * (40.0 / scale / max(1.0, float(target.norm())))
                if rot:
                    back = plain.rotate_pairs(aimed[None, None, :], torch.tensor([-q_pos]), base, rot)[0, 0]
                else:
                    back = aimed
                q[q_pos, h] = back
    width = heads * dim + kv_heads * dim
    proj = torch.zeros(n, width + (-width % 8), dtype=F)
    proj[:, :heads * dim] = q.reshape(n, -1)
    proj[:, heads * dim:width] = k.reshape(n, -1)
    proj = dev(proj, t)
    qd = proj.double().cpu()[:, :heads * dim].reshape(n, heads, dim)
    kd = proj.double().cpu()[:, heads * dim:width].reshape(n, kv_heads, dim)
    want = plain.window_attention(turn(qd), turn(kd), kd, scale, span).reshape(n, heads * dim)
    if outside:
        # a query aimed at the key just outside its window gets next to nothing of it
        probe = next(iter(outside))
        seen = plain.window_attention(turn(qd), turn(kd), kd, scale, span + 1).reshape(n, heads * dim)
        assert float((seen[probe] - want[probe]).abs().max()) > 0.3
    table = torch.zeros(3, 8, dtype=torch.int32, device="cuda")
    table[1, :5] = ints([5, 2, 7, 0, 3])
    ks = torch.zeros(8, kv_heads, 64, dim, dtype=t, device="cuda")
    vs = torch.zeros(8, kv_heads, 64, dim, dtype=t, device="cuda")
    cos, sin = tables(base, rot, 512) if rot else (None, None)
    posd, slot = torch.arange(n, dtype=torch.int32, device="cuda"), torch.ones(n, dtype=torch.int32, device="cuda")
    ops.sink_prepare_rot(proj, heads, kv_heads, dim, dim, posd, slot, table, ks, vs, cos, sin, rot, values_from_keys=True)
    # what lies in the cache: turned keys, and the keys as projected as values, on both sides of page borders
    for p_ in (0, 63, 64, 65, 191, 192, 299):
        page = int(table[1, p_ // 64])
        close(ks[page, :, p_ % 64], turn(kd)[p_], dtype, f"key {p_}", fp32=1e-6, bf16=8e-3)
        assert torch.equal(vs[page, :, p_ % 64].double().cpu(), kd[p_]), p_
    close(proj[:, :heads * dim], turn(qd).reshape(n, -1), dtype, "queries turned in place", fp32=1e-6, bf16=8e-3)
    sink = torch.zeros(heads, device="cuda")
    out = ops.sink_attention(proj, ks, vs, table, slot, posd, heads, kv_heads, dim, dim, scale, None, sink, None, None, window)
    close(out, want, dtype, "plain kernel, whole", bf16=3e-2)
    if not ops.sink_tc_takes(proj, heads, kv_heads, dim, dim):
        return
    out = ops.sink_attention_tc(proj, ks, vs, table, ints([1]), ints([0]), ints([n]), ints([n]), ints([0, 0, 0, 0, 0]),
                                ints([128, 0, 256, 192, 64]), heads, kv_heads, dim, dim, scale, None, sink, None, None, window)
    close(out, want, dtype, "tensor cores, whole", bf16=3e-2)
    tail = proj[260:].contiguous()
    out = ops.sink_attention_tc(tail, ks, vs, table, ints([1]), ints([0]), ints([40]), ints([n]), ints([0]), ints([0]), heads,
                                kv_heads, dim, dim, scale, None, sink, None, None, window)
    close(out, want[260:], dtype, "tensor cores, a later portion", bf16=3e-2)
    for parts in (1, 3, 7):
        out = ops.sink_attention_tc(proj[299:].contiguous(), ks, vs, table, ints([1]), ints([0]), ints([1]), ints([n]), ints([0]),
                                    ints([0]), heads, kv_heads, dim, dim, scale, None, sink, None, None, window, n_splits=parts)
        close(out, want[299:], dtype, f"tensor cores, one token in {parts} parts", bf16=3e-2)
    if ops.sink_tcgen05_takes(proj, dim, dim):
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        out = ops.sink_attention_tcgen05(proj, ks, vs, table, ints([1]), ints([0]), ints([n]), ints([n]), ints([0, 0, 0, 0, 0]),
                                         ints([128, 0, 256, 192, 64]), heads, kv_heads, dim, scale, None, sink, None, None,
                                         window, status, (ints([0, 0]), ints([0, 256])))
        close(out, want, dtype, "tcgen05, whole", bf16=3e-2)
        assert int(status.item()) == 0


@pytest.mark.parametrize("outputs, top, groups, keep, gate", [(6, 2, 3, 2, True), (12, 3, 2, 1, True), (3, 3, 1, 1, False), (16, 2, 4, 2, False),
                                                              (64, 8, 8, 4, True), (5, 1, 5, 1, False), (6, 1, 2, 1, True)])
def test_router_over_all_scores_alone(outputs, top, groups, keep, gate):
    """The choice against the plain statement, with rows whose scores tie (the lower index wins), with corrections
    large enough to move the choice across groups, and with the shared expert's gate as the router's last row."""
    from starter_b200 import ops

    g = torch.Generator().manual_seed(outputs * 10 + top)
    width = 48
    h = torch.randn(40, width, generator=g, dtype=F)
    h[5] = 0.0                                                   # every score equal: the first of the kept groups win
    h[6] = h[7]
    router = torch.randn(outputs, width, generator=g, dtype=F) * 0.5
    router[1] = router[0]                                        # two outputs that always tie
    correction = torch.randn(outputs, generator=g, dtype=F) * 0.1
    correction[1] = correction[0]
    sg = torch.randn(1, width, generator=g, dtype=F)
    w = {"r.router": router.float().double(), "r.correction": correction.float().double()}
    hh = dev(h)
    index, weight, _ = plain.route(hh.double().cpu(), w, "r.", dict(top=top, groups=dict(count=groups, keep=keep)))
    stacked = dev(torch.cat([router, sg]) if gate else router)
    out = ops.moe_route_all(hh, stacked, dev(correction), top, groups, keep, shared_gate=gate)
    assert torch.equal(out[0].cpu().long(), index)
    close(out[1], weight, "float32", "weights", fp32=1e-5)
    if gate:
        close(out[2], torch.sigmoid(hh.double().cpu() @ sg.float().double().T)[:, 0], "float32", "the shared expert's gate", fp32=1e-5)
    # without a correction the choice goes by the plain scores
    w["r.correction"] = torch.zeros(outputs, dtype=F)
    index, _, _ = plain.route(hh.double().cpu(), w, "r.", dict(top=top, groups=dict(count=groups, keep=keep)))
    assert torch.equal(ops.moe_route_all(hh, dev(router), None, top, groups, keep)[0].cpu().long(), index)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows", [1, 5, 70, 700])
@pytest.mark.parametrize("experts, identity, top, width, inner", [(5, 1, 2, 64, 24), (3, 0, 3, 96, 32), (8, 8, 2, 128, 64), (4, 2, 1, 40, 20)])
def test_gated_experts_with_identity_and_shared_experts_alone(experts, identity, top, width, inner, rows, dtype):
    """Given choices that include identity experts (one row chooses nothing else), on whichever tile kernel the
    step's shape picks, with a shared expert's output added times its gate; against the plain experts."""
    from starter_b200 import ops

    t = TORCH[dtype]
    g = torch.Generator().manual_seed(rows + experts)
    outputs = experts + identity
    h = dev(torch.randn(rows, width, generator=g, dtype=F), t)
    gate_up = dev(torch.randn(experts, 2 * inner, width, generator=g, dtype=F) * 0.3, t)
    down = dev(torch.randn(experts, width, inner, generator=g, dtype=F) * 0.3, t)
    ids = torch.stack([torch.randperm(outputs, generator=g)[:top] for _ in range(rows)]).int()
    if identity >= top:
        ids[0] = torch.arange(experts, experts + top)
    weights = torch.rand(rows, top, generator=g, dtype=F).float()
    shared = dev(torch.randn(rows, width, generator=g, dtype=F), t)
    sgate = torch.rand(rows, generator=g, dtype=F).float()
    h64 = h.double().cpu()
    want = sgate.double()[:, None] * shared.double().cpu()
    for e in range(outputs):
        share = (weights * (ids == e)).sum(dim=1).double()
        used = share > 0
        if e >= experts:
            want[used] += share[used, None] * h64[used]
        else:
            w = {"e.gate": gate_up[e, :inner].double().cpu(), "e.up": gate_up[e, inner:].double().cpu(),
                 "e.down": down[e].double().cpu()}
            want[used] += share[used, None] * plain.gated_expert(h64[used], w, "e.")
    out = ops.moe_experts(h, ids.cuda(), weights.cuda(), gate_up, down, expert="gated_silu", identity=identity > 0,
                          shared=shared, shared_gate=sgate.cuda())
    close(out, want, dtype, "the step's own tiles", bf16=2.5e-2)
    if dtype == "bfloat16" and width % 16 == 0 and inner % 16 == 0:
        for tile_rows in (4, 32, 64, 128, 256):
            out = ops.moe_experts(h, ids.cuda(), weights.cuda(), gate_up, down, expert="gated_silu", tile_rows=tile_rows,
                                  identity=identity > 0, shared=shared, shared_gate=sgate.cuda())
            close(out, want, dtype, f"tiles of {tile_rows} rows", bf16=2.5e-2)


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
    """The residual stream after each run of a layer, which names the first one that differs."""
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
    assert len(want) == len(cfg["layers"]) == len(got)
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
@pytest.mark.parametrize("name", ["BA", "BC"])
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


def test_a_layer_in_front_of_the_layer_whose_weights_it_runs(tmp_path_factory):
    """``weights_of`` naming a later layer, and a layer that names one which itself borrows: each run has a state of
    its own, whatever the order."""
    import copy

    from starter_b200.engine import ModelRunner, StepEntry, load_model

    raw = copy.deepcopy(TINY_B["BA"])
    raw["layers"] = [dict(raw["layers"][2], weights_of=3)] + raw["layers"]
    raw["layers"][5]["weights_of"] = 0
    folder = make_bavedra_folder(tmp_path_factory.mktemp("fw"), "FW", seed=3, raw=raw)
    cfg, w = plain.read_model_folder(folder)
    runner = ModelRunner(load_model(folder, "float32"), max_tokens=64 * 8, max_sequences=4, use_graphs=False)
    prompt = random_prompt(70, cfg["vocab"], 4)
    slot = runner.open_sequence()
    got = [runner.step([StepEntry(slot, prompt[:50], all_places(50))])]
    got += [runner.step([StepEntry(slot, [tok], [0])]) for tok in prompt[50:]]
    runner.close_sequence(slot)
    assert_close(torch.cat(got), plain.forward(cfg, w, prompt), "float32", "a borrowed layer in front")


@pytest.mark.parametrize("seed", range(10))
def test_configurations_drawn_at_random(tmp_path_factory, seed):
    """Layer kinds, their order, every size, head count, window, tap count, group and constant drawn anew: three
    unequal requests whole and alone, then begun together and decoded together, then one in portions, in float32
    (the choice of experts itself is held) and, whole, in bfloat16 with the engine's choices handed over.  The
    float32 bound is wider than elsewhere: some drawn models are ill-conditioned (the plain statement run in
    float32 differs from itself in float64 by up to 7e-5 of the largest logit on them)."""
    import random

    from starter_b200.engine import ModelRunner, StepEntry, load_model
    from tiny_bavedra import random_config

    rng = random.Random(1000 + seed)
    raw = random_config(rng)
    folder = make_bavedra_folder(tmp_path_factory.mktemp(f"r{seed}"), f"R{seed}", seed=seed, dtype=torch.bfloat16, raw=raw)
    cfg, w = plain.read_model_folder(folder)
    lengths = [rng.choice([1, 3, 40, 130]), rng.choice([2, 70, 150]), rng.choice([5, 64, 65, 200])]
    prompts = [random_prompt(n, cfg["vocab"], seed * 10 + i) for i, n in enumerate(lengths)]
    want = [plain.forward(cfg, w, p) for p in prompts]
    runner = ModelRunner(load_model(folder, "float32"), max_tokens=64 * 40, max_sequences=8, use_graphs=False)
    for p, wanted in zip(prompts, want):
        slot = runner.open_sequence()
        got = runner.step([StepEntry(slot, p, all_places(len(p)))])
        runner.close_sequence(slot)
        close(got, wanted, "float32", f"whole, length {len(p)}", fp32=3e-4)
    tails = [min(len(p) - 1, 20) for p in prompts]
    heads = [len(p) - t for p, t in zip(prompts, tails)]
    slots = [runner.open_sequence() for _ in prompts]
    first = runner.step([StepEntry(s, p[:h], all_places(h)) for s, p, h in zip(slots, prompts, heads)])
    got, at = [[] for _ in prompts], 0
    for i, h in enumerate(heads):
        got[i].append(first[at:at + h])
        at += h
    for step in range(max(tails)):
        live = [i for i in range(3) if step < tails[i]]
        out = runner.step([StepEntry(slots[i], [prompts[i][heads[i] + step]], [0]) for i in live])
        for row, i in enumerate(live):
            got[i].append(out[row:row + 1])
    for i in range(3):
        runner.close_sequence(slots[i])
        close(torch.cat(got[i]), want[i], "float32", f"begun and decoded together, request {i}", fp32=3e-4)
    slot, rows, at = runner.open_sequence(), [], 0
    for n in (2, 1, 3, 61, 70, 200):
        part = prompts[2][at:at + n]
        if part:
            rows.append(runner.step([StepEntry(slot, part, all_places(len(part)))]))
            at += len(part)
    runner.close_sequence(slot)
    close(torch.cat(rows), want[2], "float32", "in portions", fp32=3e-4)
    runner.check_status()
    runner.cache.check()
    assert runner.cache.slots.held_count == 0 and runner.cache.pages.held_count == 0
    routed = Routed(ModelRunner(load_model(folder, "bfloat16"), max_tokens=64 * 40, max_sequences=8, use_graphs=False))
    for p in prompts:
        slot = routed.runner.open_sequence()
        got = routed.step([StepEntry(slot, p, all_places(len(p)))], [len(p)])
        routed.runner.close_sequence(slot)
        held = plain.forward(cfg, w, p, routes=routed.routes(len(p), "bfloat16"))
        # a drawn model may be ill-conditioned: the mean error says whether the mechanisms are right
        mean = float((got.double().cpu() - held).abs().mean()) / float(held.abs().max())
        assert mean <= 2e-2, f"bfloat16, length {len(p)}: mean error {mean:.3e} of the largest logit"


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

    model = random_model(config_from_dict(TINY_B["BC"]), seed=5, dtype="bfloat16")
    engine = Engine.from_model(model, max_batch=2)
    out = engine.complete([[1, 2, 3], [4]], 12, temperature=0.8, seed=3)
    assert [len(c.tokens) for c in out] == [12, 12]
    assert all(0 <= t < 257 for c in out for t in c.tokens)


# ------------------------------------------------------------------------------ the programs

def test_command_line_and_trace_replay(tmp_path_factory, tmp_path):
    """``python -m starter_b200 generate`` and ``bin/trace_run`` pick the design by its config.json."""
    import json
    import os
    import subprocess
    import sys

    import numpy as np

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    folder, cfg, w = case(tmp_path_factory, "BB")
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
