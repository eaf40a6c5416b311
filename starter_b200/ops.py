"""Python face of the CUDA kernels: argument checks, output allocation, launch on the current stream.

Every function here runs a hand-written kernel from ``starter_b200/csrc`` (the one
exception: a bfloat16 matrix product of 129 to 511 rows goes to the vendor's GEMM
library, where the reference uses one too, engine/engine.py:431-450).  There is no
CPU path: tensors must live on a CUDA device, and a shape a kernel cannot take is
refused with an error that names it.
"""

from __future__ import annotations

import ctypes
import functools

import torch

from .cache.layout import PAGE_TOKENS
from .csrc import build

SMALL_ROWS = 16
#: Up to this many rows the bfloat16 product runs on this library's few-row tcgen05 kernel
#: (csrc/gemm_tcgen05.cu), where it is bound by streaming the weights.  Measured on the four
#: projections of a 2560-wide layer: 63-70 us a layer up to 64 rows against 64-86 for the vendor's
#: library; 66 against 68-77 at 96 rows, 70 against 68 at 128, 95-102 against 73 at 192.
TENSOR_CORE_MAX_ROWS = 128
#: From this many rows on it runs on this library's persistent CTA-pair kernel
#: (csrc/gemm_prompt_tcgen05.cu), whose tiles are 256 rows high.  Measured a layer against the
#: vendor's library (which needs a separate SwiGLU kernel): 114 against 106 us at 512 rows, 167
#: against 164 at 1,024, 298 against 307 at 2,048, 434 against 470 at 3,072; at 256 rows 100 against
#: 75.  In between (129 to 511 rows) the vendor's GEMM is used, as the reference does from 33 rows on
#: (engine/engine.py:431-450).
PROMPT_MIN_ROWS = 512
MAX_HEAD_DIM = 256

_DT = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    pass


_checked = set()


def _lib(name: str):
    """The kernel library of ``name.cu``; refuses one compiled for another cache page size."""
    lib = build.load(name)
    if name not in _checked:
        compiled = lib.sb_page_tokens()
        if compiled != PAGE_TOKENS:
            raise KernelError(f"libsb_{name} was compiled for cache pages of {compiled} tokens, the cache "
                              f"uses pages of {PAGE_TOKENS}")
        _checked.add(name)
    return lib


def _code(dtype) -> int:
    if dtype not in _DT:
        raise KernelError(f"kernels take float32 or bfloat16 tensors, not {dtype}")
    return _DT[dtype]


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


try:                                   # the raw handle of the current stream without building objects
    _raw_stream = torch._C._cuda_getCurrentRawStream
    _current_device = torch._C._cuda_getDevice
except AttributeError:                 # pragma: no cover - older or newer torch: the public way
    _raw_stream = _current_device = None


def _stream():
    """The current CUDA stream as a ``void*`` (called once per launch: it has to be cheap)."""
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(_current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _need(t, name, dtype=None, ndim=None):
    # the common case first and in one expression: this runs several times per launch
    try:
        if (t.is_cuda and t.is_contiguous() and (dtype is None or t.dtype == dtype)
                and (ndim is None or t.dim() == ndim)):
            return
    except AttributeError:
        pass
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU implementation)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous, got strides {t.stride()} for shape {tuple(t.shape)}")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    raise KernelError(f"{name} must have {ndim} dimensions, got shape {tuple(t.shape)}")


class _Added:
    """What ``linear`` returns when it has put its result onto ``add_to`` instead of returning it."""

    def __repr__(self):
        return "ADDED"


#: the value that stands for "already added onto the residual stream" (see ``linear``'s ``add_to``)
ADDED = _Added()

#: how many kernels of this library have been launched by this process (library GEMMs not counted)
launch_count = 0
#: switch for the decode attention's reads before its dependent-launch wait (see attention_decode_qkv)
EARLY_READS = True


def _check(rc, what, kernels=1):
    global launch_count
    launch_count += kernels
    if rc != 0:
        if rc == -1:
            raise KernelError(f"{what}: this combination of dtypes has no kernel")
        if rc == -2:
            raise KernelError(f"{what}: a size is outside what the kernel takes")
        raise KernelError(f"{what}: launch failed with CUDA error {rc}")


def _gain_code(x, gain):
    if gain.dtype == torch.float32:
        return 0
    if gain.dtype == torch.bfloat16 and x.dtype == torch.bfloat16:
        return 1
    raise KernelError(f"a {gain.dtype} gain cannot scale {x.dtype} activations")


# ---------------------------------------------------------------------------------------- rows

def embedding(tokens, table, status=None, fence=False):
    """``out[t] = table[tokens[t]]``; ``tokens`` int32 ``[T]``, ``table`` ``[V, H]``.

    ``fence``: launch it as an ordinary kernel (not a dependent launch), so that it starts only when
    everything before it on the stream has completed.  As a step's first kernel it is what lets later
    kernels of the step read, before their own dependent-launch wait, what earlier steps wrote."""
    _need(tokens, "tokens", torch.int32, 1)
    _need(table, "table", None, 2)
    out = torch.empty((tokens.shape[0], table.shape[1]), dtype=table.dtype, device=table.device)
    rc = _lib("elementwise").sb_embedding(
        _code(table.dtype), _ptr(tokens), _ptr(table), _ptr(out), tokens.shape[0], table.shape[1],
        table.shape[0], _ptr(status), int(fence), _stream())
    _check(rc, "embedding")
    return out


def rmsnorm(x, gain, eps, delta=None, rows=None, out=None):
    """RMSNorm of the rows of ``x`` ``[T, H]``.

    With ``delta`` the norm is taken of ``x + delta`` and, unless ``rows`` is given,
    ``x`` is replaced by that sum (the residual stream).  With ``rows`` (int32
    ``[R]``) only those rows are normed and ``x`` is left alone.
    """
    _need(x, "x", None, 2)
    _need(gain, "gain", None, 1)
    hidden = x.shape[1]
    if gain.shape[0] != hidden:
        raise KernelError(f"gain has {gain.shape[0]} entries for rows of {hidden}")
    if delta is not None:
        _need(delta, "delta", x.dtype, 2)
        if delta.shape != x.shape:
            raise KernelError(f"delta {tuple(delta.shape)} does not match x {tuple(x.shape)}")
    n_rows = x.shape[0]
    if rows is not None:
        _need(rows, "rows", torch.int32, 1)
        n_rows = rows.shape[0]
    if out is None:
        out = torch.empty((n_rows, hidden), dtype=x.dtype, device=x.device)
    rc = _lib("elementwise").sb_rmsnorm(
        _code(x.dtype), _gain_code(x, gain), _ptr(x), _ptr(delta), _ptr(gain), _ptr(out), _ptr(rows),
        n_rows, hidden, ctypes.c_float(eps), _stream())
    _check(rc, "rmsnorm")
    return out


#: the activations a gated product knows, and the code the kernels take for each
ACTIVATIONS = {"silu": 1, "gelu_tanh": 2}
#: the code of the clamped gate ``min(g, L) sigmoid(1.702 min(g, L)) (clamp(u, -L, L) + 1)``, which takes its limit beside it
GATE_CLAMPED = 3


def gate_code(gated) -> int:
    """``gated`` as the kernels' code: False 0, True or ``"silu"`` 1, ``"gelu_tanh"`` 2."""
    if gated is False or gated is None or gated == 0:
        return 0
    if gated is True:
        return 1
    if isinstance(gated, int) and gated in ACTIVATIONS.values():
        return gated
    try:
        return ACTIVATIONS[gated]
    except (KeyError, TypeError):
        raise KernelError(f"no gated product with activation {gated!r} (known: {', '.join(ACTIVATIONS)})") from None


def swiglu(gate_up, activation="silu"):
    """``round(act(gate)) * up`` for ``gate_up = [gate | up]`` of shape ``[T, 2 * I]``."""
    _need(gate_up, "gate_up", None, 2)
    if gate_up.shape[1] % 2:
        raise KernelError(f"gate_up has an odd width {gate_up.shape[1]}")
    inner = gate_up.shape[1] // 2
    out = torch.empty((gate_up.shape[0], inner), dtype=gate_up.dtype, device=gate_up.device)
    rc = _lib("elementwise").sb_swiglu(
        _code(gate_up.dtype), _ptr(gate_up), _ptr(out), gate_up.shape[0], inner, gate_code(activation),
        _stream())
    _check(rc, "swiglu")
    return out


# ---------------------------------------------------------------------------------------- matrix products

def linear(x, weight, out_float=False, gated=False, status=None, add_to=None):
    """``x @ weight.T`` for ``x`` ``[T, K]`` and ``weight`` ``[N, K]`` (no bias).

    ``add_to`` (``[T, N]``, the residual stream) is an offer, not an order: where the kernel that
    runs has an epilogue for it (the prompt product), ``add_to`` becomes
    ``round(add_to + round(product))`` in place and ``ADDED`` is returned; otherwise ``add_to`` is
    left alone and the product is returned as usual.

    ``gated`` (True, or an activation of ``ACTIVATIONS`` by name; True means silu): ``weight`` is
    ``[gate; up]`` stacked (``[2 * I, K]``) and the result is
    ``round(act(x @ gate.T)) * (x @ up.T)`` of shape ``[T, I]``.  ``out_float``
    returns float32 whatever the working type (used for logits).  ``status`` (int32 ``[1]``) is the
    device word in which the tensor-core kernel reports a wait that ran out.
    """
    _need(x, "x", None, 2)
    _need(weight, "weight", x.dtype, 2)
    rows, k_dim = x.shape
    if weight.shape[1] != k_dim:
        raise KernelError(f"weight {tuple(weight.shape)} does not take inputs of width {k_dim}")
    n_total = weight.shape[0]
    gated = gate_code(gated)
    if gated and n_total % 2:
        raise KernelError(f"a gated weight needs an even number of rows, got {n_total}")
    n_out = n_total // 2 if gated else n_total
    dt = _code(x.dtype)
    if dt == 1 and rows <= TENSOR_CORE_MAX_ROWS and tensor_core_ok(x, weight, gated, n_out):
        return linear_tensor_core(x, weight, out_float=out_float, gated=gated, status=status)
    if rows <= SMALL_ROWS:
        out_dtype = torch.float32 if (out_float or dt == 0) else x.dtype
        if gated and out_float and dt == 1:
            raise KernelError("a gated product cannot return float32 from bfloat16")
        y = torch.empty((rows, n_out), dtype=out_dtype, device=x.device)
        rc = _lib("linear_small").sb_linear_small(
            dt, int(out_float), int(gated), _ptr(x), _ptr(weight), _ptr(y), rows, n_out, k_dim,
            _stream())
        _check(rc, "linear_small")
        return y
    if dt == 0:
        y = torch.empty((rows, n_total), dtype=torch.float32, device=x.device)
        rc = _lib("sgemm").sb_sgemm_nt(_ptr(x), _ptr(weight), _ptr(y), rows, n_total, k_dim,
                                             _stream())
        _check(rc, "sgemm")
    elif out_float:
        y = torch.mm(x, weight.t(), out_dtype=torch.float32)
    elif rows >= PROMPT_MIN_ROWS and k_dim % 8 == 0 and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0:
        if (add_to is not None and not gated and add_to.dtype == torch.bfloat16 and add_to.is_contiguous()
                and tuple(add_to.shape) == (rows, n_out)):
            linear_prompt(x, weight, status=status, residual=add_to)
            return ADDED
        return linear_prompt(x, weight, gated=gated, status=status)
    else:
        y = torch.mm(x, weight.t())
    return swiglu(y, gated) if gated else y


def tensor_core_ok(x, weight, gated, n_out) -> bool:
    """Whether the tcgen05 product takes these operands: k a multiple of 8 (16-byte rows for TMA),
    16-byte aligned bases, gated widths in steps of 64."""
    k_dim = x.shape[1]
    if k_dim % 8 or x.data_ptr() % 16 or weight.data_ptr() % 16:
        return False
    if gated and n_out % 64:
        return False
    return True


def whole_splits(k_blocks: int, splits: int) -> int:
    """The largest number of parts up to ``splits`` that leaves no part without a k-block: the kernel gives
    every part ``ceil(k_blocks / parts)`` blocks, so with 30 blocks in 7 parts the seventh would get none
    and its accumulator would never be committed."""
    splits = max(1, min(splits, k_blocks))
    while splits > 1 and -(-k_blocks // splits) * (splits - 1) >= k_blocks:
        splits -= 1
    return splits


def gemm_plan(rows: int, n_out: int, k_dim: int, gated: bool):
    """``_gemm_plan`` with the parts of the k range cut down to a number that leaves none empty."""
    bm, splits, stages = _gemm_plan(rows, n_out, k_dim, gated)
    return bm, whole_splits(-(-k_dim // 64), splits), stages


@functools.lru_cache(maxsize=4096)     # asked once per launch, with the same few shapes step after step
def _gemm_plan(rows: int, n_out: int, k_dim: int, gated: bool):
    """``(bm, splits, stages)``: activation rows per tile; how many CTAs (one cluster) share a tile's
    k range; how deep the ring of shared-memory stages is.

    With few rows the product is bound by streaming the weights: about two CTAs per SM should be
    loading, each with some 100 KB in flight.  With more rows two or three CTAs per SM hold 128-row tiles."""
    bm = 16
    while bm < rows and bm < 128:
        bm *= 2
    tiles = (n_out // 64 if gated else -(-n_out // 128)) * -(-rows // bm)
    k_blocks = -(-k_dim // 64)
    stage_bytes = 16384 + bm * 128
    if rows <= 64:
        def fits(splits, stages):       # every CTA resident at once
            return tiles * splits <= 148 * ((227 * 1024) // (stages * stage_bytes + 2048))

        # Measured inside the captured decode step (not kernel by kernel: what a product can have on
        # its way before its predecessor ends depends on the room that predecessor leaves on an SM).
        if tiles * 6 <= 148 and k_blocks >= 32:
            # few tiles (a narrow output): eight CTAs a tile with six stages, two to an SM; where
            # the stages are too large for that, six CTAs a tile with the deepest ring
            return (bm, 8, 6) if fits(8, 6) else (bm, min(6, 148 // tiles), 8)
        if tiles <= 74 and k_blocks >= 32:
            # up to half as many tiles as SMs: six stages, two CTAs to an SM, about 1.3 CTAs per SM
            splits = max(1, min(8, k_blocks // 4, 192 // tiles))
            if fits(splits, 6):
                return bm, splits, 6
        # otherwise: rings deeper than four stages lose (fewer CTAs fit on an SM); the product is
        # fastest with about 80% of the CTA slots taken and all CTAs resident at once; when three
        # stages let a third CTA onto each SM and that buys clearly more CTAs, three stages win
        def choice(stages):
            slots = 148 * ((227 * 1024) // (stages * stage_bytes + 2048))
            return slots, max(1, min(8, k_blocks // 4, int(0.82 * slots) // tiles))

        slots4, splits4 = choice(4)
        slots3, splits3 = choice(3)
        if bm > 16 and slots3 > slots4 and (tiles > slots4 or tiles * splits3 > 1.5 * tiles * splits4):
            stages, splits = 3, splits3
        else:
            stages, splits = 4, splits4
    else:
        # measured at 96 to 500 rows (128-row tiles).  Few tiles: one CTA of six stages per SM and up
        # to four CTAs sharing a tile's k range.  More tiles than SMs: two stages (three CTAs on an
        # SM), and two CTAs a tile while there is one row tile.  In between: three stages.
        slots3 = 148 * ((227 * 1024) // (3 * stage_bytes + 2048))
        if tiles <= 74:
            # (clusters of three were measured far slower than of two or four here)
            splits = max(1, min(4, k_blocks // 8, 148 // tiles))
            stages, splits = 6, (2 if splits == 3 else splits)
        elif tiles > 148:
            stages, splits = 2, (2 if rows <= 128 and k_blocks >= 16 else 1)
        else:
            stages, splits = 3, max(1, min(4, k_blocks // 8, slots3 // tiles))
    return bm, splits, stages


def linear_tensor_core(x, weight, out_float=False, gated=False, bm=None, splits=None, stages=None,
                       status=None, withhold=None):
    """The bfloat16 product on tcgen05 tensor cores (csrc/gemm_tcgen05.cu).

    ``withhold = (k_block, limit_ns)`` is for tests of the kernel's give-up path: the activation copy
    of that k-block is left out, so a wait inside the kernel runs out after ``limit_ns``; the kernel
    returns, bit 4 of ``status`` is set and the result is undefined."""
    _need(x, "x", torch.bfloat16, 2)
    _need(weight, "weight", torch.bfloat16, 2)
    gated = gate_code(gated)
    rows, k_dim = x.shape
    n_total = weight.shape[0]
    n_out = n_total // 2 if gated else n_total
    if weight.shape[1] != k_dim:
        raise KernelError(f"weight {tuple(weight.shape)} does not take inputs of width {k_dim}")
    if not tensor_core_ok(x, weight, gated, n_out):
        raise KernelError(f"the tensor-core product needs k % 8 == 0, 16-byte aligned operands and gated "
                          f"widths in steps of 64; got k = {k_dim}, n = {n_out}")
    plan = gemm_plan(rows, n_out, k_dim, gated)
    bm = bm or plan[0]
    splits = whole_splits(-(-k_dim // 64), splits or plan[1])
    stages = stages or max(plan[2], -(-bm * 512 // (16384 + bm * 128)))
    stages = min(stages, (226 * 1024) // (16384 + bm * 128))     # a tile height other than the plan's
    out = torch.empty((rows, n_out), dtype=torch.float32 if out_float else torch.bfloat16, device=x.device)
    if withhold is not None:
        rc = _lib("gemm_tcgen05").sb_gemm_tcgen05_withheld(
            _ptr(x), _ptr(weight), _ptr(out), rows, n_out, k_dim, bm, splits, stages, int(gated),
            int(out_float), _ptr(status), ctypes.c_ulonglong(int(withhold[1])), int(withhold[0]), _stream())
    else:
        rc = _lib("gemm_tcgen05").sb_gemm_tcgen05(
            _ptr(x), _ptr(weight), _ptr(out), rows, n_out, k_dim, bm, splits, stages, int(gated),
            int(out_float), _ptr(status), _stream())
    if rc in (-3, -4):
        raise KernelError("the TMA descriptors for the tensor-core product could not be made "
                          f"(code {rc}); is the driver too old for cuTensorMapEncodeTiled?")
    _check(rc, "gemm_tcgen05")
    return out


def linear_prompt(x, weight, gated=False, bn=0, pairs=0, status=None, withhold=None, residual=None):
    """The bfloat16 product for many rows: the persistent CTA-pair kernel (csrc/gemm_prompt_tcgen05.cu).

    ``bn`` is the number of weight rows per tile (0: chosen by the kernel's host side), ``pairs`` the
    number of CTA pairs (0: one per two SMs).  ``withhold = (k_block, limit_ns)`` is for tests of the
    give-up path: one weight copy is left out, a wait runs out after ``limit_ns``, the kernel returns,
    bit 4 of ``status`` is set and the result is undefined.  With ``residual`` (``[rows, n]``
    bfloat16, not with ``gated``) the result is ``round(residual + round(product))``, written into
    ``residual`` itself, which is returned."""
    _need(x, "x", torch.bfloat16, 2)
    _need(weight, "weight", torch.bfloat16, 2)
    gated = gate_code(gated)
    rows, k_dim = x.shape
    n_total = weight.shape[0]
    n_out = n_total // 2 if gated else n_total
    if weight.shape[1] != k_dim:
        raise KernelError(f"weight {tuple(weight.shape)} does not take inputs of width {k_dim}")
    if k_dim % 8 or (gated and n_total % 2) or x.data_ptr() % 16 or weight.data_ptr() % 16:
        raise KernelError(f"the prompt product needs k % 8 == 0 and 16-byte aligned operands; got k = {k_dim}")
    if residual is not None:
        _need(residual, "residual", torch.bfloat16, 2)
        if gated or tuple(residual.shape) != (rows, n_out) or withhold is not None:
            raise KernelError(f"a residual of shape {tuple(residual.shape)} cannot take a "
                              f"{'gated ' if gated else ''}product of shape {(rows, n_out)}")
        out = residual
    else:
        out = torch.empty((rows, n_out), dtype=torch.bfloat16, device=x.device)
    lib = _lib("gemm_prompt_tcgen05")
    if withhold is not None:
        rc = lib.sb_gemm_prompt_withheld(_ptr(x), _ptr(weight), _ptr(out), rows, n_out, k_dim, int(bn), int(pairs),
                                         int(gated), _ptr(status), ctypes.c_ulonglong(int(withhold[1])),
                                         int(withhold[0]), _stream())
    else:
        rc = lib.sb_gemm_prompt(_ptr(x), _ptr(weight), _ptr(out), _ptr(residual), rows, n_out, k_dim, int(bn), int(pairs),
                                int(gated), _ptr(status), _stream())
    if rc in (-3, -4):
        raise KernelError("the TMA descriptors for the prompt product could not be made "
                          f"(code {rc}); is the driver too old for cuTensorMapEncodeTiled?")
    _check(rc, "gemm_prompt_tcgen05")
    return out


# ---------------------------------------------------------------------------------------- attention

def rotation_tables(rotation, head_dim: int):
    """``(cos, sin)`` for the kernels from a position part's ``Rotation`` (or ``(None, None)``).

    The kernels here (``qk_norm_rope_store`` and the decode attention that rotates the new token
    itself) turn the whole head in half-split layout; anything else is refused by name."""
    if rotation is None:
        return None, None
    if rotation.layout != "half_split" or rotation.rotary_dim != head_dim:
        raise KernelError(f"the kernels rotate the whole head ({head_dim} dimensions) in half-split layout; "
                          f"asked for {rotation.rotary_dim} dimensions in {rotation.layout!r} layout")
    return rotation.cos, rotation.sin


def qk_norm_rope_store(qkv, heads, kv_heads, head_dim, q_gain, k_gain, eps, cos_table, sin_table,
                       tok_pos, tok_slot, block_table, k_store, v_store, write_cache=True):
    """Norm and rotate the query and key heads of ``qkv`` and file keys and values in the cache.

    ``qkv`` is ``[T, (heads + 2 * kv_heads) * head_dim]`` (queries alone,
    ``[T, heads * head_dim]``, when ``write_cache`` is false); returns the queries
    ``[T, heads * head_dim]``.  ``k_store``/``v_store`` are one cache entry's pages
    ``[pages, kv_heads, 64, head_dim]``; ``block_table`` int32 ``[slots, max_pages]``.
    """
    _need(qkv, "qkv", None, 2)
    n_tokens = qkv.shape[0]
    width = (heads + 2 * kv_heads) * head_dim if write_cache else heads * head_dim
    if qkv.shape[1] != width:
        raise KernelError(f"qkv has width {qkv.shape[1]}, expected {width}")
    if head_dim % 2 or head_dim > MAX_HEAD_DIM:
        raise KernelError(f"head_dim {head_dim} must be even and at most {MAX_HEAD_DIM}")
    _need(tok_pos, "tok_pos", torch.int32, 1)
    _need(tok_slot, "tok_slot", torch.int32, 1)
    _need(block_table, "block_table", torch.int32, 2)
    gain_code = 0
    for g in (q_gain, k_gain):
        if g is not None:
            _need(g, "head gain", None, 1)
            if g.shape[0] != head_dim:
                raise KernelError(f"head gain has {g.shape[0]} entries for head_dim {head_dim}")
            gain_code = _gain_code(qkv, g)
    if (q_gain is None) != (k_gain is None):
        raise KernelError("q and k head norms come together")
    if cos_table is not None:
        _need(cos_table, "cos_table", torch.float32, 2)
        _need(sin_table, "sin_table", torch.float32, 2)
        if cos_table.shape[1] != head_dim // 2 or sin_table.shape != cos_table.shape:
            raise KernelError("rotary tables must be [positions, head_dim / 2]")
    if write_cache:
        for store in (k_store, v_store):
            _need(store, "cache pages", qkv.dtype, 4)
            if tuple(store.shape[1:]) != (kv_heads, PAGE_TOKENS, head_dim):
                raise KernelError(f"cache pages have shape {tuple(store.shape)}, expected "
                                  f"[pages, {kv_heads}, {PAGE_TOKENS}, {head_dim}]")
    q_out = torch.empty((n_tokens, heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    rc = _lib("rope_cache").sb_qk_norm_rope_store(
        _code(qkv.dtype), gain_code, _ptr(qkv), _ptr(q_out), _ptr(q_gain), _ptr(k_gain),
        _ptr(cos_table), _ptr(sin_table), _ptr(tok_pos), _ptr(tok_slot), _ptr(block_table),
        block_table.shape[1], _ptr(k_store if write_cache else None),
        _ptr(v_store if write_cache else None), n_tokens, heads, kv_heads, head_dim,
        ctypes.c_float(eps), int(write_cache), qkv.shape[1], _stream())
    _check(rc, "qk_norm_rope_store")
    return q_out


def attention_rowwise(q, k_store, v_store, block_table, tok_slot, tok_pos, heads, kv_heads, head_dim,
                      scale, window=None):
    """Causal attention of each query row over its sequence's cached keys (plain kernel)."""
    _need(q, "q", None, 2)
    if q.shape[1] != heads * head_dim:
        raise KernelError(f"q has width {q.shape[1]}, expected {heads * head_dim}")
    if head_dim > MAX_HEAD_DIM:
        raise KernelError(f"head_dim {head_dim} exceeds {MAX_HEAD_DIM}")
    if heads % kv_heads:
        raise KernelError(f"{heads} query heads cannot share {kv_heads} key/value heads")
    for store in (k_store, v_store):
        _need(store, "cache pages", q.dtype, 4)
        if tuple(store.shape[1:]) != (kv_heads, PAGE_TOKENS, head_dim):
            raise KernelError(f"cache pages have shape {tuple(store.shape)}")
    _need(block_table, "block_table", torch.int32, 2)
    _need(tok_slot, "tok_slot", torch.int32, 1)
    _need(tok_pos, "tok_pos", torch.int32, 1)
    out = torch.empty_like(q)
    rc = _lib("attention_rowwise").sb_attention_rowwise(
        _code(q.dtype), _ptr(q), _ptr(out), _ptr(k_store), _ptr(v_store), _ptr(block_table),
        block_table.shape[1], _ptr(tok_slot), _ptr(tok_pos), q.shape[0], heads, kv_heads, head_dim,
        ctypes.c_float(scale), int(window or 0), _stream())
    _check(rc, "attention_rowwise")
    return out


PREFILL_HEAD_DIMS = (16, 32, 64, 128)


def attention_prefill(q, k_store, v_store, block_table, seq_slot, seq_q_start, seq_q_len, seq_kv_len,
                      tile_seq, tile_first, heads, kv_heads, head_dim, scale, window=None, status=None,
                      kernel=None, max_q_len=None, blocks=None, withhold=None):
    """Causal attention for steps with many tokens per sequence (bfloat16, tensor cores).

    ``q`` ``[T, heads * head_dim]`` packed by sequence; the ``seq_*`` arrays describe each sequence
    of the step, ``tile_seq``/``tile_first`` list the tiles of 64 queries.  Head sizes 64 and 128 run
    on the tcgen05 kernel (256 queries a block, S and O in tensor memory) when some sequence brings
    more than 128 queries (``max_q_len``, taken as large when not given); everything else runs on
    the mma.sync kernel, which has the smaller blocks.  ``kernel`` ("tcgen05" or "mma") forces one.
    ``blocks = (block_seq, block_first)`` is the same work list in blocks of 256 queries, which is what
    the tcgen05 kernel launches; without it that kernel is launched once per tile of 64 and three of
    four launches find nothing to do.  ``withhold = (step, limit_ns)`` is for tests of the tcgen05
    kernel's give-up path: half of the values of that step of 128 keys are not copied, the wait on them
    runs out after ``limit_ns``, bit 16 of ``status`` is set and the result is undefined."""
    _need(q, "q", torch.bfloat16, 2)
    if q.shape[1] != heads * head_dim:
        raise KernelError(f"q has width {q.shape[1]}, expected {heads * head_dim}")
    if head_dim not in PREFILL_HEAD_DIMS:
        raise KernelError(f"head_dim {head_dim} is not one of {PREFILL_HEAD_DIMS}")
    if heads % kv_heads:
        raise KernelError(f"{heads} query heads cannot share {kv_heads} key/value heads")
    for store in (k_store, v_store):
        _need(store, "cache pages", q.dtype, 4)
        if tuple(store.shape[1:]) != (kv_heads, PAGE_TOKENS, head_dim):
            raise KernelError(f"cache pages have shape {tuple(store.shape)}")
    _need(block_table, "block_table", torch.int32, 2)
    for name, t in (("seq_slot", seq_slot), ("seq_q_start", seq_q_start), ("seq_q_len", seq_q_len),
                    ("seq_kv_len", seq_kv_len), ("tile_seq", tile_seq), ("tile_first", tile_first)):
        _need(t, name, torch.int32, 1)
    out = torch.empty_like(q)
    if kernel is None:
        long_enough = max_q_len is None or max_q_len > 128
        kernel = "tcgen05" if head_dim in PREFILL_TC_HEAD_DIMS and long_enough else "mma"
    if kernel == "tcgen05":
        if head_dim not in PREFILL_TC_HEAD_DIMS:
            raise KernelError(f"the tcgen05 prefill kernel takes head_dim {PREFILL_TC_HEAD_DIMS}, not {head_dim}")
        if not q.is_contiguous():
            raise KernelError("q must be contiguous")
        own_list = blocks is not None and blocks[0] is not None
        if own_list:
            for name, t in (("block_seq", blocks[0]), ("block_first", blocks[1])):
                _need(t, name, torch.int32, 1)
        list_seq, list_first = blocks if own_list else (tile_seq, tile_first)
        if withhold is not None:
            _lib("attention_prefill_tc").sb_attention_prefill_tc_withhold(
                int(withhold[0]), ctypes.c_ulonglong(int(withhold[1])))
        rc = _lib("attention_prefill_tc").sb_attention_prefill_tc(
            _ptr(q), _ptr(out), _ptr(k_store), _ptr(v_store), _ptr(block_table), block_table.shape[1],
            _ptr(seq_slot), _ptr(seq_q_start), _ptr(seq_q_len), _ptr(seq_kv_len), _ptr(list_seq),
            _ptr(list_first), list_seq.shape[0], q.shape[0], k_store.shape[0], heads, kv_heads, head_dim,
            ctypes.c_float(scale), int(window or 0), _ptr(status) if status is not None else None,
            int(own_list), _stream())
        _check(rc, "attention_prefill_tc")
        return out
    rc = _lib("attention_prefill").sb_attention_prefill(
        _ptr(q), _ptr(out), _ptr(k_store), _ptr(v_store), _ptr(block_table), block_table.shape[1],
        _ptr(seq_slot), _ptr(seq_q_start), _ptr(seq_q_len), _ptr(seq_kv_len), _ptr(tile_seq),
        _ptr(tile_first), tile_seq.shape[0], heads, kv_heads, head_dim, ctypes.c_float(scale),
        int(window or 0), _stream())
    _check(rc, "attention_prefill")
    return out


PREFILL_TC_HEAD_DIMS = (64, 128)
DECODE_CLUSTER_SPLITS = 8
DECODE_HEAD_DIMS = (16, 32, 64, 128, 256)


def decode_attention_takes(head_dim: int, dtype) -> bool:
    """Whether the split-key decode kernel takes this head size: 16 elements per lane, and two
    stages of a page's keys and values (2 * 2 * 64 * head_dim elements) within shared memory."""
    return head_dim in DECODE_HEAD_DIMS and head_dim * dtype.itemsize <= 512


@functools.lru_cache(maxsize=4096)
def decode_splits(rows: int, kv_heads: int, groups: int, group_rows: int = 4, kv_hint: int = 0) -> int:
    """How many parts to cut each row's keys into, so that every block is resident at once and the
    SMs are busy.

    The tensor-core kernel (``group_rows`` 16) merges up to ``DECODE_CLUSTER_SPLITS`` parts inside a
    thread-block cluster at no extra launch, and every part may be as short as a page.  Measured
    inside the captured decode step at 3,073 keys: the step is fastest with at most 256 blocks (two
    fit on an SM, 296 in all, but 280 or 288 blocks cost 12-17% of the whole step at 5, 6 and 12
    rows), with 224 rather than 256 when that means 7 parts instead of 8, and with no more than 8
    parts at 3,073 keys: 17 parts through scratch memory and the merge kernel lose 1-2% of the step
    to 8 in a cluster at 1 and 2 rows.  The CUDA-core kernel always merges with a second kernel and
    wants three pages per part."""
    blocks = rows * kv_heads * (-(-groups // group_rows))
    pages = -(-kv_hint // PAGE_TOKENS) if kv_hint > 0 else None
    if group_rows < 16:
        want = max(1, min(32, (2 * 148) // blocks))
        return want if pages is None else max(1, min(want, -(-pages // 3)))
    want = max(1, min(DECODE_CLUSTER_SPLITS, 256 // blocks))
    if want > 4 and want * blocks > 240:
        want -= 1
    if pages is None:
        return want
    want = max(1, min(want, pages))
    # Few rows of many keys: 8 parts a row leave most SMs without a block, and a block streams about
    # 60 GB/s.  More parts through scratch memory cost a merge kernel (3 us) and fill the SMs.
    # Estimated both ways in microseconds from the bytes (a page of keys and values of a 128-wide
    # head is 32 KB) and taken when the estimate says so; the crossover it gives for one row of 8
    # key/value heads, 6,700 keys, lies between the measured 3,073 (cluster faster by 0.7 us a
    # layer) and 16,384 (scratch faster by 6.2 us).
    more = max(1, min(32, 256 // blocks, pages // 3))
    if more >= 12 and more > want:
        megabytes = blocks * pages * 0.032768
        in_cluster = megabytes / min(6.5, want * blocks * 0.06)
        through_scratch = 3.0 + megabytes / min(6.5, more * blocks * 0.06)
        if through_scratch < in_cluster:
            return more
    return want


def decode_from_qkv_takes(head_dim: int, dtype) -> bool:
    """Whether ``attention_decode_qkv`` takes this head size and type (the tensor-core decode kernel)."""
    return dtype == torch.bfloat16 and head_dim in PREFILL_HEAD_DIMS


def attention_decode_qkv(qkv, k_store, v_store, block_table, row_slot, row_kv_len, heads, kv_heads, head_dim,
                         scale, window, q_gain, k_gain, eps, cos_table, sin_table, write_cache=True,
                         n_splits=None, kv_hint=0, early=False):
    """One-token attention straight from the q/k/v product (bfloat16, tensor cores): head norm,
    rotation and the cache write of ``qk_norm_rope_store`` happen inside the attention kernel, with
    the same arithmetic.  Row ``i`` of ``qkv`` is the new token of the sequence in ``row_slot[i]``, at
    position ``row_kv_len[i] - 1``.  ``qkv`` holds the queries alone when ``write_cache`` is false.

    ``early``: the caller vouches that ``row_kv_len``, the page table and every cached key and value
    but the new token's were complete before this step's first kernel started (``embedding(...,
    fence=True)``) and that nothing else in this step writes them; the kernel then reads the lengths
    and the page numbers before its dependent-launch wait, while the q/k/v product still runs."""
    _need(qkv, "qkv", torch.bfloat16, 2)
    if not decode_from_qkv_takes(head_dim, qkv.dtype):
        raise KernelError(f"head_dim {head_dim} is not one of {PREFILL_HEAD_DIMS}")
    if heads % kv_heads:
        raise KernelError(f"{heads} query heads cannot share {kv_heads} key/value heads")
    rows = qkv.shape[0]
    width = (heads + 2 * kv_heads) * head_dim if write_cache else heads * head_dim
    if qkv.shape[1] != width:
        raise KernelError(f"qkv has width {qkv.shape[1]}, expected {width}")
    for store in (k_store, v_store):
        _need(store, "cache pages", qkv.dtype, 4)
        if tuple(store.shape[1:]) != (kv_heads, PAGE_TOKENS, head_dim):
            raise KernelError(f"cache pages have shape {tuple(store.shape)}")
    _need(block_table, "block_table", torch.int32, 2)
    _need(row_slot, "row_slot", torch.int32, 1)
    _need(row_kv_len, "row_kv_len", torch.int32, 1)
    gain_code = 0
    if (q_gain is None) != (k_gain is None):
        raise KernelError("q and k head norms come together")
    for g in (q_gain, k_gain):
        if g is not None:
            _need(g, "head gain", None, 1)
            if g.shape[0] != head_dim:
                raise KernelError(f"head gain has {g.shape[0]} entries for head_dim {head_dim}")
            gain_code = _gain_code(qkv, g)
    if cos_table is not None:
        _need(cos_table, "cos_table", torch.float32, 2)
        _need(sin_table, "sin_table", torch.float32, 2)
        if cos_table.shape[1] != head_dim // 2 or sin_table.shape != cos_table.shape:
            raise KernelError("rotary tables must be [positions, head_dim / 2]")
    if n_splits is None:
        n_splits = decode_splits(rows, kv_heads, heads // kv_heads, 16, kv_hint)
    out = torch.empty((rows, heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    part_acc = part_ml = None
    in_cluster = 1 < n_splits <= DECODE_CLUSTER_SPLITS
    if n_splits > 1 and not in_cluster:
        part_acc = torch.empty((rows * heads * n_splits * head_dim,), dtype=torch.float32, device=qkv.device)
        part_ml = torch.empty((rows * heads * n_splits * 2,), dtype=torch.float32, device=qkv.device)
    rc = _lib("attention_decode_mma").sb_attention_decode_mma_fused(
        _ptr(qkv), qkv.shape[1], _ptr(out), _ptr(k_store), _ptr(v_store), _ptr(block_table),
        block_table.shape[1], _ptr(row_slot), _ptr(row_kv_len), rows, heads, kv_heads, head_dim,
        ctypes.c_float(scale), int(window or 0), n_splits, _ptr(part_acc), _ptr(part_ml), _ptr(q_gain),
        _ptr(k_gain), gain_code, ctypes.c_float(eps), _ptr(cos_table), _ptr(sin_table), int(write_cache),
        int(bool(early) and write_cache and EARLY_READS), _stream())
    _check(rc, "attention_decode_fused", 2 if n_splits > 1 and not in_cluster else 1)
    return out


def attention_decode(q, k_store, v_store, block_table, row_slot, row_kv_len, heads, kv_heads, head_dim,
                     scale, window=None, n_splits=None, status=None, kv_hint=0, withhold=None):
    """One query per row (the newest token of its sequence) over that sequence's cached keys.

    ``row_kv_len[r]`` is the sequence's length with the query's own key already filed; the lengths
    stay on the device.  ``head_dim`` must be one of ``DECODE_HEAD_DIMS``.

    ``withhold = (page, limit_ns)`` is for tests of the CUDA-core kernel's give-up path: the values of
    that page of every block's range are not copied, the wait on them runs out after ``limit_ns``,
    the kernel returns with bit 8 of ``status`` set and the result is undefined."""
    _need(q, "q", None, 2)
    rows = q.shape[0]
    if q.shape[1] != heads * head_dim:
        raise KernelError(f"q has width {q.shape[1]}, expected {heads * head_dim}")
    if not decode_attention_takes(head_dim, q.dtype):
        raise KernelError(f"head_dim {head_dim} in {q.dtype} is outside what the decode kernel takes: "
                          f"one of {DECODE_HEAD_DIMS} and at most 512 bytes per head row")
    if heads % kv_heads:
        raise KernelError(f"{heads} query heads cannot share {kv_heads} key/value heads")
    for store in (k_store, v_store):
        _need(store, "cache pages", q.dtype, 4)
        if tuple(store.shape[1:]) != (kv_heads, PAGE_TOKENS, head_dim):
            raise KernelError(f"cache pages have shape {tuple(store.shape)}")
    _need(block_table, "block_table", torch.int32, 2)
    _need(row_slot, "row_slot", torch.int32, 1)
    _need(row_kv_len, "row_kv_len", torch.int32, 1)
    tensor_cores = q.dtype == torch.bfloat16 and head_dim in PREFILL_HEAD_DIMS
    if n_splits is None:
        n_splits = decode_splits(rows, kv_heads, heads // kv_heads, 16 if tensor_cores else 4, kv_hint)
    out = torch.empty_like(q)
    part_acc = part_ml = None
    # up to DECODE_CLUSTER_SPLITS splits of the tensor-core kernel are one thread-block cluster and
    # merge through distributed shared memory; more go through scratch and a merge kernel
    in_cluster = tensor_cores and 1 < n_splits <= DECODE_CLUSTER_SPLITS
    if n_splits > 1 and not in_cluster:
        part_acc = torch.empty((rows * heads * n_splits * head_dim,), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((rows * heads * n_splits * 2,), dtype=torch.float32, device=q.device)
    if tensor_cores:
        rc = _lib("attention_decode_mma").sb_attention_decode_mma(
            _ptr(q), _ptr(out), _ptr(k_store), _ptr(v_store), _ptr(block_table), block_table.shape[1],
            _ptr(row_slot), _ptr(row_kv_len), rows, heads, kv_heads, head_dim, ctypes.c_float(scale),
            int(window or 0), n_splits, _ptr(part_acc), _ptr(part_ml), _stream())
    else:
        if withhold is not None:
            _lib("attention_decode").sb_attention_decode_withhold(int(withhold[0]), ctypes.c_ulonglong(int(withhold[1])))
        rc = _lib("attention_decode").sb_attention_decode(
            _code(q.dtype), _ptr(q), _ptr(out), _ptr(k_store), _ptr(v_store), _ptr(block_table),
            block_table.shape[1], _ptr(row_slot), _ptr(row_kv_len), rows, heads, kv_heads, head_dim,
            ctypes.c_float(scale), int(window or 0), n_splits, _ptr(part_acc), _ptr(part_ml),
            _ptr(status), _stream())
    _check(rc, "attention_decode", 2 if n_splits > 1 and not in_cluster else 1)
    return out


# ---------------------------------------------------------------------------------------- several streams

def _f32(t, name, shape=None):
    _need(t, name, torch.float32)
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise KernelError(f"{name} has shape {tuple(t.shape)}, expected {tuple(shape)}")


def max_streams() -> int:
    return _lib("streams").sb_max_streams()


def embedding_streams(tokens, table, streams: int, status=None, fence=False):
    """``out[t, s] = float(table[tokens[t]])`` for every stream ``s``: float32 ``[T, streams, H]``, the
    residual streams of a model with hyper-connections at their start.  ``fence`` as in ``embedding``."""
    _need(tokens, "tokens", torch.int32, 1)
    _need(table, "table", None, 2)
    out = torch.empty((tokens.shape[0], streams, table.shape[1]), dtype=torch.float32, device=table.device)
    rc = _lib("streams").sb_embed_streams(
        _code(table.dtype), _ptr(tokens), _ptr(table), _ptr(out), tokens.shape[0], table.shape[1],
        table.shape[0], int(streams), _ptr(status), int(fence), _stream())
    _check(rc, "embedding_streams")
    return out


def hyper_step(streams, dtype, pending=None, read=None, norm=None, rows=None):
    """One kernel around a sublayer of a model with several residual streams (float32 ``[T, S, H]``).

    ``pending = (y, mix, out, bias)``: the output ``y`` ``[T, H]`` of the sublayer before (``bias``
    float32 ``[H]`` or None is added to it), which updates the streams, each from the
    values before the update, to ``x_t = sum_s mix[s, t] * x_s + out[t] * y``.  ``read``: float32 ``[S]``, the weights of
    the sum ``u = sum_s read[s] * x_s`` that is returned (None: the plain sum of the streams).
    ``norm = (alpha, weight, bias)`` makes it ``tanh(alpha * u) * weight + bias`` (Dynamic Tanh); None
    returns ``u``.  The result is ``[T, H]`` in ``dtype``.  With ``rows`` (int32 ``[R]``) only those rows
    are computed, the result is ``[R, H]`` and the streams are left as they were; without, the update
    is written into ``streams``."""
    _need(streams, "streams", torch.float32, 3)
    n_tokens, n_streams, hidden = streams.shape
    y = mix = out = bias = None
    if pending is not None:
        y, mix, out, bias = pending
        _need(y, "y", dtype, 2)
        if tuple(y.shape) != (n_tokens, hidden):
            raise KernelError(f"y {tuple(y.shape)} does not match streams {tuple(streams.shape)}")
        _f32(mix, "mix", (n_streams, n_streams))
        _f32(out, "out", (n_streams,))
        if bias is not None:
            _f32(bias, "bias", (hidden,))
    if read is not None:
        _f32(read, "read", (n_streams,))
    alpha = weight = shift = None
    if norm is not None:
        alpha, weight, shift = norm
        _f32(alpha, "alpha")
        _f32(weight, "norm weight", (hidden,))
        _f32(shift, "norm bias", (hidden,))
    n_rows = n_tokens
    if rows is not None:
        _need(rows, "rows", torch.int32, 1)
        n_rows = rows.shape[0]
    normed = torch.empty((n_rows, hidden), dtype=dtype, device=streams.device)
    rc = _lib("streams").sb_hyper_step(
        _code(dtype), n_streams, _ptr(streams), _ptr(y), _ptr(bias), _ptr(mix), _ptr(out), _ptr(read),
        int(norm is not None), _ptr(alpha), _ptr(weight), _ptr(shift), _ptr(normed), _ptr(rows), n_rows,
        hidden, _stream())
    if rc == -2:
        raise KernelError(f"the stream kernels take 1 to {max_streams()} streams, not {n_streams}")
    _check(rc, "hyper_step")
    return normed


def dynamic_tanh(x, alpha, weight, bias, delta=None, rows=None):
    """``tanh(alpha * x) * weight + bias`` on the rows of ``x`` ``[T, H]``; ``delta`` and ``rows`` as in
    ``rmsnorm`` (the residual sum in front of the norm, the norm of selected rows)."""
    _need(x, "x", None, 2)
    hidden = x.shape[1]
    _f32(alpha, "alpha")
    _f32(weight, "weight", (hidden,))
    _f32(bias, "bias", (hidden,))
    if delta is not None:
        _need(delta, "delta", x.dtype, 2)
        if delta.shape != x.shape:
            raise KernelError(f"delta {tuple(delta.shape)} does not match x {tuple(x.shape)}")
    n_rows = x.shape[0]
    if rows is not None:
        _need(rows, "rows", torch.int32, 1)
        n_rows = rows.shape[0]
    out = torch.empty((n_rows, hidden), dtype=x.dtype, device=x.device)
    rc = _lib("streams").sb_dyt(_code(x.dtype), _ptr(x), _ptr(delta), _ptr(alpha), _ptr(weight), _ptr(bias),
                                _ptr(out), _ptr(rows), n_rows, hidden, _stream())
    _check(rc, "dynamic_tanh")
    return out


# ---------------------------------------------------------------------------------------- differential attention

DIFF_MAX_ROW = 256
#: from this many tokens of one sequence in a step the tensor-core kernel is used
DIFF_PREFILL_MIN_Q = 16
#: up to this many parts of a row's keys are one thread-block cluster in the single-token kernel
DIFF_CLUSTER_PARTS = 8


def diff_prefill_takes(dtype, dim: int, v_dim: int) -> bool:
    """Whether the tensor-core prompt kernel takes these sizes (csrc/attention_diff_prefill.cu)."""
    return dtype == torch.bfloat16 and bool(_lib("attention_diff_prefill").sb_diff_prefill_takes(int(dim), int(v_dim)))


def diff_prefill_tc_takes(dtype, dim: int, v_dim: int) -> bool:
    """Whether the tcgen05 prompt kernel takes these sizes (csrc/attention_diff_prefill_tc.cu)."""
    return dtype == torch.bfloat16 and bool(_lib("attention_diff_prefill_tc").sb_diff_prefill_tc_takes(int(dim), int(v_dim)))


def diff_attention_prefill(q, gate, k_store, v_store, block_table, seq_slot, seq_q_start, seq_q_len, seq_kv_len,
                           tile_seq, tile_first, heads, kv_heads, dim, v_dim, scale, lam, out_scale, eps,
                           window=None, status=None, kernel=None, max_q_len=None):
    """``diff_attention`` for steps with many tokens per sequence, on tensor cores (bfloat16), both maps
    in one pass over the pages.  ``q`` is packed by sequence; the ``seq_*`` arrays and the list of
    64-query tiles are the step context's.  With ``dim`` 64 and ``v_dim`` 64 or 128 and a sequence that
    brings at least 128 tokens (``max_q_len``, taken as large when not given) the tcgen05 kernel runs
    (128 queries of a head a block, scores and outputs of both maps in tensor memory); otherwise the
    mma.sync kernel (64 queries a block; sizes: ``diff_prefill_takes``).  ``kernel`` ("tcgen05" or
    "mma") forces one.  ``status``: the device word in which the tcgen05 kernel reports a wait that
    ran out (bit 16)."""
    gate_stride = _diff_check(q, gate, k_store, v_store, heads, kv_heads, dim, v_dim)
    _need(block_table, "block_table", torch.int32, 2)
    for name, t in (("seq_slot", seq_slot), ("seq_q_start", seq_q_start), ("seq_q_len", seq_q_len),
                    ("seq_kv_len", seq_kv_len), ("tile_seq", tile_seq), ("tile_first", tile_first)):
        _need(t, name, torch.int32, 1)
    tc_ok = (diff_prefill_tc_takes(q.dtype, dim, v_dim) and q.data_ptr() % 16 == 0
             and (gate is None or (gate_stride % 8 == 0 and gate.data_ptr() % 16 == 0)))
    if kernel is None:
        kernel = "tcgen05" if tc_ok and (max_q_len is None or max_q_len >= 128) else "mma"
    out = torch.empty((q.shape[0], heads * v_dim), dtype=q.dtype, device=q.device)
    if kernel == "tcgen05":
        if not tc_ok:
            raise KernelError(f"the tcgen05 differential attention takes dim 64 and v_dim 64 or 128 in bfloat16 with "
                              f"16-byte aligned rows; got dim {dim}, v_dim {v_dim}, {q.dtype}")
        rc = _lib("attention_diff_prefill_tc").sb_diff_prefill_tc(
            _ptr(q), _ptr(gate), int(gate_stride), _ptr(out), _ptr(k_store), _ptr(v_store), _ptr(block_table),
            block_table.shape[1], _ptr(seq_slot), _ptr(seq_q_start), _ptr(seq_q_len), _ptr(seq_kv_len),
            _ptr(tile_seq), _ptr(tile_first), tile_seq.shape[0], q.shape[0], k_store.shape[0], heads, kv_heads, dim,
            v_dim, ctypes.c_float(scale), int(window or 0), ctypes.c_float(lam), ctypes.c_float(out_scale),
            ctypes.c_float(eps), _ptr(status), _stream())
        if rc in (-3, -4):
            raise KernelError(f"the TMA descriptors for the differential attention could not be made (code {rc})")
        _check(rc, "diff_attention_prefill_tc")
        return out
    if not diff_prefill_takes(q.dtype, dim, v_dim):
        raise KernelError(f"the tensor-core differential attention is not built for dim {dim}, v_dim {v_dim} in {q.dtype}")
    if gate is not None and (gate_stride % 2 or gate.data_ptr() % 4):
        raise KernelError("the gate's rows must start on 4-byte boundaries")
    rc = _lib("attention_diff_prefill").sb_diff_prefill(
        _ptr(q), _ptr(gate), int(gate_stride), _ptr(out), _ptr(k_store), _ptr(v_store), _ptr(block_table),
        block_table.shape[1], _ptr(seq_slot), _ptr(seq_q_start), _ptr(seq_q_len), _ptr(seq_kv_len),
        _ptr(tile_seq), _ptr(tile_first), tile_seq.shape[0], heads, kv_heads, dim, v_dim, ctypes.c_float(scale),
        int(window or 0), ctypes.c_float(lam), ctypes.c_float(out_scale), ctypes.c_float(eps), _stream())
    _check(rc, "diff_attention_prefill")
    return out


def diff_prepare(proj, bias, heads, kv_heads, dim, v_dim, gate_width, temperature, tok_pos, tok_slot,
                 block_table, k_store, v_store, write_cache=True):
    """Finish the projections of a differential attention and file the new keys and values.

    ``proj`` ``[T, heads * 2 * dim + gate_width (+ kv_heads * 2 * dim + kv_heads * v_dim)]`` is the
    stacked product ``[q | gate | k | v]`` (the last two only with ``write_cache``); ``bias`` float32
    of the same width or None.  Returns the queries ``[T, heads * 2 * dim]`` with their bias added and
    scaled by ``1 + coef * ln(floor((p + 1) / every) + 1)`` at position ``p`` (``temperature = (coef,
    every)`` or None).  Keys go to ``k_store`` ``[pages, kv_heads, 64, 2 * dim]``, values to ``v_store``
    ``[pages, kv_heads, 64, v_dim]``; the gate columns are left where they are."""
    _need(proj, "proj", None, 2)
    n_tokens = proj.shape[0]
    q_w = heads * 2 * dim
    width = q_w + gate_width + (kv_heads * (2 * dim + v_dim) if write_cache else 0)
    if proj.shape[1] != width:
        raise KernelError(f"the stacked projection has width {proj.shape[1]}, expected {width}")
    if bias is not None:
        _f32(bias, "bias", (width,))
    _need(tok_pos, "tok_pos", torch.int32, 1)
    _need(tok_slot, "tok_slot", torch.int32, 1)
    _need(block_table, "block_table", torch.int32, 2)
    if write_cache:
        _need(k_store, "key pages", proj.dtype, 4)
        _need(v_store, "value pages", proj.dtype, 4)
        if tuple(k_store.shape[1:]) != (kv_heads, PAGE_TOKENS, 2 * dim) or \
                tuple(v_store.shape[1:]) != (kv_heads, PAGE_TOKENS, v_dim):
            raise KernelError(f"cache pages have shapes {tuple(k_store.shape)} and {tuple(v_store.shape)}, expected "
                              f"[pages, {kv_heads}, {PAGE_TOKENS}, {2 * dim}] and [pages, {kv_heads}, {PAGE_TOKENS}, {v_dim}]")
    coef, every = temperature if temperature is not None else (0.0, 0)
    q_out = torch.empty((n_tokens, q_w), dtype=proj.dtype, device=proj.device)
    rc = _lib("attention_diff").sb_diff_prepare(
        _code(proj.dtype), _ptr(proj), proj.shape[1], _ptr(bias), _ptr(q_out), _ptr(tok_pos), _ptr(tok_slot),
        _ptr(block_table), block_table.shape[1], _ptr(k_store if write_cache else None),
        _ptr(v_store if write_cache else None), n_tokens, heads, kv_heads, dim, v_dim, gate_width,
        ctypes.c_float(coef), int(every), int(write_cache), _stream())
    _check(rc, "diff_prepare")
    return q_out


def _diff_check(q, gate, k_store, v_store, heads, kv_heads, dim, v_dim):
    _need(q, "q", None, 2)
    if q.shape[1] != heads * 2 * dim:
        raise KernelError(f"q has width {q.shape[1]}, expected {heads * 2 * dim}")
    if 2 * dim > DIFF_MAX_ROW or v_dim > DIFF_MAX_ROW:
        raise KernelError(f"differential attention takes 2 * dim and v_dim up to {DIFF_MAX_ROW}, got {2 * dim} and {v_dim}")
    if heads % kv_heads:
        raise KernelError(f"{heads} query heads cannot share {kv_heads} key/value heads")
    _need(k_store, "key pages", q.dtype, 4)
    _need(v_store, "value pages", q.dtype, 4)
    if tuple(k_store.shape[1:]) != (kv_heads, PAGE_TOKENS, 2 * dim) or \
            tuple(v_store.shape[1:]) != (kv_heads, PAGE_TOKENS, v_dim):
        raise KernelError(f"cache pages have shapes {tuple(k_store.shape)} and {tuple(v_store.shape)}")
    gate_stride = 0
    if gate is not None:
        if gate.dtype != q.dtype or gate.dim() != 2 or gate.stride(1) != 1 or gate.shape[1] != heads * v_dim \
                or gate.shape[0] != q.shape[0]:
            raise KernelError(f"the gate must be [T, {heads * v_dim}] of {q.dtype} with unit column stride")
        gate_stride = gate.stride(0)
    return gate_stride


def diff_attention(q, gate, k_store, v_store, block_table, tok_slot, tok_pos, heads, kv_heads, dim, v_dim,
                   scale, lam, out_scale, eps, window=None, warps=None, kv_hint=0):
    """Differential attention of each query row over its sequence's cached keys (csrc/attention_diff.cu):
    per head ``o = a1 - lam * a2`` from two softmax maps over the same values, divided by its root mean
    square over ``v_dim`` (``eps`` inside the root), times ``out_scale``, times ``sigmoid(gate)`` where
    ``gate`` ``[T, heads * v_dim]`` (a view with a row stride is fine) is given.  One block per (row,
    head); ``warps`` of it share the keys (chosen from ``kv_hint``, the longest sequence, when None)."""
    gate_stride = _diff_check(q, gate, k_store, v_store, heads, kv_heads, dim, v_dim)
    _need(block_table, "block_table", torch.int32, 2)
    _need(tok_slot, "tok_slot", torch.int32, 1)
    _need(tok_pos, "tok_pos", torch.int32, 1)
    if warps is None:
        warps = 1 if kv_hint <= 32 else 2 if kv_hint <= 128 else 4 if kv_hint <= 512 else 8
    out = torch.empty((q.shape[0], heads * v_dim), dtype=q.dtype, device=q.device)
    rc = _lib("attention_diff").sb_diff_attention(
        _code(q.dtype), _ptr(q), _ptr(gate), int(gate_stride), _ptr(out), _ptr(k_store), _ptr(v_store),
        _ptr(block_table), block_table.shape[1], _ptr(tok_slot), _ptr(tok_pos), q.shape[0], heads, kv_heads,
        dim, v_dim, ctypes.c_float(scale), int(window or 0), ctypes.c_float(lam), ctypes.c_float(out_scale),
        ctypes.c_float(eps), int(warps), _stream())
    _check(rc, "diff_attention")
    return out


def diff_attention_decode(q, gate, k_store, v_store, block_table, row_slot, row_kv_len, heads, kv_heads, dim, v_dim,
                          scale, lam, out_scale, eps, window=None, n_splits=None, kv_hint=0, early=False,
                          cluster=True):
    """``diff_attention`` for one new token per sequence, on tensor cores (bfloat16): the query heads
    of a key/value head are the MMA's rows, so a page is read once for all of them and both maps;
    each row's keys are cut into ``n_splits`` parts (chosen from ``kv_hint``, the longest sequence,
    so that the blocks fill the GPU).  Up to ``DIFF_CLUSTER_PARTS`` parts are the blocks of one
    thread-block cluster and join through distributed shared memory in the same launch (``cluster``
    false: never); more leave their results in scratch memory and a second kernel joins them.  Row
    ``i`` is the newest token of the sequence in ``row_slot[i]``, already in the cache;
    ``row_kv_len[i]`` counts it.

    ``early``: the caller vouches that ``row_kv_len``, the page table and every cached key and value
    but the newest token's were complete before this step's first kernel started (``embedding(...,
    fence=True)``) and that nothing else in this step writes them; the kernel then asks for its first
    pages before its dependent-launch wait, while the kernels before it still run."""
    gate_stride = _diff_check(q, gate, k_store, v_store, heads, kv_heads, dim, v_dim)
    if not diff_prefill_takes(q.dtype, dim, v_dim):
        raise KernelError(f"the tensor-core differential attention is not built for dim {dim}, v_dim {v_dim} in {q.dtype}")
    _need(block_table, "block_table", torch.int32, 2)
    _need(row_slot, "row_slot", torch.int32, 1)
    _need(row_kv_len, "row_kv_len", torch.int32, 1)
    rows = q.shape[0]
    if n_splits is None:
        blocks = rows * kv_heads * (-(-(heads // kv_heads) // 16))
        pages = max(1, -(-kv_hint // PAGE_TOKENS))
        # measured at 512 to 8,192 keys: all blocks resident at once (two fit on an SM); parts that join
        # inside a cluster want about three pages or more, parts that join through scratch memory and a
        # second launch seven (shorter ones pay the ring's start and the merge for too little
        # streaming), and those are worth it only when they are at least three times as many
        resident = (2 * 148) // max(blocks, 1)
        n_splits = max(1, min((pages + 1) // 3, resident, DIFF_CLUSTER_PARTS if cluster else 1))
        through_scratch = max(1, min(pages // 7, resident, 64))
        if through_scratch >= 3 * n_splits:
            n_splits = through_scratch
    out = torch.empty((rows, heads * v_dim), dtype=q.dtype, device=q.device)
    part = None
    if not cluster or n_splits > DIFF_CLUSTER_PARTS:
        part = torch.empty((rows * heads * n_splits * 2 * (v_dim + 2),), dtype=torch.float32, device=q.device)
    rc = _lib("attention_diff_prefill").sb_diff_decode(
        _ptr(q), _ptr(gate), int(gate_stride), _ptr(out), _ptr(k_store), _ptr(v_store), _ptr(block_table),
        block_table.shape[1], _ptr(row_slot), _ptr(row_kv_len), rows, heads, kv_heads, dim, v_dim,
        ctypes.c_float(scale), int(window or 0), ctypes.c_float(lam), ctypes.c_float(out_scale), ctypes.c_float(eps),
        int(n_splits), _ptr(part), int(bool(early) and EARLY_READS), int(bool(cluster)), _stream())
    # 0: one launch; 1: two (walk and merge); above: a CUDA error code plus one
    _check(rc - 1 if rc > 1 else 0 if rc == 1 else rc, "diff_attention_decode", 2 if rc == 1 else 1)
    return out


def diff_attention_step(q, gate, k_store, v_store, block_table, ctx, heads, kv_heads, dim, v_dim, scale, lam,
                        out_scale, eps, window=None):
    """The differential attention of one step, by the kernel that suits it: steps in which a sequence
    brings many tokens run the bfloat16 tensor-core kernel (64 queries of a head a block); steps of
    single tokens the tensor-core kernel whose rows are the heads of a key/value head; short chunks,
    the 32-bit path and sizes those kernels are not built for run one block per (row, head) whose warps
    share the keys."""
    if (ctx.max_q_len >= DIFF_PREFILL_MIN_Q and ctx.host is not None and diff_prefill_takes(q.dtype, dim, v_dim)
            and (gate is None or (gate.stride(0) % 2 == 0 and gate.data_ptr() % 4 == 0))):
        return diff_attention_prefill(q, gate, k_store, v_store, block_table, ctx.seq_slot, ctx.seq_q_start,
                                      ctx.seq_q_len, ctx.seq_kv_len, ctx.tile_seq, ctx.tile_first, heads,
                                      kv_heads, dim, v_dim, scale, lam, out_scale, eps, window,
                                      status=ctx.status, max_q_len=ctx.max_q_len)
    if ctx.max_q_len == 1 and diff_prefill_takes(q.dtype, dim, v_dim):
        return diff_attention_decode(q, gate, k_store, v_store, block_table, ctx.seq_slot, ctx.seq_kv_len, heads,
                                     kv_heads, dim, v_dim, scale, lam, out_scale, eps, window,
                                     kv_hint=ctx.max_kv_len, early=ctx.fenced)
    return diff_attention(q, gate, k_store, v_store, block_table, ctx.tok_slot, ctx.tok_pos, heads, kv_heads,
                          dim, v_dim, scale, lam, out_scale, eps, window, kv_hint=ctx.max_kv_len)


def add_bias(y, bias):
    """``y += bias`` in place (``bias`` float32 ``[N]``, the sum rounded once to ``y``'s type)."""
    _need(y, "y", None, 2)
    _f32(bias, "bias", (y.shape[1],))
    rc = _lib("streams").sb_add_bias(_code(y.dtype), _ptr(y), _ptr(bias), y.shape[0], y.shape[1], _stream())
    _check(rc, "add_bias")
    return y


# ---------------------------------------------------------------------------------------- sampling

def sample(logits, temperature=None, request_key=None, position=None, status=None, out=None, feed=None):
    """One token per row of float32 ``logits`` ``[B, V]``: argmax, or a draw where temperature > 0.

    ``feed = (tokens, positions, lengths)`` (int32 ``[B]`` each): the drawn token is also stored as
    the row's next input and its position and length are advanced by one."""
    _need(logits, "logits", torch.float32, 2)
    rows, vocab = logits.shape
    if temperature is not None:
        _need(temperature, "temperature", torch.float32, 1)
        _need(request_key, "request_key", torch.int32, 1)
        _need(position, "position", torch.int32, 1)
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    lib = _lib("sampling")
    chunks = lib.sb_sample_chunks(vocab)
    cand_v = torch.empty((rows * chunks,), dtype=torch.float32, device=logits.device)
    cand_i = torch.empty((rows * chunks,), dtype=torch.int32, device=logits.device)
    rc = lib.sb_sample(
        _ptr(logits), rows, vocab, ctypes.c_longlong(logits.stride(0)), _ptr(temperature),
        _ptr(request_key), _ptr(position), _ptr(out), _ptr(status),
        _ptr(feed[0] if feed else None), _ptr(feed[1] if feed else None),
        _ptr(feed[2] if feed else None), _ptr(cand_v), _ptr(cand_i), _stream())
    _check(rc, "sample", 2)
    return out


# ---------------------------------------------------------------------------------------- chains

CHAIN_MAX_ROWS = 64
CHAIN_MAX_STAGES = 8
CHAIN_MAX_LINEAR = 6
CHAIN_STATUS_BIT = 32
_chain_state = {}      # device index -> {"sync": int64[2], "partial": float32 arena}


def _chain_scratch(device, floats: int):
    """The chains of one device share two 64-bit words (grid-barrier counter, give-up flag) and one
    float arena for partial tiles.  A chain writes the arena only after the kernel before it on the
    stream has completed, so consecutive chains can use the same memory."""
    state = _chain_state.get(device.index)
    if state is None:
        state = _chain_state[device.index] = {
            "sync": torch.zeros((2,), dtype=torch.int64, device=device), "partial": None}
    if state["partial"] is None or state["partial"].numel() < floats:
        state["partial"] = torch.empty((max(floats, 1 << 20),), dtype=torch.float32, device=device)
    return state["sync"], state["partial"]


def reset_chains(device=None) -> None:
    """Clear the chains' shared words after a chain gave up (its barrier count is then off and every
    later chain on the device gives up at once until this is called)."""
    for index, state in _chain_state.items():
        if device is None or torch.device(device).index in (None, index):
            state["sync"].zero_()


class ChainValue:
    """A ``[rows, width]`` bfloat16 tensor that a chain which is still open will produce.  ``resolve``
    launches the chain and gives the tensor."""

    __slots__ = ("chain", "stage", "tensor", "shape")

    def __init__(self, chain, stage, tensor, shape):
        self.chain, self.stage, self.tensor, self.shape = chain, stage, tensor, shape

    @property
    def dtype(self):
        return torch.bfloat16


def resolve(value):
    """The tensor behind ``value``: a tensor as it is, a ``ChainValue`` after its chain has run."""
    if isinstance(value, ChainValue):
        value.chain.close()
        if value.tensor is None:
            raise KernelError("this value was summed straight into the norm after it and was never stored")
        return value.tensor
    return value


def chain_takes_linear(x, weight, gated: bool) -> bool:
    """Whether a chain can run ``x @ weight.T``: bfloat16, at most 64 rows, 16-byte aligned operands,
    k a multiple of 8, a gated width a multiple of 64."""
    rows, k_dim = x.shape
    n_total = weight.shape[0]
    if weight.dtype != torch.bfloat16 or x.dtype != torch.bfloat16 or not 1 <= rows <= CHAIN_MAX_ROWS:
        return False
    if k_dim % 8 or weight.data_ptr() % 16 or not weight.is_contiguous() or weight.shape[1] != k_dim:
        return False
    if gated and (n_total % 2 or (n_total // 2) % 64):
        return False
    return True


def chain_takes_norm(hidden: int, gain) -> bool:
    return hidden % 8 == 0 and hidden <= 16384 and gain.dtype in (torch.float32, torch.bfloat16) \
        and gain.data_ptr() % 16 == 0


class OpenChain:
    """Few-row projections and row norms that run as ONE persistent kernel (csrc/dense_chain.cu).

    Stages are added with ``linear`` and ``add_norm`` and run when the chain is closed (by ``close`` or
    by ``resolve`` of one of its values).  A stage may read tensors that exist when the chain is
    launched and values of earlier stages of the same chain."""

    def __init__(self, rows: int, device, status=None):
        if not 1 <= rows <= CHAIN_MAX_ROWS:
            raise KernelError(f"a chain runs 1 to {CHAIN_MAX_ROWS} rows, not {rows}")
        self.rows, self.device, self.status = rows, device, status
        self.stages = []
        self.closed = False
        #: None, or a zeroed int64 tensor [ctas, 64]: each CTA's time stamps (ns) at its stage boundaries
        self.trace = None
        self.n_ctas = _lib("dense_chain").sb_dense_chain_ctas()
        self.bm = 16 if rows <= 16 else 32 if rows <= 32 else 64

    # ------------------------------------------------------------------ building

    def room_for(self, linear: bool) -> bool:
        if self.closed or len(self.stages) >= CHAIN_MAX_STAGES:
            return False
        return not linear or sum(s["kind"] == 0 for s in self.stages) < CHAIN_MAX_LINEAR

    def _input(self, x, what):
        """(tensor, keep-alive) of a stage input: a tensor, or a stored value of this chain."""
        if isinstance(x, ChainValue):
            if x.chain is not self:
                return resolve(x)
            if x.tensor is None:
                raise KernelError(f"{what} was summed straight into a norm and cannot be read again")
            return x.tensor
        return x

    def linear(self, x, weight, gated=False) -> ChainValue:
        shape = x.shape
        xt = self._input(x, "the input of a projection")
        _need(xt, "x", torch.bfloat16, 2)
        _need(weight, "weight", torch.bfloat16, 2)
        if not chain_takes_linear(xt, weight, gated) or shape[0] != self.rows or not self.room_for(True):
            raise KernelError("this projection does not fit the chain (see chain_takes_linear)")
        n_out = weight.shape[0] // 2 if gated else weight.shape[0]
        out = torch.empty((self.rows, n_out), dtype=torch.bfloat16, device=self.device)
        parts = _lib("dense_chain").sb_dense_chain_parts(n_out, x.shape[1], int(gated), self.n_ctas)
        tiles = n_out // 64 if gated else -(-n_out // 128)
        self.stages.append({"kind": 0, "n_out": n_out, "k_dim": x.shape[1], "gated": int(gated), "store": 1,
                            "x": xt, "w": weight, "out": out, "parts": parts,
                            "floats": tiles * parts * self.bm * 128})
        return ChainValue(self, len(self.stages) - 1, out, (self.rows, n_out))

    def add_norm(self, residual, delta, gain, eps) -> ChainValue:
        """``residual += delta`` (in place, rounded) and its RMSNorm; ``delta`` None norms ``residual``
        alone; ``residual`` None norms ``delta`` alone.  A ``delta`` that is the value of the stage just
        before, a plain projection, is summed from that stage's partial tiles and never stored."""
        hidden = (residual if residual is not None else delta).shape[1]
        if not chain_takes_norm(hidden, gain) or not self.room_for(False):
            raise KernelError("this norm does not fit the chain (see chain_takes_norm)")
        fused = (isinstance(delta, ChainValue) and delta.chain is self and delta.stage == len(self.stages) - 1
                 and self.stages[-1]["kind"] == 0 and not self.stages[-1]["gated"] and delta.tensor is not None)
        if fused:
            self.stages[-1]["store"] = 0
            self.stages[-1]["out"] = None
            delta.tensor = None
            dt = None
        else:
            dt = self._input(delta, "the delta of a norm") if delta is not None else None
        if residual is not None:
            _need(residual, "residual", torch.bfloat16, 2)
        if dt is not None:
            _need(dt, "delta", torch.bfloat16, 2)
        normed = torch.empty((self.rows, hidden), dtype=torch.bfloat16, device=self.device)
        self.stages.append({"kind": 1, "hidden": hidden, "gain": gain, "eps": float(eps), "residual": residual,
                            "delta": dt, "normed": normed})
        return ChainValue(self, len(self.stages) - 1, normed, (self.rows, hidden))

    # ------------------------------------------------------------------ running

    def close(self) -> None:
        if self.closed:
            return
        self.closed = True
        if not self.stages:
            return
        floats = sum(s.get("floats", 0) for s in self.stages)
        sync, arena = _chain_scratch(self.device, floats)
        desc = (ctypes.c_longlong * (16 * len(self.stages)))()
        eps = (ctypes.c_float * len(self.stages))()
        at = 0
        for i, s in enumerate(self.stages):
            d = [0] * 16
            if s["kind"] == 0:
                partial = arena.data_ptr() + 4 * at
                at += s["floats"]
                d[:10] = [0, s["n_out"], s["k_dim"], s["gated"], s["store"], s["x"].data_ptr(), s["w"].data_ptr(),
                          s["out"].data_ptr() if s["out"] is not None else 0, partial, s["parts"]]
            else:
                d[:8] = [1, s["hidden"], int(s["gain"].dtype == torch.float32), int(s["residual"] is not None),
                         s["residual"].data_ptr() if s["residual"] is not None else 0,
                         s["delta"].data_ptr() if s["delta"] is not None else 0, s["gain"].data_ptr(),
                         s["normed"].data_ptr()]
                eps[i] = s["eps"]
            for j, v in enumerate(d):
                desc[16 * i + j] = v
        rc = _lib("dense_chain").sb_dense_chain(
            desc, eps, len(self.stages), self.rows, _ptr(sync), _ptr(self.status), ctypes.c_ulonglong(0),
            _ptr(self.trace), _stream())
        if rc in (-3, -4):
            raise KernelError(f"the TMA descriptors for a chain could not be made (code {rc})")
        _check(rc, "dense_chain")


# ---------------------------------------------------------------------------------------- a float32 residual stream

def embedding32(tokens, table, scale=1.0, status=None, fence=False, out=None):
    """``out[t] = float(table[tokens[t]]) * scale``: float32 ``[T, H]``, the start of a residual stream
    that is kept in 32-bit whatever the working type.  ``fence`` as in ``embedding``.  ``out``: where to
    write (float32 ``[T, H]``, contiguous) instead of a new tensor."""
    _need(tokens, "tokens", torch.int32, 1)
    _need(table, "table", None, 2)
    if out is None:
        out = torch.empty((tokens.shape[0], table.shape[1]), dtype=torch.float32, device=table.device)
    else:
        _f32(out, "out", (tokens.shape[0], table.shape[1]))
    rc = _lib("residual32").sb_embed32(
        _code(table.dtype), _ptr(tokens), _ptr(table), _ptr(out), tokens.shape[0], table.shape[1],
        table.shape[0], ctypes.c_float(scale), _ptr(status), int(fence), _stream())
    _check(rc, "embedding32")
    return out


def residual_norm(x, dtype, eps, pending=None, next_gain=None, rows=None):
    """One kernel between two sublayers of a model whose residual stream ``x`` is float32 ``[T, H]`` and
    whose sublayers have a norm behind them as well as in front.

    ``pending = (y, post_gain, bias, post_eps)``: the output ``y`` ``[T, H]`` (in ``dtype``) of the sublayer
    before, with a float32 ``bias`` ``[H]`` still to be added to it (or None); it is RMS-normed with
    ``post_gain`` (float32 ``[H]``; None: taken as it is) and ``post_eps`` and added onto ``x`` in place.  ``next_gain``
    (float32 ``[H]``): the RMS norm of the new row is returned in ``dtype``; None: nothing is returned.
    With ``rows`` (int32 ``[R]``) only those rows are computed, ``x`` is left as it was and the result is
    ``[R, H]``.  Sums, norms and the row itself are float32; the gains are the factors themselves."""
    _need(x, "x", torch.float32, 2)
    n_tokens, hidden = x.shape
    y = post = bias = None
    post_eps = eps
    if pending is not None:
        y, post, bias, post_eps = pending
        _need(y, "y", dtype, 2)
        if tuple(y.shape) != (n_tokens, hidden):
            raise KernelError(f"y {tuple(y.shape)} does not match the residual stream {tuple(x.shape)}")
        if post is not None:
            _f32(post, "post gain", (hidden,))
        if bias is not None:
            _f32(bias, "bias", (hidden,))
    n_rows = n_tokens
    if rows is not None:
        _need(rows, "rows", torch.int32, 1)
        n_rows = rows.shape[0]
    out = None
    if next_gain is not None:
        _f32(next_gain, "next gain", (hidden,))
        out = torch.empty((n_rows, hidden), dtype=dtype, device=x.device)
    rc = _lib("residual32").sb_residual_norm(
        _code(dtype), _ptr(x), _ptr(y), _ptr(bias), _ptr(post), _ptr(next_gain), _ptr(out), _ptr(rows), n_rows,
        hidden, ctypes.c_float(post_eps), ctypes.c_float(eps), _stream())
    _check(rc, "residual_norm")
    return out


#: what ``bias_act`` can apply after the bias
BIAS_ACTIVATIONS = {None: 0, "none": 0, "relu2": 1, "tanh": 2, "decay": 3}


def bias_act(x, bias=None, activation=None):
    """``act(x + bias)`` for ``x`` ``[T, N]`` and a float32 ``bias`` ``[N]`` (or None); ``activation``:
    None, ``"relu2"`` (the square of relu), ``"tanh"`` or ``"decay"`` (``exp(-exp(.))``: a recurrence's decay
    factor from the logarithm of its negated logarithm).  The sum and the activation are float."""
    _need(x, "x", None, 2)
    if activation not in BIAS_ACTIVATIONS:
        raise KernelError(f"no activation {activation!r} here (known: relu2, tanh)")
    if bias is not None:
        _f32(bias, "bias", (x.shape[1],))
    out = torch.empty_like(x)
    rc = _lib("residual32").sb_bias_act(_code(x.dtype), _ptr(x), _ptr(bias), _ptr(out), x.shape[0], x.shape[1],
                                        BIAS_ACTIVATIONS[activation], _stream())
    _check(rc, "bias_act")
    return out


# ---------------------------------------------------------------------------------------- recurrence with a matrix state

def wkv_max_dim() -> int:
    return _lib("wkv").sb_wkv_max_dim()


def token_shift(h, state, mu, tok_slot):
    """``out[s] = h + (previous(h) - h) * mu[s]`` for each of the ``mu`` ``[S, W]`` (float32): ``[S, T, W]`` in
    the type of ``h`` ``[T, W]``.  A row's predecessor is the row before it when that belongs to the same
    sequence, else the first ``W`` floats of its slot's ``state`` (float32 ``[slots, N]``): what the
    sequence's last token left there, zeros for a sequence that starts."""
    _need(h, "h", None, 2)
    _need(state, "state", torch.float32, 2)
    _need(mu, "mu", torch.float32, 2)
    _need(tok_slot, "tok_slot", torch.int32, 1)
    n_tokens, width = h.shape
    if mu.shape[1] != width or state.shape[1] < width:
        raise KernelError(f"mu {tuple(mu.shape)} / state {tuple(state.shape)} do not fit rows of {width}")
    out = torch.empty((mu.shape[0], n_tokens, width), dtype=h.dtype, device=h.device)
    rc = _lib("wkv").sb_token_shift(_code(h.dtype), _ptr(h), _ptr(state), ctypes.c_longlong(state.shape[1]), _ptr(mu),
                                    _ptr(out), _ptr(tok_slot), n_tokens, width, mu.shape[0], _stream())
    _check(rc, "token_shift")
    return out


def wkv_scan(r, k, v, decay, u, g, gain, state, h, seq_slot, seq_q_start, seq_q_len, heads, dim, eps):
    """The recurrence ``o_t = (S + diag(u) k_t v_t^T)^T r_t``, ``S <- diag(w_t) S + k_t v_t^T`` with
    the decay factors ``w_t`` per head over the sequences of a step, followed by the head's unit norm,
    ``gain`` and ``silu(g)``.

    ``r, k, v, g`` ``[T, heads * dim]`` in the working type; ``decay`` float32 of that shape (the factors
    themselves, in (0, 1)); ``gain`` float32 ``[heads * dim]``; ``u`` float32 ``[heads, dim]``.  ``state`` float32 ``[slots, W +
    heads * dim * dim]``: each slot's last mixer input (``h``'s row, ``W`` floats, written here for the
    sequence's last token of this step) and its ``S``, read at the start and written at the end.
    Returns ``[T, heads * dim]`` in the working type."""
    _need(r, "r", None, 2)
    n_tokens = r.shape[0]
    hd = heads * dim
    for name, t in (("k", k), ("v", v), ("g", g)):
        _need(t, name, r.dtype, 2)
        if tuple(t.shape) != (n_tokens, hd):
            raise KernelError(f"{name} has shape {tuple(t.shape)}, expected {(n_tokens, hd)}")
    if r.shape[1] != hd:
        raise KernelError(f"r has width {r.shape[1]}, expected {hd}")
    _f32(decay, "decay", (n_tokens, hd))
    _f32(gain, "gain", (hd,))
    _need(u, "u", torch.float32)
    if u.numel() != hd:
        raise KernelError(f"u has {u.numel()} entries, expected {hd}")
    _need(h, "h", r.dtype, 2)
    width = h.shape[1]
    _need(state, "state", torch.float32, 2)
    if state.shape[1] != width + heads * dim * dim:
        raise KernelError(f"a slot's state has {state.shape[1]} floats, expected {width + heads * dim * dim}")
    for name, t in (("seq_slot", seq_slot), ("seq_q_start", seq_q_start), ("seq_q_len", seq_q_len)):
        _need(t, name, torch.int32, 1)
    out = torch.empty_like(r)
    # many tokens of few sequences: scratch with which several blocks may share a head
    o32 = torch.empty((n_tokens, hd), dtype=torch.float32, device=r.device) if n_tokens >= 4 * seq_slot.shape[0] else None
    rc = _lib("wkv").sb_wkv_scan(
        _code(r.dtype), _ptr(r), _ptr(k), _ptr(v), _ptr(decay), _ptr(u), _ptr(g), _ptr(gain),
        _ptr(state), ctypes.c_longlong(state.shape[1]), width, _ptr(h), width, _ptr(out), _ptr(seq_slot),
        _ptr(seq_q_start), _ptr(seq_q_len), seq_slot.shape[0], heads, dim, ctypes.c_float(eps), _ptr(o32), n_tokens,
        _stream())
    if rc == -2:
        raise KernelError(f"the recurrence kernel takes heads of 1 to {wkv_max_dim()} channels, not {dim}")
    _check(rc, "wkv_scan", 2 if o32 is not None and dim == 64 and seq_slot.shape[0] * heads <= 74 else 1)
    return out


# ---------------------------------------------------------------------------------------- latent attention

def latent_max_row() -> int:
    return _lib("attention_latent").sb_latent_max_row()


#: the pairings the latent-attention kernels turn, and the code they take for each
LATENT_LAYOUTS = {"interleaved": 0, "half_split": 1}


def latent_tables(rotation, rot_dims: int):
    """``(cos, sin)`` for the latent-attention kernels: they turn the first ``rot_dims`` entries of the
    rotated part, entry ``2i`` with ``2i + 1`` (``"interleaved"``) or ``i`` with ``i + rot_dims / 2``
    (``"half_split"``); ``latent_prepare`` and ``latent_rotate_q`` take the layout's name."""
    if rotation is None:
        raise KernelError("latent attention needs a position part that offers a rotation")
    if rotation.layout not in LATENT_LAYOUTS or rotation.rotary_dim != rot_dims:
        raise KernelError(f"the latent-attention kernels turn {rot_dims} entries in interleaved or half-split layout; "
                          f"asked for {rotation.rotary_dim} in {rotation.layout!r} layout")
    return rotation.cos, rotation.sin


def latent_prepare(proj, q_gain, kv_gain, eps, cos_table, sin_table, tok_pos, tok_slot, block_table, store,
                   q_rank, rank, rot, rot_dims, write_cache=True, layout="interleaved"):
    """What follows a token's stacked down-projections ``proj`` = ``[query latent | key/value latent | shared
    key part]`` (the query latent alone with ``write_cache`` false): returns the RMS-normed query latent
    ``[T, q_rank]``; norms the key/value latent, turns the shared key part by the token's position and files
    both in the token's row of ``store`` ``[pages, 1, 64, rank + rot]``."""
    _need(proj, "proj", None, 2)
    n_tokens = proj.shape[0]
    want = q_rank + (rank + rot if write_cache else 0)
    if proj.shape[1] != want:
        raise KernelError(f"proj has width {proj.shape[1]}, expected {want}")
    _f32(q_gain, "query latent gain", (q_rank,))
    _f32(cos_table, "cos_table")
    _f32(sin_table, "sin_table")
    if cos_table.dim() != 2 or cos_table.shape[1] < rot_dims // 2 or sin_table.shape != cos_table.shape:
        raise KernelError("rotary tables must be [positions, at least rot_dims / 2]")
    _need(tok_pos, "tok_pos", torch.int32, 1)
    _need(tok_slot, "tok_slot", torch.int32, 1)
    _need(block_table, "block_table", torch.int32, 2)
    if write_cache:
        _f32(kv_gain, "key/value latent gain", (rank,))
        _need(store, "cache pages", proj.dtype, 4)
        if tuple(store.shape[1:]) != (1, PAGE_TOKENS, rank + rot):
            raise KernelError(f"cache pages have shape {tuple(store.shape)}, expected [pages, 1, {PAGE_TOKENS}, {rank + rot}]")
    cq = torch.empty((n_tokens, q_rank), dtype=proj.dtype, device=proj.device)
    rc = _lib("attention_latent").sb_latent_prepare(
        _code(proj.dtype), _ptr(proj), proj.shape[1], _ptr(q_gain), _ptr(kv_gain if write_cache else None),
        ctypes.c_float(eps), _ptr(cos_table), _ptr(sin_table), cos_table.shape[1], _ptr(tok_pos), _ptr(tok_slot),
        _ptr(block_table), block_table.shape[1], _ptr(store if write_cache else None), _ptr(cq), n_tokens, q_rank,
        rank, rot, rot_dims, int(write_cache), LATENT_LAYOUTS[layout], _stream())
    _check(rc, "latent_prepare")
    return cq


def latent_rotate_q(q, qa, cos_table, sin_table, tok_pos, heads, dim, rot, rot_dims, rank, layout="interleaved"):
    """Turns the last ``rot`` entries of every head of ``q`` ``[T, heads * (dim + rot)]`` by the token's
    position and files them behind the first ``rank`` entries of that head in ``qa`` ``[T, heads, rank + rot]``."""
    _need(q, "q", None, 2)
    _need(qa, "qa", q.dtype, 3)
    if q.shape[1] != heads * (dim + rot) or tuple(qa.shape) != (q.shape[0], heads, rank + rot):
        raise KernelError(f"q {tuple(q.shape)} / qa {tuple(qa.shape)} do not fit {heads} heads of {dim} + {rot}")
    rc = _lib("attention_latent").sb_latent_rotate_q(
        _code(q.dtype), _ptr(q), _ptr(qa), _ptr(cos_table), _ptr(sin_table), cos_table.shape[1], _ptr(tok_pos),
        q.shape[0], heads, dim, rot, rot_dims, rank, LATENT_LAYOUTS[layout], _stream())
    _check(rc, "latent_rotate_q")


def latent_attention(qa, store, block_table, tok_slot, tok_pos, heads, rank, rot, scale, window=None):
    """Softmax attention of every query row over its sequence's cached latent rows: ``qa`` ``[T, heads, rank
    + rot]`` (queries with the key up-projection folded in, then the rotated part), ``store`` ``[pages, 1,
    64, rank + rot]``; returns ``[T, heads, rank]``, the weighted sums of the latents."""
    _need(qa, "qa", None, 3)
    n_tokens = qa.shape[0]
    if tuple(qa.shape[1:]) != (heads, rank + rot):
        raise KernelError(f"qa has shape {tuple(qa.shape)}, expected [T, {heads}, {rank + rot}]")
    if rank + rot > latent_max_row():
        raise KernelError(f"latent rows of {rank + rot} entries exceed {latent_max_row()}")
    _need(store, "cache pages", qa.dtype, 4)
    if tuple(store.shape[1:]) != (1, PAGE_TOKENS, rank + rot):
        raise KernelError(f"cache pages have shape {tuple(store.shape)}")
    _need(block_table, "block_table", torch.int32, 2)
    _need(tok_slot, "tok_slot", torch.int32, 1)
    _need(tok_pos, "tok_pos", torch.int32, 1)
    out = torch.empty((n_tokens, heads, rank), dtype=qa.dtype, device=qa.device)
    rc = _lib("attention_latent").sb_latent_attention(
        _code(qa.dtype), _ptr(qa), _ptr(out), _ptr(store), _ptr(block_table), block_table.shape[1], _ptr(tok_slot),
        _ptr(tok_pos), n_tokens, heads, rank, rot, ctypes.c_float(scale), int(window or 0), _stream())
    _check(rc, "latent_attention")
    return out


def latent_tc_takes(dtype, rank: int, rot: int) -> bool:
    """Whether the tensor-core latent attention takes these sizes: bfloat16, ``rank`` and ``rot`` multiples
    of 16, ``rank`` up to 512 and rows of up to 640 entries."""
    return dtype == torch.bfloat16 and rank % 16 == 0 and rot % 16 == 0 and 16 <= rank <= 512 and rank + rot <= 640


def latent_attention_tc(qa, store, block_table, seq_slot, seq_q_start, seq_q_len, seq_kv_len, tile_seq, tile_first,
                        heads, rank, rot, scale, window=None, n_splits=1, max_q_len=0):
    """``latent_attention`` on tensor cores (bfloat16): a block takes the heads of consecutive tokens of a
    sequence (up to 64 query rows), which all score the same cache rows.  The ``seq_*`` arrays describe the
    sequences of the step, ``tile_seq`` / ``tile_first`` list its tiles of 64 tokens.  ``n_splits`` > 1 deals
    the keys of every block out to that many blocks, which a second kernel joins: for steps of few rows.
    ``max_q_len``: the most tokens a sequence brings, if known (fewer idle blocks are launched)."""
    _need(qa, "qa", torch.bfloat16, 3)
    n_tokens = qa.shape[0]
    if tuple(qa.shape[1:]) != (heads, rank + rot):
        raise KernelError(f"qa has shape {tuple(qa.shape)}, expected [T, {heads}, {rank + rot}]")
    if not latent_tc_takes(qa.dtype, rank, rot):
        raise KernelError(f"the tensor-core latent attention takes rank and rot in multiples of 16, rank up to 512 "
                          f"and rows up to 640; got {rank} and {rot}")
    _need(store, "cache pages", qa.dtype, 4)
    if tuple(store.shape[1:]) != (1, PAGE_TOKENS, rank + rot):
        raise KernelError(f"cache pages have shape {tuple(store.shape)}")
    _need(block_table, "block_table", torch.int32, 2)
    for name, t in (("seq_slot", seq_slot), ("seq_q_start", seq_q_start), ("seq_q_len", seq_q_len),
                    ("seq_kv_len", seq_kv_len), ("tile_seq", tile_seq), ("tile_first", tile_first)):
        _need(t, name, torch.int32, 1)
    out = torch.empty((n_tokens, heads, rank), dtype=qa.dtype, device=qa.device)
    part_acc = part_ml = None
    n_splits = max(1, int(n_splits))
    if n_splits > 1:
        part_acc = torch.empty((n_splits, n_tokens * heads, rank), dtype=torch.float32, device=qa.device)
        part_ml = torch.empty((n_splits, n_tokens * heads, 2), dtype=torch.float32, device=qa.device)
    rc = _lib("attention_latent").sb_latent_attention_tc(
        _ptr(qa), _ptr(out), _ptr(part_acc), _ptr(part_ml), _ptr(store), _ptr(block_table), block_table.shape[1],
        _ptr(seq_slot), _ptr(seq_q_start), _ptr(seq_q_len), _ptr(seq_kv_len), _ptr(tile_seq), _ptr(tile_first),
        tile_seq.shape[0], n_tokens, heads, rank, rot, ctypes.c_float(scale), int(window or 0), n_splits,
        int(max_q_len), _stream())
    _check(rc, "latent_attention_tc", 2 if n_splits > 1 else 1)
    return out


def latent_splits(rows: int, heads: int, window, kv_hint: int) -> int:
    """Into how many parts the keys of a single-token step are cut: enough blocks to fill the SMs, no part
    shorter than a block of 32 keys, at most 32."""
    blocks = rows * -(-heads // 64)
    keys = kv_hint if not window else min(window, max(kv_hint, 1))
    return max(1, min(32, 148 // max(1, blocks), -(-max(keys, 1) // 32)))


def latent_attention_step(qa, store, block_table, ctx, heads, rank, rot, scale, window=None):
    """``latent_attention`` for the step ``ctx`` describes, on the kernel that fits its shape: tensor cores
    for bfloat16 at sizes they take, the plain kernel otherwise (float32, other sizes)."""
    if latent_tc_takes(qa.dtype, rank, rot):
        splits = latent_splits(ctx.n_seqs, heads, window, ctx.max_kv_len) if ctx.max_q_len == 1 else 1
        return latent_attention_tc(qa, store, block_table, ctx.seq_slot, ctx.seq_q_start, ctx.seq_q_len,
                                   ctx.seq_kv_len, ctx.tile_seq, ctx.tile_first, heads, rank, rot, scale, window,
                                   splits, ctx.max_q_len)
    return latent_attention(qa, store, block_table, ctx.tok_slot, ctx.tok_pos, heads, rank, rot, scale, window)


# ---------------------------------------------------------------------------------------- routed experts

def moe_limits():
    lib = _lib("moe")
    return lib.sb_moe_max_experts(), lib.sb_moe_max_top()


#: how the chosen experts' weights are formed from their logits, and the code the router takes
MOE_SCORINGS = {"softmax_top": 0, "sigmoid_normalised": 1, "softmax_all": 2}
#: the experts the tile kernels know, and the code of their up pass (``gated_silu`` is the gated pass without clamps)
MOE_EXPERTS = {"gated_clamped": 1, "relu2": 2, "gated_silu": 1}


def moe_route(h, router, router_bias, top, scoring="softmax_top", weight_scale=1.0):
    """``(ids int32 [T, top], weights float32 [T, top])``: the ``top`` largest of ``router @ h + bias``
    (float32 ``[E, W]`` and ``[E]`` or None), and either the softmax over those alone or, with ``scoring``
    ``"sigmoid_normalised"``, their sigmoids divided by their sum (+ 1e-20) times ``weight_scale``."""
    if scoring not in MOE_SCORINGS:
        raise KernelError(f"no router scoring {scoring!r} (known: {', '.join(MOE_SCORINGS)})")
    _need(h, "h", None, 2)
    experts = router.shape[0]
    _f32(router, "router", (experts, h.shape[1]))
    if router_bias is not None:
        _f32(router_bias, "router bias", (experts,))
    ids = torch.empty((h.shape[0], top), dtype=torch.int32, device=h.device)
    weights = torch.empty((h.shape[0], top), dtype=torch.float32, device=h.device)
    rc = _lib("moe").sb_moe_route(_code(h.dtype), _ptr(h), _ptr(router), _ptr(router_bias), _ptr(ids), _ptr(weights),
                                  h.shape[0], h.shape[1], experts, top, MOE_SCORINGS[scoring],
                                  ctypes.c_float(weight_scale), _stream())
    if rc == -2:
        raise KernelError(f"the router takes up to {moe_limits()[0]} experts and {moe_limits()[1]} choices, not "
                          f"{experts} and {top}")
    _check(rc, "moe_route")
    return ids, weights


def moe_route_all(h, router, correction, top, groups=1, keep=1, weight_scale=1.0, shared_gate=False):
    """The router that scores by the softmax over ALL rows of ``router`` (float32 ``[N, W]``): ``(ids int32 [T, top],
    weights float32 [T, top])``, the ``top`` largest of ``score + correction`` (float32 ``[N]`` or None) among the
    outputs of the ``keep`` of ``groups`` equal groups of neighbours whose largest such number is largest (the lower
    index first among equals), weighted by their plain scores over their sum (+ 1e-20) times ``weight_scale``.  With
    ``shared_gate`` the router has one row more and a third result, float32 ``[T]``: the sigmoid of that row's
    product (the gate of a shared expert)."""
    _need(h, "h", None, 2)
    outputs = router.shape[0] - (1 if shared_gate else 0)
    _f32(router, "router", (router.shape[0], h.shape[1]))
    if correction is not None:
        _f32(correction, "correction", (outputs,))
    ids = torch.empty((h.shape[0], top), dtype=torch.int32, device=h.device)
    weights = torch.empty((h.shape[0], top), dtype=torch.float32, device=h.device)
    gate = torch.empty((h.shape[0],), dtype=torch.float32, device=h.device) if shared_gate else None
    rc = _lib("moe").sb_moe_route_all(_code(h.dtype), _ptr(h), _ptr(router), _ptr(correction), _ptr(ids), _ptr(weights),
                                      _ptr(gate), h.shape[0], h.shape[1], outputs, top, groups, keep,
                                      ctypes.c_float(weight_scale), _stream())
    if rc == -2:
        raise KernelError(f"the router takes up to {moe_limits()[0]} outputs and {moe_limits()[1]} choices among the "
                          f"kept groups, not {outputs} outputs, {top} choices, {keep} of {groups} groups")
    _check(rc, "moe_route_all")
    return (ids, weights, gate) if shared_gate else (ids, weights)


def moe_experts(h, ids, weights, gate_up, down, limit=0.0, expert="gated_clamped", tile_rows=None, status=None,
                identity=False, shared=None, shared_gate=None):
    """The chosen experts of every row and their weighted sum: ``gate_up`` ``[E, 2 * F, W]`` (an expert's
    gate rows, then its up rows), ``down`` ``[E, W, F]``; an expert is ``down(g * sigmoid(1.702 g) * (u +
    1))`` with ``g = min(gate(h), limit)`` and ``u = clamp(up(h), -limit, limit)``.  With ``expert``
    ``"relu2"`` the experts have no gate: ``gate_up`` is ``[E, F, W]`` and an expert is
    ``down(relu(up(h))^2)``.  Returns ``[T, W]``.  ``tile_rows`` names the tile kind (32: plain; 4: the few-row kernel;
    64 and 128: ``mma.sync`` tiles; 256: the grouped tcgen05 product over rows gathered in the experts' order) instead of
    the one the step's shape chooses: 4 up to four rows an expert on average, 128 from 128, 256 from 256.  ``status``: the
    device word a tcgen05 wait that ran out is noted in.

    ``expert`` ``"gated_silu"``: ``down(silu(gate(h)) * up(h))``, no clamps.  ``identity``: an id from ``E`` on names
    an expert without weights that hands the row itself on.  ``shared`` ``[T, W]`` with ``shared_gate`` float32
    ``[T]``: ``shared_gate[t] * shared[t]`` is added to row ``t`` of the result."""
    if expert not in MOE_EXPERTS:
        raise KernelError(f"no expert kind {expert!r} (known: {', '.join(MOE_EXPERTS)})")
    up_mode = MOE_EXPERTS[expert]
    if expert == "gated_silu":
        limit = 0.0                       # the gated pass without clamps
    elif up_mode == 1 and not limit > 0.0:
        raise KernelError(f"the clamped gate needs a positive limit, not {limit}")
    _need(h, "h", None, 2)
    if shared is not None:
        _need(shared, "shared", h.dtype, 2)
        _f32(shared_gate, "shared gate", (h.shape[0],))
        if tuple(shared.shape) != tuple(h.shape):
            raise KernelError(f"the shared expert's output {tuple(shared.shape)} does not match the rows {tuple(h.shape)}")
    extras = (_ptr(ids if identity else None), gate_up.shape[0], _ptr(h if identity else None), _ptr(shared),
              _ptr(shared_gate if shared is not None else None))
    _need(gate_up, "gate_up", h.dtype, 3)
    _need(down, "down", h.dtype, 3)
    _need(ids, "ids", torch.int32, 2)
    _need(weights, "weights", torch.float32, 2)
    n_tokens, width = h.shape
    experts, two_f, _ = gate_up.shape
    inner = two_f // 2 if up_mode == 1 else two_f
    top = ids.shape[1]
    if tuple(gate_up.shape) != (experts, (2 if up_mode == 1 else 1) * inner, width) or tuple(down.shape) != (experts, width, inner):
        raise KernelError(f"expert weights {tuple(gate_up.shape)} / {tuple(down.shape)} do not fit rows of {width}")
    lib = _lib("moe")
    n_pairs = n_tokens * top
    # 64 and 128: tensor-core tiles (128 with many rows an expert); 32: the plain ones
    bm = lib.sb_moe_tile_rows_for(_code(h.dtype), width, inner, ctypes.c_longlong(n_pairs), experts)
    if tile_rows is not None:
        if tile_rows not in (4, 32, 64, 128, 256) or (tile_rows != 32 and lib.sb_moe_tile_rows(_code(h.dtype), width, inner) != 64):
            raise KernelError(f"no expert tiles of {tile_rows} rows for {h.dtype}, width {width}, inner size {inner}")
        bm = int(tile_rows)
    max_tiles = -(-n_pairs // bm) + min(experts, n_pairs)
    capacity = max_tiles * bm
    meta = torch.empty((capacity + max_tiles + 1,), dtype=torch.int32, device=h.device)
    sorted_pairs, tile_expert, n_tiles = meta[:capacity], meta[capacity:capacity + max_tiles], meta[capacity + max_tiles:]
    rc = lib.sb_moe_align(_ptr(ids), n_pairs, experts, _ptr(sorted_pairs), capacity, _ptr(tile_expert), _ptr(n_tiles),
                          bm, _stream())
    _check(rc, "moe_align")
    act = torch.empty((capacity, inner), dtype=h.dtype, device=h.device)
    per_pair = torch.empty((n_pairs, width), dtype=h.dtype, device=h.device)
    if bm == 256:
        grouped = _lib("gemm_prompt_tcgen05").sb_gemm_prompt_grouped
        gathered = torch.empty((capacity, width), dtype=h.dtype, device=h.device)
        rc = lib.sb_moe_gather(_ptr(h), _ptr(sorted_pairs), _ptr(n_tiles), bm, top, _ptr(gathered), capacity, width, _stream())
        _check(rc, "moe_gather")
        rc = grouped(_ptr(gathered), _ptr(gate_up), _ptr(act), capacity, inner, width, experts, _ptr(tile_expert),
                     _ptr(n_tiles), max_tiles, None,
                     (GATE_CLAMPED if limit > 0.0 else ACTIVATIONS["silu"]) if up_mode == 1 else 0, 1 if up_mode == 2 else 0,
                     ctypes.c_float(limit), _ptr(status), _stream())
        _check(rc, "moe_up (grouped tcgen05)")
        rc = grouped(_ptr(act), _ptr(down), _ptr(per_pair), capacity, width, inner, experts, _ptr(tile_expert),
                     _ptr(n_tiles), max_tiles, _ptr(sorted_pairs), 0, 0, ctypes.c_float(0.0), _ptr(status), _stream())
        _check(rc, "moe_down (grouped tcgen05)")
        out = torch.empty_like(h)
        rc = lib.sb_moe_combine(_code(h.dtype), _ptr(per_pair), _ptr(weights), _ptr(out), n_tokens, width, top, *extras,
                                _stream())
        _check(rc, "moe_combine")
        return out
    rc = lib.sb_moe_tiles(_code(h.dtype), up_mode, bm, _ptr(h), _ptr(gate_up), _ptr(act), _ptr(sorted_pairs), _ptr(tile_expert),
                          _ptr(n_tiles), max_tiles, width, inner, top, ctypes.c_float(limit), _stream())
    _check(rc, "moe_up")
    rc = lib.sb_moe_tiles(_code(h.dtype), 0, bm, _ptr(act), _ptr(down), _ptr(per_pair), _ptr(sorted_pairs),
                          _ptr(tile_expert), _ptr(n_tiles), max_tiles, inner, width, top, ctypes.c_float(limit), _stream())
    _check(rc, "moe_down")
    out = torch.empty_like(h)
    rc = lib.sb_moe_combine(_code(h.dtype), _ptr(per_pair), _ptr(weights), _ptr(out), n_tokens, width, top, *extras,
                                _stream())
    _check(rc, "moe_combine")
    return out


# ---------------------------------------------------------------------------------------- a stream joined over depth

#: the norms ``depth_step`` can apply, and the code the kernel takes
DEPTH_NORMS = {"rmsnorm": 0, "layernorm": 1}


def depth_step(base, dtype, pending=None, mult=1.0, history=None, mix=None, dst=None, norm=None, rows=None):
    """One kernel between two sublayers of a model whose float32 residual stream is joined over depth.

    ``base`` float32 ``[T, H]``: the rows the sum starts from.  ``pending`` (``[T, H]`` in ``dtype``, or
    None): the output of the sublayer before; ``v = base + mult * pending``.  With ``mix`` (float32
    ``[levels]``) and ``history`` (float32 ``[>= levels, T, H]``): ``v`` is filed as ``history[levels - 1]``
    and the stream becomes ``x = sum_j mix[j] * history[j]``; otherwise ``x = v``.  ``dst`` (float32 ``[T,
    H]``, not ``base``): where ``x`` is written.  ``norm = (kind, gain, eps)`` with ``kind`` of
    ``DEPTH_NORMS`` and a float32 gain: the norm of ``x`` is returned in ``dtype``.  With ``rows`` (int32
    ``[R]``) only those rows are computed, nothing but the result is written, and it is ``[R, H]``."""
    _need(base, "base", torch.float32, 2)
    n_tokens, hidden = base.shape
    if pending is not None:
        _need(pending, "pending", dtype, 2)
        if tuple(pending.shape) != (n_tokens, hidden):
            raise KernelError(f"pending {tuple(pending.shape)} does not match the stream {tuple(base.shape)}")
    levels = 0
    if mix is not None:
        _need(mix, "mix", torch.float32, 1)
        levels = mix.shape[0]
        _need(history, "history", torch.float32, 3)
        if history.shape[0] < levels or tuple(history.shape[1:]) != (n_tokens, hidden):
            raise KernelError(f"history {tuple(history.shape)} does not hold {levels} levels of {tuple(base.shape)}")
    if dst is not None:
        _f32(dst, "dst", (n_tokens, hidden))
        if dst.data_ptr() == base.data_ptr():
            raise KernelError("dst must not be base")
    n_rows = n_tokens
    if rows is not None:
        _need(rows, "rows", torch.int32, 1)
        n_rows = rows.shape[0]
    out = gain = None
    eps, kind = 0.0, 0
    if norm is not None:
        name, gain, eps = norm
        if name not in DEPTH_NORMS:
            raise KernelError(f"no norm {name!r} here (known: {', '.join(DEPTH_NORMS)})")
        kind = DEPTH_NORMS[name]
        _f32(gain, "gain", (hidden,))
        out = torch.empty((n_rows, hidden), dtype=dtype, device=base.device)
    rc = _lib("depth").sb_depth_step(
        _code(dtype), _ptr(base), _ptr(pending), ctypes.c_float(mult), _ptr(history if mix is not None else None),
        ctypes.c_longlong(n_tokens * hidden), _ptr(mix), levels, _ptr(dst), _ptr(gain), _ptr(out), _ptr(rows), n_rows,
        hidden, ctypes.c_float(eps), kind, _stream())
    _check(rc, "depth_step")
    return out


def softcap(logits, cap):
    """``logits <- cap * tanh(logits / cap)`` in place (float32)."""
    _need(logits, "logits", torch.float32)
    rc = _lib("depth").sb_softcap(_ptr(logits), ctypes.c_longlong(logits.numel()), ctypes.c_float(cap), _stream())
    _check(rc, "softcap")
    return logits


def gated_clamped(gate_up, limit):
    """``g * sigmoid(1.702 g) * (u + 1)`` with ``g = min(gate, limit)``, ``u = clamp(up, -limit, limit)`` for
    ``gate_up = [gate | up]`` of shape ``[T, 2 * I]``."""
    _need(gate_up, "gate_up", None, 2)
    if gate_up.shape[1] % 2:
        raise KernelError(f"gate_up has an odd width {gate_up.shape[1]}")
    inner = gate_up.shape[1] // 2
    out = torch.empty((gate_up.shape[0], inner), dtype=gate_up.dtype, device=gate_up.device)
    rc = _lib("elementwise").sb_gated_clamped(_code(gate_up.dtype), _ptr(gate_up), _ptr(out), gate_up.shape[0], inner,
                                              ctypes.c_float(limit), _stream())
    _check(rc, "gated_clamped")
    return out


# ---------------------------------------------------------------------------------------- attention with a sink

def sink_max_dim() -> int:
    return _lib("attention_sink").sb_sink_max_dim()


def sink_prepare(proj, heads, kv_heads, dim, vdim, tok_pos, tok_slot, block_table, k_store, v_store, gated=True,
                 write_cache=True):
    """What follows a token's stacked projections ``proj`` = ``[q | k | v | g]`` (``[q | g]`` with
    ``write_cache`` false; no ``g`` with ``gated`` false; up to 7 unused entries may follow): files the keys and values in the token's cache
    row (``k_store`` ``[pages, kv_heads, 64, dim]``, ``v_store`` ``[pages, kv_heads, 64, vdim]``) and returns
    the gates ``sigmoid(g)`` as float32 ``[T, heads]`` (None without).  The queries stay where they are."""
    _need(proj, "proj", None, 2)
    n_tokens = proj.shape[0]
    want = heads * dim + (kv_heads * (dim + vdim) if write_cache else 0) + (heads if gated else 0)
    if not want <= proj.shape[1] < want + 8:
        raise KernelError(f"proj has width {proj.shape[1]}, expected {want} (and up to 7 entries of padding)")
    _need(tok_pos, "tok_pos", torch.int32, 1)
    _need(tok_slot, "tok_slot", torch.int32, 1)
    _need(block_table, "block_table", torch.int32, 2)
    if write_cache:
        _need(k_store, "key pages", proj.dtype, 4)
        _need(v_store, "value pages", proj.dtype, 4)
        if tuple(k_store.shape[1:]) != (kv_heads, PAGE_TOKENS, dim) or tuple(v_store.shape[1:]) != (kv_heads, PAGE_TOKENS, vdim):
            raise KernelError(f"cache pages have shapes {tuple(k_store.shape)} / {tuple(v_store.shape)}, expected "
                              f"[pages, {kv_heads}, {PAGE_TOKENS}, {dim}] / [.., {vdim}]")
    gate = torch.empty((n_tokens, heads), dtype=torch.float32, device=proj.device) if gated else None
    rc = _lib("attention_sink").sb_sink_prepare(
        _code(proj.dtype), _ptr(proj), proj.shape[1], _ptr(tok_pos), _ptr(tok_slot), _ptr(block_table),
        block_table.shape[1], _ptr(k_store if write_cache else None), _ptr(v_store if write_cache else None),
        _ptr(gate), n_tokens, heads, kv_heads, dim, vdim, int(write_cache), _stream())
    _check(rc, "sink_prepare")
    return gate


def sink_tables(rotation, dim: int):
    """``(cos, sin, dims)`` for ``sink_prepare_rot``: it turns the first ``dims`` entries of a head, entry ``2i``
    with ``2i + 1``; None: nothing turns."""
    if rotation is None:
        return None, None, 0
    if rotation.layout != "interleaved" or rotation.rotary_dim > dim or rotation.rotary_dim % 2:
        raise KernelError(f"this attention turns up to {dim} leading entries of a head in interleaved layout; asked for "
                          f"{rotation.rotary_dim} in {rotation.layout!r} layout")
    return rotation.cos, rotation.sin, rotation.rotary_dim


def sink_prepare_rot(proj, heads, kv_heads, dim, vdim, tok_pos, tok_slot, block_table, k_store, v_store, cos_table,
                     sin_table, rot_dims, values_from_keys=False, write_cache=True):
    """``sink_prepare`` for a layer with rotary positions and no gates: ``proj`` = ``[q | k | v]`` (``[q | k]`` with
    ``values_from_keys``, ``[q]`` with ``write_cache`` false; up to 7 unused entries may follow).  The first
    ``rot_dims`` entries of every query and key head turn by the token's position, entry ``2i`` with ``2i + 1``
    (float32 tables ``[positions, rot_dims / 2]``): the queries in place, the keys on their way into the cache.
    Values are filed as they are; with ``values_from_keys`` a head's value is its key before the turn."""
    _need(proj, "proj", None, 2)
    n_tokens = proj.shape[0]
    want = heads * dim + (kv_heads * (dim + (0 if values_from_keys else vdim)) if write_cache else 0)
    if not want <= proj.shape[1] < want + 8:
        raise KernelError(f"proj has width {proj.shape[1]}, expected {want} (and up to 7 entries of padding)")
    _need(tok_pos, "tok_pos", torch.int32, 1)
    _need(tok_slot, "tok_slot", torch.int32, 1)
    _need(block_table, "block_table", torch.int32, 2)
    if rot_dims:
        _need(cos_table, "cos table", torch.float32, 2)
        _need(sin_table, "sin table", torch.float32, 2)
        if cos_table.shape[1] != rot_dims // 2 or tuple(sin_table.shape) != tuple(cos_table.shape):
            raise KernelError(f"rotation tables {tuple(cos_table.shape)} do not turn {rot_dims} entries")
    if write_cache:
        _need(k_store, "key pages", proj.dtype, 4)
        _need(v_store, "value pages", proj.dtype, 4)
        if tuple(k_store.shape[1:]) != (kv_heads, PAGE_TOKENS, dim) or tuple(v_store.shape[1:]) != (kv_heads, PAGE_TOKENS, vdim):
            raise KernelError(f"cache pages have shapes {tuple(k_store.shape)} / {tuple(v_store.shape)}, expected "
                              f"[pages, {kv_heads}, {PAGE_TOKENS}, {dim}] / [.., {vdim}]")
    rc = _lib("attention_sink").sb_sink_prepare_rot(
        _code(proj.dtype), _ptr(proj), proj.shape[1], _ptr(tok_pos), _ptr(tok_slot), _ptr(block_table),
        block_table.shape[1], _ptr(k_store if write_cache else None), _ptr(v_store if write_cache else None),
        _ptr(cos_table if rot_dims else None), _ptr(sin_table if rot_dims else None), int(rot_dims), n_tokens, heads,
        kv_heads, dim, vdim, int(values_from_keys), int(write_cache), _stream())
    if rc == -2:
        raise KernelError(f"sink_prepare_rot: rot_dims={rot_dims} must be even and at most dim={dim}; values taken from "
                          f"keys need vdim == dim (got {vdim})")
    _check(rc, "sink_prepare_rot")


def _sink_check(q, k_store, v_store, heads, kv_heads, dim, vdim, penalty, sink, gate):
    _need(q, "q", None, 2)
    if q.shape[1] < heads * dim:
        raise KernelError(f"q rows of {q.shape[1]} entries do not hold {heads} heads of {dim}")
    _need(k_store, "key pages", q.dtype, 4)
    _need(v_store, "value pages", q.dtype, 4)
    if tuple(k_store.shape[1:]) != (kv_heads, PAGE_TOKENS, dim) or tuple(v_store.shape[1:]) != (kv_heads, PAGE_TOKENS, vdim):
        raise KernelError(f"cache pages have shapes {tuple(k_store.shape)} / {tuple(v_store.shape)}")
    r1 = r2 = None
    if penalty is not None:
        r1, r2 = penalty
        _f32(r1, "r1", (heads,))
        _f32(r2, "r2", (heads,))
    if sink is not None:
        _f32(sink, "sink", (heads,))
    if gate is not None:
        _f32(gate, "gate", (q.shape[0], heads))
    return r1, r2


def sink_attention(q, k_store, v_store, block_table, tok_slot, tok_pos, heads, kv_heads, dim, vdim, scale,
                   penalty=None, sink=None, gate=None, chunk=None, window=None):
    """Attention of every query row over its sequence's cached keys, plain kernel (any sizes up to
    ``sink_max_dim()``, both types).  ``q``: rows whose first ``heads * dim`` entries are the queries (a
    stacked projection may carry more behind them).  ``penalty = (r1, r2)``: ``r1_h ln(1 + r2_h (i - j))`` is
    taken off the scaled scores; ``sink``: one more term ``exp(sink_h)`` in the softmax's denominator;
    ``gate`` float32 ``[T, heads]``: multiplies the head's output; ``chunk``: keys of the query's own chunk of
    that many positions only; ``window``: the most recent that many keys.  Returns ``[T, heads * vdim]``."""
    r1, r2 = _sink_check(q, k_store, v_store, heads, kv_heads, dim, vdim, penalty, sink, gate)
    _need(block_table, "block_table", torch.int32, 2)
    _need(tok_slot, "tok_slot", torch.int32, 1)
    _need(tok_pos, "tok_pos", torch.int32, 1)
    out = torch.empty((q.shape[0], heads * vdim), dtype=q.dtype, device=q.device)
    rc = _lib("attention_sink").sb_sink_attention(
        _code(q.dtype), _ptr(q), q.shape[1], _ptr(out), _ptr(k_store), _ptr(v_store), _ptr(block_table),
        block_table.shape[1], _ptr(tok_slot), _ptr(tok_pos), _ptr(r1), _ptr(r2), _ptr(sink), _ptr(gate), q.shape[0],
        heads, kv_heads, dim, vdim, ctypes.c_float(scale), int(chunk or 0), int(window or 0), _stream())
    _check(rc, "sink_attention")
    return out


SINK_TC_DIMS = (16, 32, 64, 128)


def sink_tc_takes(q, heads, kv_heads, dim, vdim) -> bool:
    """Whether the tensor-core kernel takes these operands: bfloat16, ``dim`` and ``vdim`` of 16, 32, 64 or
    128, up to 64 query heads a key/value head, query rows that start on 16-byte boundaries."""
    return (q.dtype == torch.bfloat16 and dim in SINK_TC_DIMS and vdim in SINK_TC_DIMS and heads // kv_heads <= 64
            and q.shape[1] % 8 == 0 and q.data_ptr() % 16 == 0)


def sink_splits(rows: int, kv_heads: int, chunk, window, kv_hint: int) -> int:
    """Into how many parts the pages of a single-token step are cut: enough blocks for two an SM, no part
    shorter than a page, at most 16."""
    keys = max(kv_hint, 1)
    for bound in (chunk, window):
        if bound:
            keys = min(keys, bound)
    pages = -(-keys // PAGE_TOKENS) + 1
    return max(1, min(16, (2 * 148) // max(1, rows * kv_heads), pages))


def sink_attention_tc(q, k_store, v_store, block_table, seq_slot, seq_q_start, seq_q_len, seq_kv_len, tile_seq,
                      tile_first, heads, kv_heads, dim, vdim, scale, penalty=None, sink=None, gate=None, chunk=None,
                      window=None, n_splits=1, max_q_len=0):
    """``sink_attention`` on tensor cores (bfloat16): a block takes one key/value head and the query heads
    that share it for consecutive tokens of a sequence (up to 64 rows), so a page is fetched once for all
    of them.  The ``seq_*`` arrays describe the sequences of the step, ``tile_seq`` / ``tile_first`` list
    its tiles of 64 tokens.  ``n_splits`` > 1 deals the pages of every block out to that many blocks, which
    a second kernel joins: for steps of few rows."""
    r1, r2 = _sink_check(q, k_store, v_store, heads, kv_heads, dim, vdim, penalty, sink, gate)
    if not sink_tc_takes(q, heads, kv_heads, dim, vdim):
        raise KernelError(f"the tensor-core attention takes bfloat16 heads of 16, 32, 64 or 128 entries in rows "
                          f"that are multiples of 8 wide; got {q.dtype}, {dim} / {vdim}, rows of {q.shape[1]}")
    _need(block_table, "block_table", torch.int32, 2)
    for name, t in (("seq_slot", seq_slot), ("seq_q_start", seq_q_start), ("seq_q_len", seq_q_len),
                    ("seq_kv_len", seq_kv_len), ("tile_seq", tile_seq), ("tile_first", tile_first)):
        _need(t, name, torch.int32, 1)
    n_tokens = q.shape[0]
    out = torch.empty((n_tokens, heads * vdim), dtype=q.dtype, device=q.device)
    part_acc = part_ml = None
    n_splits = max(1, int(n_splits))
    if n_splits > 1:
        part_acc = torch.empty((n_splits, n_tokens * heads, vdim), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n_splits, n_tokens * heads, 2), dtype=torch.float32, device=q.device)
    rc = _lib("attention_sink_tc").sb_sink_attention_tc(
        _ptr(q), q.shape[1], _ptr(out), _ptr(part_acc), _ptr(part_ml), _ptr(k_store), _ptr(v_store), _ptr(block_table),
        block_table.shape[1], _ptr(seq_slot), _ptr(seq_q_start), _ptr(seq_q_len), _ptr(seq_kv_len), _ptr(tile_seq),
        _ptr(tile_first), tile_seq.shape[0], _ptr(r1), _ptr(r2), _ptr(sink), _ptr(gate), n_tokens, heads, kv_heads,
        dim, vdim, ctypes.c_float(scale), int(chunk or 0), int(window or 0), n_splits, int(max_q_len), _stream())
    _check(rc, "sink_attention_tc", 2 if n_splits > 1 else 1)
    return out


def sink_tcgen05_takes(q, dim, vdim) -> bool:
    """Whether the tcgen05 prompt kernel takes these operands: bfloat16, keys and values of one size, 64 or
    128, query rows that are a multiple of 8 wide and start on 16-byte boundaries."""
    return (q.dtype == torch.bfloat16 and dim == vdim and dim in PREFILL_TC_HEAD_DIMS and q.shape[1] % 8 == 0
            and q.data_ptr() % 16 == 0)


def sink_attention_tcgen05(q, k_store, v_store, block_table, seq_slot, seq_q_start, seq_q_len, seq_kv_len, tile_seq,
                           tile_first, heads, kv_heads, dim, scale, penalty=None, sink=None, gate=None, chunk=None,
                           window=None, status=None, blocks=None):
    """``sink_attention`` for prompts on the tcgen05 kernel of ``attention_prefill`` (256 queries of a head a
    block, S and O in tensor memory), which takes the penalty, the chunks, the sink and the gate as extras.
    ``blocks = (block_seq, block_first)``: the work list in blocks of 256 queries (else the tiles of 64 are
    launched and three of four blocks find nothing to do)."""
    r1, r2 = _sink_check(q, k_store, v_store, heads, kv_heads, dim, dim, penalty, sink, gate)
    if not sink_tcgen05_takes(q, dim, dim):
        raise KernelError(f"the tcgen05 attention takes bfloat16 heads of 64 or 128 entries, keys and values alike, in "
                          f"rows that are multiples of 8 wide; got {q.dtype}, {dim}, rows of {q.shape[1]}")
    if not scale > 0:
        raise KernelError("the tcgen05 attention needs a positive scale")
    _need(block_table, "block_table", torch.int32, 2)
    for name, t in (("seq_slot", seq_slot), ("seq_q_start", seq_q_start), ("seq_q_len", seq_q_len),
                    ("seq_kv_len", seq_kv_len), ("tile_seq", tile_seq), ("tile_first", tile_first)):
        _need(t, name, torch.int32, 1)
    own_list = blocks is not None and blocks[0] is not None
    if own_list:
        for name, t in (("block_seq", blocks[0]), ("block_first", blocks[1])):
            _need(t, name, torch.int32, 1)
    list_seq, list_first = blocks if own_list else (tile_seq, tile_first)
    out = torch.empty((q.shape[0], heads * dim), dtype=q.dtype, device=q.device)
    rc = _lib("attention_prefill_tc").sb_sink_attention_tcgen05(
        _ptr(q), q.shape[1], _ptr(out), _ptr(k_store), _ptr(v_store), _ptr(block_table), block_table.shape[1],
        _ptr(seq_slot), _ptr(seq_q_start), _ptr(seq_q_len), _ptr(seq_kv_len), _ptr(list_seq), _ptr(list_first),
        list_seq.shape[0], q.shape[0], k_store.shape[0], heads, kv_heads, dim, ctypes.c_float(scale), _ptr(r1), _ptr(r2),
        _ptr(sink), _ptr(gate), int(chunk or 0), int(window or 0), _ptr(status), int(own_list), _stream())
    _check(rc, "sink_attention_tcgen05")
    return out


def sink_attention_step(q, k_store, v_store, block_table, ctx, heads, kv_heads, dim, vdim, scale, penalty=None,
                        sink=None, gate=None, chunk=None, window=None):
    """``sink_attention`` for the step ``ctx`` describes, on the kernel that fits its shape: for bfloat16 the
    tcgen05 kernel when a sequence brings more than 128 tokens and keys and values have 64 or 128 entries, the
    mma.sync kernel for other steps and sizes it takes; the plain kernel otherwise (float32, other sizes)."""
    if ctx.max_q_len > 128 and scale > 0 and sink_tcgen05_takes(q, dim, vdim):
        return sink_attention_tcgen05(q, k_store, v_store, block_table, ctx.seq_slot, ctx.seq_q_start, ctx.seq_q_len,
                                      ctx.seq_kv_len, ctx.tile_seq, ctx.tile_first, heads, kv_heads, dim, scale, penalty,
                                      sink, gate, chunk, window, ctx.status, (ctx.block_seq, ctx.block_first))
    if sink_tc_takes(q, heads, kv_heads, dim, vdim):
        splits = sink_splits(ctx.n_seqs, kv_heads, chunk, window, ctx.max_kv_len) if ctx.max_q_len == 1 else 1
        return sink_attention_tc(q, k_store, v_store, block_table, ctx.seq_slot, ctx.seq_q_start, ctx.seq_q_len,
                                 ctx.seq_kv_len, ctx.tile_seq, ctx.tile_first, heads, kv_heads, dim, vdim, scale,
                                 penalty, sink, gate, chunk, window, splits, ctx.max_q_len)
    return sink_attention(q, k_store, v_store, block_table, ctx.tok_slot, ctx.tok_pos, heads, kv_heads, dim, vdim,
                          scale, penalty, sink, gate, chunk, window)


def linear_gated_clamped(x, weight, limit, status=None):
    """``g * sigmoid(1.702 g) * (u + 1)`` with ``g = min(x @ gate.T, limit)`` and ``u = clamp(x @ up.T, -limit,
    limit)`` for ``weight = [gate; up]`` stacked (``[2 * I, K]``); returns ``[T, I]``.  In bfloat16 the
    activation is the epilogue of the tensor-core products (few rows; 512 rows and more) where they take the
    operands; elsewhere the product is followed by ``gated_clamped``."""
    _need(x, "x", None, 2)
    _need(weight, "weight", x.dtype, 2)
    rows, k_dim = x.shape
    n_total = weight.shape[0]
    if weight.shape[1] != k_dim or n_total % 2:
        raise KernelError(f"weight {tuple(weight.shape)} is no stacked [gate; up] for inputs of width {k_dim}")
    n_out = n_total // 2
    fused = x.dtype == torch.bfloat16 and rows > 0 and tensor_core_ok(x, weight, True, n_out)
    if fused and rows <= TENSOR_CORE_MAX_ROWS:
        bm, splits, stages = gemm_plan(rows, n_out, k_dim, True)
        stages = min(max(stages, -(-bm * 512 // (16384 + bm * 128))), (226 * 1024) // (16384 + bm * 128))
        out = torch.empty((rows, n_out), dtype=torch.bfloat16, device=x.device)
        rc = _lib("gemm_tcgen05").sb_gemm_tcgen05_clamped(_ptr(x), _ptr(weight), _ptr(out), rows, n_out, k_dim, bm, splits,
                                                          stages, ctypes.c_float(limit), _ptr(status), _stream())
        _check(rc, "gemm_tcgen05 (clamped gate)")
        return out
    if fused and rows >= PROMPT_MIN_ROWS:
        out = torch.empty((rows, n_out), dtype=torch.bfloat16, device=x.device)
        rc = _lib("gemm_prompt_tcgen05").sb_gemm_prompt_clamped(_ptr(x), _ptr(weight), _ptr(out), rows, n_out, k_dim, 0, 0,
                                                                ctypes.c_float(limit), _ptr(status), _stream())
        _check(rc, "gemm_prompt_tcgen05 (clamped gate)")
        return out
    return gated_clamped(linear(x, weight, status=status), limit)


# ---------------------------------------------------------------------------------------- per-channel recurrences

def _at(t, offset: int):
    """The address of element ``offset`` of a contiguous tensor."""
    return ctypes.c_void_p(t.data_ptr() + offset * t.element_size())


def _seq_arrays(seq_slot, seq_q_start, seq_q_len):
    for name, t in (("seq_slot", seq_slot), ("seq_q_start", seq_q_start), ("seq_q_len", seq_q_len)):
        _need(t, name, torch.int32, 1)
    return seq_slot.shape[0]


def conv_max_taps() -> int:
    return _lib("short_conv").sb_conv_max_taps()


def short_conv(x, col, channels, taps, bias, in_bias, state, state_at, seq_slot, seq_q_start, seq_q_len, max_q_len,
               activation=None):
    """A causal convolution over time with one filter per channel, over the sequences of a step:
    ``y[t, c] = act(bias[c] + sum_j taps[c, K - 1 - j] * (x[t - j, col + c] + in_bias[c]))``, zeros in front of a
    sequence.  ``x`` ``[T, N]`` (the channels are its columns ``col .. col + channels``); ``taps`` float32
    ``[channels, K]``; ``bias``, ``in_bias`` float32 ``[channels]`` or None; ``activation`` None or ``"silu"``.
    ``state`` float32 ``[slots, M]``: a slot's last ``K - 1`` inputs (``(K - 1) * channels`` floats from
    ``state_at`` on) stand in front of the tokens it brings and are replaced by the step's last ones.
    ``max_q_len``: the most tokens a sequence brings.  Returns ``[T, channels]`` in the type of ``x``."""
    _need(x, "x", None, 2)
    _need(taps, "taps", torch.float32, 2)
    k = taps.shape[1]
    if taps.shape[0] != channels:
        raise KernelError(f"taps {tuple(taps.shape)} do not filter {channels} channels")
    if bias is not None:
        _f32(bias, "bias", (channels,))
    if in_bias is not None:
        _f32(in_bias, "in_bias", (channels,))
    _need(state, "state", torch.float32, 2)
    if col < 0 or col + channels > x.shape[1] or state_at < 0 or state_at + (k - 1) * channels > state.shape[1]:
        raise KernelError(f"{channels} channels from column {col} of rows of {x.shape[1]}, or {k - 1} rows of them from "
                          f"float {state_at} of a slot's {state.shape[1]}, do not fit")
    if activation not in (None, "silu"):
        raise KernelError(f"the short convolution applies silu or nothing, not {activation!r}")
    n_seqs = _seq_arrays(seq_slot, seq_q_start, seq_q_len)
    y = torch.empty((x.shape[0], channels), dtype=x.dtype, device=x.device)
    rc = _lib("short_conv").sb_short_conv(
        _code(x.dtype), _at(x, col), x.shape[1], _ptr(taps), _ptr(bias), _ptr(in_bias), _ptr(y), channels,
        _at(state, state_at), ctypes.c_longlong(state.shape[1]), _ptr(seq_slot), _ptr(seq_q_start), _ptr(seq_q_len),
        n_seqs, int(max_q_len), channels, k, 1 if activation == "silu" else 0, _stream())
    if rc == -2:
        raise KernelError(f"the short convolution takes 1 to {conv_max_taps()} taps, not {k}")
    _check(rc, "short_conv")
    return y


def glru_scan(u, gates, r_bias, i_bias, lam, decay_scale, proj, y_col, y_bias, state, state_at, seq_slot, seq_q_start,
              seq_q_len, max_q_len):
    """The real-gated linear recurrent unit over the sequences of a step, per channel ``c`` of ``C``:
    ``r = sigmoid(zr + r_bias)``, ``i = sigmoid(zi + i_bias)``, ``a = exp(-decay_scale * r * softplus(lam))``,
    ``S <- a S + sqrt(1 - a^2) i u`` and the result ``S * gelu_tanh(y + y_bias)``.  ``u`` ``[T, C]``; ``gates`` float32
    ``[blocks, T, 2 * C / blocks]``: for each block of channels its ``zr`` then its ``zi``; ``y`` = columns ``y_col ..
    y_col + C`` of ``proj`` ``[T, N]``; the biases and ``lam`` float32 ``[C]`` (``y_bias`` may be None).  ``state``
    float32 ``[slots, M]``: a slot's ``S`` is its ``C`` floats from ``state_at`` on.  Returns ``[T, C]``."""
    _need(u, "u", None, 2)
    n_tokens, channels = u.shape
    _need(gates, "gates", torch.float32, 3)
    blocks = gates.shape[0]
    if blocks < 1 or channels % blocks or tuple(gates.shape) != (blocks, n_tokens, 2 * channels // blocks):
        raise KernelError(f"gate logits {tuple(gates.shape)} do not fit {n_tokens} tokens of {channels} channels")
    for name, t in (("r_bias", r_bias), ("i_bias", i_bias), ("lam", lam)):
        _f32(t, name, (channels,))
    if y_bias is not None:
        _f32(y_bias, "y_bias", (channels,))
    _need(proj, "proj", u.dtype, 2)
    _need(state, "state", torch.float32, 2)
    if proj.shape[0] != n_tokens or y_col < 0 or y_col + channels > proj.shape[1] or state_at + channels > state.shape[1]:
        raise KernelError("the gated branch or the state does not hold the channels asked for")
    n_seqs = _seq_arrays(seq_slot, seq_q_start, seq_q_len)
    out = torch.empty_like(u)
    rc = _lib("short_conv").sb_glru_scan(
        _code(u.dtype), _ptr(u), channels, _ptr(gates), n_tokens, channels // blocks, _ptr(r_bias), _ptr(i_bias), _ptr(lam),
        ctypes.c_float(decay_scale), _at(proj, y_col), proj.shape[1], _ptr(y_bias), _ptr(out), _at(state, state_at),
        ctypes.c_longlong(state.shape[1]), _ptr(seq_slot), _ptr(seq_q_start), _ptr(seq_q_len), n_seqs, int(max_q_len),
        channels, _stream())
    _check(rc, "glru_scan")
    return out


# ---------------------------------------------------------------------------------------- recurrences with a matrix state

SCAN_MODES = {"state_space": 0, "gated_delta": 1}


def scan_max_state() -> int:
    return _lib("state_scan").sb_scan_max_state()


def state_scan(mode, q, k, v, a_raw, b_raw, A_log, dt_bias, skip, state, state_at, seq_slot, seq_q_start, seq_q_len,
               heads, groups, n_state, v_dim):
    """A linear recurrence with a state ``S`` ``[n_state, v_dim]`` per head over the sequences of a step.

    ``q, k, v, a_raw, b_raw`` are ``(tensor [T, N], first column)`` pairs of the working type: ``groups`` heads of
    ``n_state`` queries and keys (head ``h`` reads ``h // (heads // groups)``), ``heads`` heads of ``v_dim`` values,
    ``heads`` entries each of ``a_raw`` and ``b_raw``.  ``A_log``, ``dt_bias`` (and ``skip`` or None) float32 ``[heads]``.

    ``"state_space"``: ``dt = softplus(a_raw + dt_bias)``, ``S <- exp(-exp(A_log) dt) S + k (dt v)^T``, ``o = S^T q +
    skip * v`` (``b_raw`` None).  ``"gated_delta"``: q and k made unit vectors (``x / sqrt(sum x^2 + 1e-6)``), q times
    ``n_state ** -0.5``; ``S <- exp(-exp(A_log) softplus(a_raw + dt_bias)) S``, ``u = sigmoid(b_raw) (v - S^T k)``, ``S
    <- S + k u^T``, ``o = S^T q``.  ``state`` float32 ``[slots, M]``: a slot's ``[heads, n_state, v_dim]`` from
    ``state_at`` on, read at the start and written at the end.  Returns float32 ``[T, heads * v_dim]``."""
    if mode not in SCAN_MODES:
        raise KernelError(f"no recurrence {mode!r} (known: {', '.join(SCAN_MODES)})")
    dtype = q[0].dtype
    n_tokens = q[0].shape[0]
    args = []
    for name, pair, width in (("q", q, groups * n_state), ("k", k, groups * n_state), ("v", v, heads * v_dim),
                              ("a_raw", a_raw, heads), ("b_raw", b_raw, heads)):
        if pair is None:
            args += [ctypes.c_void_p(0), 0]
            continue
        t, col = pair
        _need(t, name, dtype, 2)
        if t.shape[0] != n_tokens or col < 0 or col + width > t.shape[1]:
            raise KernelError(f"{name}: {width} columns from {col} of {tuple(t.shape)} do not fit {n_tokens} tokens")
        args += [_at(t, col), t.shape[1]]
    _f32(A_log, "A_log", (heads,))
    _f32(dt_bias, "dt_bias", (heads,))
    if skip is not None:
        _f32(skip, "skip", (heads,))
    _need(state, "state", torch.float32, 2)
    if state_at < 0 or state_at + heads * n_state * v_dim > state.shape[1]:
        raise KernelError(f"a slot's {state.shape[1]} floats do not hold {heads} states of {n_state} x {v_dim} from {state_at}")
    n_seqs = _seq_arrays(seq_slot, seq_q_start, seq_q_len)
    out = torch.empty((n_tokens, heads * v_dim), dtype=torch.float32, device=state.device)
    rc = _lib("state_scan").sb_state_scan(
        _code(dtype), SCAN_MODES[mode], *args, _ptr(A_log), _ptr(dt_bias), _ptr(skip), _at(state, state_at),
        ctypes.c_longlong(state.shape[1]), _ptr(out), _ptr(seq_slot), _ptr(seq_q_start), _ptr(seq_q_len), n_seqs, heads,
        groups, n_state, v_dim, _stream())
    if rc == -2:
        raise KernelError(f"the recurrence takes states of 1 to {scan_max_state()} rows and heads in whole groups, not "
                          f"{n_state} rows, {heads} heads, {groups} groups")
    _check(rc, "state_scan")
    return out


def group_norm_gate(o, z, z_col, weight, parts, eps, gate_first, dtype):
    """The RMS norm of each of the ``parts`` equal parts of a float32 row ``o`` ``[T, N]`` with ``silu`` of the
    gate ``z`` (columns ``z_col .. z_col + N`` of a ``[T, M]`` tensor of ``dtype``): ``gate_first``: ``rms(o *
    silu(z)) * w``; else ``rms(o) * w * silu(z)``.  ``weight`` float32 of ``N`` entries, or of one part's size when
    the parts share it.  Returns ``[T, N]`` in ``dtype``."""
    _need(o, "o", torch.float32, 2)
    n_tokens, width = o.shape
    _need(z, "z", dtype, 2)
    _need(weight, "weight", torch.float32, 1)
    if parts < 1 or width % parts or z.shape[0] != n_tokens or z_col < 0 or z_col + width > z.shape[1]:
        raise KernelError(f"rows of {width} in {parts} parts with a gate from column {z_col} of {tuple(z.shape)} do not fit")
    if weight.shape[0] not in (width, width // parts):
        raise KernelError(f"a gain of {weight.shape[0]} entries fits neither the row ({width}) nor a part ({width // parts})")
    y = torch.empty((n_tokens, width), dtype=dtype, device=o.device)
    rc = _lib("state_scan").sb_group_norm_gate(_code(dtype), _ptr(o), _at(z, z_col), z.shape[1], _ptr(weight),
                                               weight.shape[0], _ptr(y), n_tokens, parts, width // parts,
                                               ctypes.c_float(eps), 0 if gate_first else 1, _stream())
    _check(rc, "group_norm_gate")
    return y


def norm_pair_mean(a, b, gain_a, gain_b, eps):
    """``(rms(a) * gain_a + rms(b) * gain_b) / 2`` row by row for ``a``, ``b`` ``[T, W]`` and float32 gains ``[W]``."""
    _need(a, "a", None, 2)
    _need(b, "b", a.dtype, 2)
    if tuple(a.shape) != tuple(b.shape):
        raise KernelError(f"rows {tuple(a.shape)} and {tuple(b.shape)} differ")
    _f32(gain_a, "gain_a", (a.shape[1],))
    _f32(gain_b, "gain_b", (a.shape[1],))
    out = torch.empty_like(a)
    rc = _lib("state_scan").sb_norm_pair_mean(_code(a.dtype), _ptr(a), _ptr(b), _ptr(gain_a), _ptr(gain_b), _ptr(out),
                                              a.shape[0], a.shape[1], ctypes.c_float(eps), _stream())
    _check(rc, "norm_pair_mean")
    return out
