"""bfloat16 tensor-core attention kernels, one build per head size."""

from __future__ import annotations

from typing import Any

import os

import numpy as np
import torch

from . import native
from ..errors import KernelError
from .native import c_float, c_int, c_void_p

c_long = native.ctypes.c_long
MAX_HEAD_DIM = 256
_CTAS_PER_SM = 4         # resident CTAs of the cp.async decode kernel on one SM (registers allow four)
_MIN_KEYS_PER_SPLIT = 128

_TABLE = {
    "b200_attention_head_dim": [],
    "b200_attention_prefill_rows": [],
    "b200_attention_prefill_bf16": [c_void_p] * 6 + [c_int, c_int, c_int, c_int, c_float, c_int] + [c_void_p] * 3 + [c_int, c_void_p],
    "b200_attention_decode_scratch_floats": [c_int, c_int, c_int],
    "b200_attention_decode_bf16": [c_void_p] * 6 + [c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_long, c_void_p],
}


_TMA_TABLE = {
    "b200_attention_decode_tma_head_dim": [],
    "b200_attention_decode_tma_ctas_per_sm": [],
    "b200_attention_decode_tma_scratch_floats": [c_int, c_int, c_int],
    "b200_attention_decode_tma_tickets": [c_int, c_int, c_int],
    "b200_attention_decode_tma_error": [],
    "b200_attention_decode_tma": [c_void_p] * 6 + [c_int] * 6 + [c_float, c_int, c_void_p, c_long, c_void_p, c_long]
                                 + [c_void_p, c_void_p],
    "b200_attention_decode_tma_fused": [c_void_p, c_int, c_void_p, c_void_p, c_float, c_void_p] + [c_void_p] * 5 + [c_int] * 6
                                       + [c_float, c_int, c_void_p, c_long, c_void_p, c_long]
                                       + [c_void_p, c_void_p],
}
FUSE_DECODE = os.environ.get("LLM_RUNTIME_STUDY_B200_FUSE_DECODE", "1") != "0"
# "tma": pages streamed by TMA, parts merged in the same launch; "mma": the cp.async kernels of attention_mma.cu
DECODE_BACKEND = os.environ.get("LLM_RUNTIME_STUDY_B200_DECODE_ATTENTION", "tma")
# Stages of each warp's ring: 3 keeps most bytes in flight when few CTAs share the machine; with one
# stage more CTAs (and warps) fit on an SM, which is what a batch that fills every SM several times
# needs.  LLM_RUNTIME_STUDY_B200_DECODE_DEPTH forces one value.
DECODE_DEPTHS = (1, 3)
_FORCED_DEPTH = int(os.environ.get("LLM_RUNTIME_STUDY_B200_DECODE_DEPTH", "0"))
DEEP_RING_MAX_CTAS = int(os.environ.get("LLM_RUNTIME_STUDY_B200_DECODE_DEEP_MAX", "296"))
TMA_MAX_SPLITS = 64

_TC_TABLE = {
    "b200_attention_tcgen05_error": [],
    "b200_attention_tcgen05_tokens_per_tile": [c_int],
    "b200_attention_prefill_tcgen05": [c_void_p] * 6 + [c_int, c_int, c_int, c_int, c_int, c_int, c_float] + [c_void_p] * 3 + [c_int, c_void_p],
    "b200_attention_prefill_tcgen05_pair": [c_void_p] * 6 + [c_int, c_int, c_int, c_int, c_int, c_int, c_float] + [c_void_p] * 3 + [c_int, c_void_p],
}
# Two row tiles per CTA (one CTA per SM, 128 keys a tile) for steps with a portion of at least this many tokens
# (measured at the Qwen3-8B geometry: half again as fast at 2,048 new tokens and beyond, 7 % slower at 1,024);
# below it the one-tile kernel (64 keys a tile).  0 turns the two-tile kernel off.
TC_PAIR_MIN_PORTION = int(os.environ.get("LLM_RUNTIME_STUDY_B200_ATTENTION_PAIR_MIN", "1280"))
TC_HEAD_DIMS = (64, 128)
TC_PAGE_SIZES = (8, 16, 32, 64)
TC_MIN_PORTION = 32     # shorter portions only: the mma.sync kernel wastes fewer rows
PREFILL_BACKEND = os.environ.get("LLM_RUNTIME_STUDY_B200_ATTENTION", "tcgen05")


def tc_library_name(head_dim: int) -> str:
    name = f"b200_attention_tcgen05_d{head_dim}"
    if name not in native.library_specs():
        native.register_library(name, ("attention_tcgen05.cu",), _TC_TABLE, defines=(f"HEAD_DIM={head_dim}",))
        native.register_error_probe(name, "b200_attention_tcgen05_error", f"tcgen05 attention (head size {head_dim})")
    return name


def tc_supported(head_dim: int, page_size: int, window: int) -> bool:
    """The tcgen05 kernel takes head sizes 64 and 128, pages of 8 to 64 tokens, no window."""

    return head_dim in TC_HEAD_DIMS and page_size in TC_PAGE_SIZES and not window


def tma_library_name(head_dim: int, depth: int = 3) -> str:
    name = f"b200_attention_decode_tma_d{head_dim}_s{depth}"
    if name not in native.library_specs():
        native.register_library(name, ("attention_decode_tma.cu",), _TMA_TABLE,
                                defines=(f"HEAD_DIM={head_dim}", f"DECODE_DEPTH={depth}"))
        native.register_error_probe(name, "b200_attention_decode_tma_error", f"TMA decode attention (head size {head_dim})")
    return name


def tma_depth(ctas: int) -> int:
    """Ring depth for a launch whose (request, KV head, slice) triples number ``ctas``."""

    if _FORCED_DEPTH:
        return _FORCED_DEPTH
    return DECODE_DEPTHS[1] if ctas <= DEEP_RING_MAX_CTAS else DECODE_DEPTHS[0]


def tma_supported(head_dim: int, page_size: int, window: int) -> bool:
    """The TMA decode kernel takes head sizes that are multiples of 64, pages of a multiple of 16 tokens, no window."""

    return head_dim % 64 == 0 and head_dim <= MAX_HEAD_DIM and page_size % 16 == 0 and not window


def library_name(head_dim: int) -> str:
    name = f"b200_attention_mma_d{head_dim}"
    if name not in native.library_specs():
        native.register_library(name, ("attention_mma.cu",), _TABLE, defines=(f"HEAD_DIM={head_dim}",))
    return name


def supported(head_dim: int) -> bool:
    return head_dim % 16 == 0 and 16 <= head_dim <= MAX_HEAD_DIM


def build(head_dim: int) -> None:
    """Compile the kernels for one head size."""

    from ..csrc.build import build_library

    name = library_name(head_dim)
    build_library(name, ("attention_mma.cu",), native.library_defines(name))
    if head_dim in TC_HEAD_DIMS:
        name = tc_library_name(head_dim)
        build_library(name, ("attention_tcgen05.cu",), native.library_defines(name))
    if head_dim % 64 == 0:
        for depth in DECODE_DEPTHS:
            name = tma_library_name(head_dim, depth)
            build_library(name, ("attention_decode_tma.cu",), native.library_defines(name))


def decode_splits(requests: int, kv_heads: int, slices: int, longest: int, slots: int = 0, head_dim: int = 128) -> int:
    """Into how many parts each sequence is cut, from a small model of the launch's time: the CTAs
    of all parts run in rounds of ``slots`` (what fits on the GPU at once); a CTA streams its part's
    keys and values at what one SM can pull (about 40 GB/s) or at its share of the memory
    bandwidth, whichever is less; every further part costs the merge a fraction of a microsecond.
    A part is not shorter than two tiles of keys, and there are at most 64."""

    slots = slots or _CTAS_PER_SM * native.sm_count()
    ctas = max(1, requests * kv_heads * slices)
    most = max(1, -(-longest // _MIN_KEYS_PER_SPLIT))
    bytes_per_key = 4 * head_dim                     # K and V rows of one KV head, bfloat16
    best, best_cost = 1, None
    for s in range(1, min(most, 64) + 1):
        rounds = -(-(ctas * s) // slots)
        keys = -(-(-(-longest // s)) // 64) * 64     # a part is a multiple of 64 keys
        rate = min(40.0, 6000.0 / min(ctas * s, slots))                 # GB/s = KB/us per CTA
        cost = rounds * keys * bytes_per_key / (rate * 1e3) + 0.15 * s  # microseconds
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = s, cost
    return best


def tile_map(q_lens, tokens_per_tile: int, device, kv_lens=None) -> tuple[torch.Tensor, int]:
    """Cut every entry into tiles of consecutive tokens: rows [entry, first token, count].
    With ``kv_lens`` (each entry's length after this step) the tiles are ordered by
    falling number of keys they attend to, so that the longest start first and the
    short ones fill the tail of the launch."""

    rows, first = [], 0
    for entry, n in enumerate(q_lens):
        before = 0 if kv_lens is None else kv_lens[entry] - n
        for s in range(0, n, tokens_per_tile):
            count = min(tokens_per_tile, n - s)
            rows.append((before + s + count, entry, first + s, count))
        first += n
    if kv_lens is not None:
        rows.sort(key=lambda r: -r[0])
    table = np.ascontiguousarray(np.asarray([r[1:] for r in rows], dtype=np.int32).T)
    return torch.from_numpy(table).to(device), len(rows)


def _geometry(q: torch.Tensor, keys: torch.Tensor):
    n, nq, d = q.shape
    nkv, page_size = keys.shape[1], keys.shape[2]
    if keys.shape[3] != d or nq % nkv:
        raise KernelError(f"attention shapes do not fit: q {tuple(q.shape)}, cache {tuple(keys.shape)}")
    group = nq // nkv
    gs = min(group, 16)
    return n, nq, d, nkv, page_size, gs, -(-group // gs)


def prefill_attention(
    q: torch.Tensor, keys: torch.Tensor, values: torch.Tensor, *, positions: torch.Tensor, block_table: torch.Tensor,
    q_lens, scale: float, window: int = 0, tiles: tuple[torch.Tensor, int] | None = None,
) -> torch.Tensor:
    """Causal attention for a batch whose entries hold ``q_lens[i]`` consecutive
    tokens each (prompt portions and single tokens alike); ``block_table[i]`` is
    entry ``i``'s row."""

    for t, name in ((q, "q"), (keys, "keys"), (values, "values")):
        native.require(t, name, dtype=torch.bfloat16)
    n, nq, d, nkv, page_size, gs, _ = _geometry(q, keys)
    lib = library_name(d)
    if tiles is None:
        tiles = tile_map(q_lens, 64 // gs, q.device)
    table, count = tiles
    out = torch.empty_like(q)
    native.call(
        "b200_attention_prefill_bf16", q.data_ptr(), keys.data_ptr(), values.data_ptr(), out.data_ptr(),
        positions.data_ptr(), block_table.data_ptr(), block_table.shape[1], page_size, nq, nkv, float(scale), int(window),
        table[0].data_ptr(), table[1].data_ptr(), table[2].data_ptr(), count, native.stream_ptr(), library=lib)
    return out


def prefill_attention_tcgen05(
    q: torch.Tensor, keys: torch.Tensor, values: torch.Tensor, *, positions: torch.Tensor, block_table: torch.Tensor,
    q_lens, scale: float, tiles: tuple[torch.Tensor, int] | None = None, pair: bool = False,
) -> torch.Tensor:
    """The same contract as ``prefill_attention`` (no window), on tcgen05 tensor cores with
    TMEM accumulators and TMA loads of the pages.  ``pair``: the kernel with two row tiles
    per CTA; ``tiles`` must then hold tiles of ``2 * (128 // gs)`` tokens."""

    for t, name in ((q, "q"), (keys, "keys"), (values, "values")):
        native.require(t, name, dtype=torch.bfloat16)
    n, nq, d, nkv, page_size, gs, _ = _geometry(q, keys)
    if not tc_supported(d, page_size, 0):
        raise KernelError(f"the tcgen05 attention kernel does not take head size {d} with pages of {page_size}")
    lib = tc_library_name(d)
    if tiles is None:
        tiles = tile_map(q_lens, (2 if pair else 1) * (128 // gs), q.device)
    table, count = tiles
    out = torch.empty_like(q)
    native.call(
        "b200_attention_prefill_tcgen05_pair" if pair else "b200_attention_prefill_tcgen05", q.data_ptr(), keys.data_ptr(), values.data_ptr(), out.data_ptr(),
        positions.data_ptr(), block_table.data_ptr(), block_table.shape[1], page_size, keys.shape[0], n, nq, nkv,
        float(scale), table[0].data_ptr(), table[1].data_ptr(), table[2].data_ptr(), count, native.stream_ptr(),
        library=lib)
    return out


def check_tcgen05_error(head_dim: int) -> None:
    """Synchronise and raise if a bounded wait inside the tcgen05 attention kernel ran out."""

    code = native.query("b200_attention_tcgen05_error", library=tc_library_name(head_dim))
    if code:
        raise KernelError(f"tcgen05 attention: a bounded wait ran out (code {code})")


def decode_attention(
    q: torch.Tensor, keys: torch.Tensor, values: torch.Tensor, *, kv_len: torch.Tensor, block_table: torch.Tensor,
    scale: float, window: int = 0, splits: int = 1, backend: str | None = None, live: "LiveParts | None" = None,
) -> torch.Tensor:
    """One query token per request (row ``i`` of ``q`` belongs to row ``i`` of
    ``block_table``) over its ``kv_len[i]`` cached keys, the sequence cut into
    ``splits`` parts that are merged afterwards.  ``backend``: "tma" or "mma";
    by default the TMA kernel wherever it takes the shape."""

    for t, name in ((q, "q"), (keys, "keys"), (values, "values")):
        native.require(t, name, dtype=torch.bfloat16)
    n, nq, d, nkv, page_size, _, _ = _geometry(q, keys)
    if (backend or DECODE_BACKEND) == "tma" and tma_supported(d, page_size, window) and splits <= TMA_MAX_SPLITS:
        return _decode_attention_tma(q, keys, values, kv_len, block_table, scale, splits, live)
    lib = library_name(d)
    floats = native.query("b200_attention_decode_scratch_floats", n, nq, splits, library=lib)
    scratch = torch.empty(max(floats, 1), dtype=torch.float32, device=q.device)
    out = torch.empty_like(q)
    native.call(
        "b200_attention_decode_bf16", q.data_ptr(), keys.data_ptr(), values.data_ptr(), out.data_ptr(),
        kv_len.data_ptr(), block_table.data_ptr(), block_table.shape[1], page_size, n, nq, nkv, float(scale),
        int(window), splits, scratch.data_ptr(), floats, native.stream_ptr(), library=lib,
        launches=2 if splits > 1 else 1)
    return out


_TICKETS: dict[tuple, list[torch.Tensor]] = {}


def _tickets(device: torch.device, count: int) -> torch.Tensor:
    """Zeroed counters that the TMA decode kernel leaves at zero after every launch; one buffer
    per device, made on first use.  A larger one replaces it when needed, and the old ones are
    kept for good: a captured graph may still hold their address."""

    made = _TICKETS.setdefault((device.type, device.index), [])
    if not made or made[-1].numel() < count:
        made.append(torch.zeros(max(count, 4096), dtype=torch.int32, device=device))
    return made[-1]


def decode_slots(head_dim: int, page_size: int, window: int, ctas: int = 1) -> int:
    """CTAs of the decode kernel that fit on the GPU at once."""

    if DECODE_BACKEND == "tma" and tma_supported(head_dim, page_size, window):
        return native.sm_count() * native.query("b200_attention_decode_tma_ctas_per_sm",
                                                library=tma_library_name(head_dim, tma_depth(ctas)))
    return _CTAS_PER_SM * native.sm_count()


def _decode_attention_tma(q, keys, values, kv_len, block_table, scale, splits, live=None) -> torch.Tensor:
    n, nq, d, nkv, page_size, _, _ = _geometry(q, keys)
    count = native.query("b200_attention_decode_tma_tickets", n, nq, nkv, library=tma_library_name(d))
    lib = tma_library_name(d, tma_depth(count))
    floats = native.query("b200_attention_decode_tma_scratch_floats", n, nq, splits, library=lib)
    scratch = torch.empty(max(floats, 1), dtype=torch.float32, device=q.device)
    tickets = _tickets(q.device, count)
    out = torch.empty_like(q)
    native.call(
        "b200_attention_decode_tma", q.data_ptr(), keys.data_ptr(), values.data_ptr(), out.data_ptr(), kv_len.data_ptr(),
        block_table.data_ptr(), block_table.shape[1], page_size, keys.shape[0], n, nq, nkv, float(scale), splits,
        scratch.data_ptr(), floats, tickets.data_ptr(), tickets.numel(),
        _live_argument(live, n, nq, nkv, d, page_size), native.stream_ptr(), library=lib)
    return out


PARTS_TABLE_SHIFT = 7       # the host's choices of parts are tabulated per 128 tokens of length


class LiveParts:
    """For decode attention launches that are recorded into a CUDA graph: a launch's grid is sized for ``bound``
    (the longest sequence there may ever be), and every replay uses as many parts as the host would choose for
    the longest sequence of *that* batch.  Each kind of launch (a geometry of heads and pages) registers once,
    while the graph is being made, and gets a place in ``values`` (device ints that travel with the step's other
    inputs); before every replay ``fill(longest)`` gives the numbers for all places."""

    def __init__(self, values: torch.Tensor, bound: int) -> None:
        self.values, self.bound = values, bound
        self._places: dict[tuple, int] = {}
        self._choices: list[list[int]] = []      # per place: parts by length >> PARTS_TABLE_SHIFT

    def place(self, requests: int, nq: int, nkv: int, d: int, page_size: int, window: int) -> torch.Tensor:
        key = (requests, nq, nkv, d, page_size, window)
        at = self._places.get(key)
        if at is None:
            if len(self._places) >= self.values.numel():
                raise KernelError(f"more than {self.values.numel()} kinds of decode attention in one captured step")
            at = self._places[key] = len(self._places)
            entries = (self.bound >> PARTS_TABLE_SHIFT) + 1
            # entry i serves the lengths i * 128 .. i * 128 + 127: what the host picks for the longest of them
            self._choices.append([parts_for(requests, nq, nkv, d, page_size, window, min(self.bound, ((i + 1) << PARTS_TABLE_SHIFT) - 1))
                                  for i in range(entries)])
        return self.values[at : at + 1]

    def most(self, requests: int, nq: int, nkv: int, d: int, page_size: int, window: int) -> int:
        """The largest number of parts any length up to the bound takes: what the recorded grid is sized for."""

        self.place(requests, nq, nkv, d, page_size, window)
        return max(self._choices[self._places[(requests, nq, nkv, d, page_size, window)]])

    def fill(self, longest: int) -> list[int]:
        """The numbers of parts, place by place, for a batch whose longest sequence holds ``longest`` tokens."""

        return [choices[min(max(longest, 0) >> PARTS_TABLE_SHIFT, len(choices) - 1)] for choices in self._choices]


def _live_argument(live: "LiveParts | None", n: int, nq: int, nkv: int, d: int, page_size: int):
    return None if live is None else live.place(n, nq, nkv, d, page_size, 0).data_ptr()


def fused_decode_supported(head_dim: int, page_size: int, window: int, rotary_dim: int) -> bool:
    """Whether the TMA decode kernel can itself normalise, rotate and store the new token's q, k and v: wherever
    it runs at all, provided the whole head is rotated or none of it."""

    return (FUSE_DECODE and DECODE_BACKEND == "tma" and tma_supported(head_dim, page_size, window)
            and rotary_dim in (0, head_dim))


def decode_attention_fused(
    qkv: torch.Tensor, keys: torch.Tensor, values: torch.Tensor, *, num_q_heads: int, q_weight: torch.Tensor | None,
    k_weight: torch.Tensor | None, eps: float, inv_freq: torch.Tensor | None, kv_len: torch.Tensor, block_table: torch.Tensor,
    scale: float, splits: int = 1, live: "LiveParts | None" = None,
) -> torch.Tensor:
    """Decode attention straight from the rows of the stacked q/k/v projection (``[requests, (nq + 2 nkv) d]``, one new
    token per request): per-head RMS norm of q and k (weights optional), rotation by the token's position
    ``kv_len - 1`` (``inv_freq`` optional), write of the new k and v into the pools, attention over all ``kv_len`` keys."""

    for t, name in ((qkv, "qkv"), (keys, "keys"), (values, "values")):
        native.require(t, name, dtype=torch.bfloat16)
    n = qkv.shape[0]
    nkv, page_size, d = keys.shape[1], keys.shape[2], keys.shape[3]
    nq = num_q_heads
    if qkv.dim() != 2 or qkv.shape[1] != (nq + 2 * nkv) * d or nq % nkv:
        raise KernelError(f"qkv rows of width {tuple(qkv.shape)} do not hold {nq} + 2 x {nkv} heads of {d}")
    if not tma_supported(d, page_size, 0) or splits > TMA_MAX_SPLITS:
        raise KernelError(f"the TMA decode kernel does not take head size {d} with pages of {page_size} in {splits} parts")
    for w, name in ((q_weight, "q_weight"), (k_weight, "k_weight")):
        if w is not None:
            native.require(w, name, dtype=torch.float32, shape=(d,))
    if inv_freq is not None:
        native.require(inv_freq, "inv_freq", dtype=torch.float32, shape=(d // 2,))
    count = native.query("b200_attention_decode_tma_tickets", n, nq, nkv, library=tma_library_name(d))
    lib = tma_library_name(d, tma_depth(count))
    floats = native.query("b200_attention_decode_tma_scratch_floats", n, nq, splits, library=lib)
    scratch = torch.empty(max(floats, 1), dtype=torch.float32, device=qkv.device)
    tickets = _tickets(qkv.device, count)
    out = torch.empty((n, nq, d), dtype=torch.bfloat16, device=qkv.device)
    native.call(
        "b200_attention_decode_tma_fused", qkv.data_ptr(), qkv.stride(0), native.ptr(q_weight), native.ptr(k_weight), float(eps),
        native.ptr(inv_freq), keys.data_ptr(), values.data_ptr(), out.data_ptr(), kv_len.data_ptr(), block_table.data_ptr(),
        block_table.shape[1], page_size, keys.shape[0], n, nq, nkv, float(scale), splits, scratch.data_ptr(), floats,
        tickets.data_ptr(), tickets.numel(), _live_argument(live, n, nq, nkv, d, page_size),
        native.stream_ptr(), library=lib)
    return out


def parts_for(n: int, nq: int, nkv: int, d: int, page_size: int, window: int, longest: int) -> int:
    """The number of parts the decode kernels cut each of ``n`` sequences into when the longest holds ``longest`` tokens."""

    slices = -(-(nq // nkv) // 16)
    if DECODE_BACKEND == "tma" and tma_supported(d, page_size, window):
        slices = -(-(nq // nkv) // 8)        # that kernel takes eight query heads of a group per CTA
    return decode_splits(n, nkv, slices, longest, decode_slots(d, page_size, window, n * nkv * slices), d)


def decode_parts(ctx: Any, n: int, nq: int, nkv: int, d: int, page_size: int, window: int) -> int:
    """The number of parts for this batch.  Under a graph capture: the most that any length up to the longest there
    may ever be would take (the choice does not grow steadily with the length), so that the recorded grid has room
    for whatever a replay is told to use."""

    live = getattr(ctx, "live_parts", None)
    if live is not None and not window:
        return live.most(n, nq, nkv, d, page_size, window)
    return parts_for(n, nq, nkv, d, page_size, window, ctx.max_kv_len)


def check_decode_tma_error(head_dim: int) -> None:
    """Raise if a wait inside the TMA decode kernel ever gave up (synchronises the device)."""

    for depth in DECODE_DEPTHS + ((_FORCED_DEPTH,) if _FORCED_DEPTH else ()):
        name = tma_library_name(head_dim, depth)
        if not native.library_loaded(name):
            continue
        code = native.query("b200_attention_decode_tma_error", library=name)
        if code:
            raise KernelError(f"TMA decode attention: a copy did not arrive within the poll limit (code {code})")


def try_paged_attention(q: torch.Tensor, cache: Any, ctx: Any, table: torch.Tensor, *, scale: float, window: int):
    """Return the attention output, or ``None`` when no tensor-core kernel takes
    this head size (the caller then uses the CUDA-core kernel)."""

    n, nq, d = q.shape
    if not supported(d):
        return None
    _, _, _, nkv, _, gs, slices = _geometry(q, cache.keys)
    if ctx.all_decode and n == ctx.num_entries:
        return decode_attention(q, cache.keys, cache.values, kv_len=ctx.kv_len, block_table=table, scale=scale,
                                window=window, splits=decode_parts(ctx, n, nq, nkv, d, cache.keys.shape[2], window),
                                live=getattr(ctx, "live_parts", None))
    maps = ctx.__dict__.setdefault("_tile_maps", {})
    page_size = cache.keys.shape[2]
    if PREFILL_BACKEND == "tcgen05" and tc_supported(d, page_size, window) and ctx.max_q_len >= TC_MIN_PORTION:
        pair = 0 < TC_PAIR_MIN_PORTION <= ctx.max_q_len
        per_tile = (2 if pair else 1) * (128 // gs)
        key = ("tc", per_tile)
        if key not in maps:
            maps[key] = tile_map(ctx.q_lens, per_tile, q.device, ctx.kv_lens)
        return prefill_attention_tcgen05(q, cache.keys, cache.values, positions=ctx.positions, block_table=table,
                                         q_lens=ctx.q_lens, scale=scale, tiles=maps[key], pair=pair)
    per_tile = 64 // gs
    if per_tile not in maps:
        maps[per_tile] = tile_map(ctx.q_lens, per_tile, q.device, ctx.kv_lens)
    return prefill_attention(q, cache.keys, cache.values, positions=ctx.positions, block_table=table,
                             q_lens=ctx.q_lens, scale=scale, window=window, tiles=maps[per_tile])
