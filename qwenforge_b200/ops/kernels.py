"""Python entry of every CUDA kernel: argument checks, pointer passing, error codes.

Each function checks dtypes, shapes and contiguity on the host, then calls the exported C
function of its library with raw device pointers and the current stream. There is no other
implementation behind these names: tensors that are not on a CUDA device are refused, and a
missing or failing kernel library raises `KernelLibraryError`.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ..csrc import library

_P = ctypes.c_void_p
_I = ctypes.c_int
_LL = ctypes.c_longlong
_ULL = ctypes.c_ulonglong
_F = ctypes.c_float

ERR_TOKEN_RANGE = 1
ERR_NO_PAGE = 2
ERR_ROW_RANGE = 4
ERR_COPY_TIMEOUT = 8
ERR_BARRIER_TIMEOUT = 16
ERR_POSITION_RANGE = 32

_ERROR_TEXT = {
    ERR_TOKEN_RANGE: "a token id lies outside the embedding table",
    ERR_NO_PAGE: "a position was read or written whose cache page is not held by its sequence",
    ERR_ROW_RANGE: "a wanted row lies outside the step's tokens",
    ERR_COPY_TIMEOUT: "a bulk copy into shared memory did not complete within its wait limit",
    ERR_BARRIER_TIMEOUT: "the blocks of a persistent kernel did not all reach a barrier within its wait limit",
    ERR_POSITION_RANGE: "a token's position lies outside the learned position table",
}


class KernelError(RuntimeError):
    pass


def describe_error_word(word: int) -> str:
    return "; ".join(text for bit, text in _ERROR_TEXT.items() if word & bit) or f"unknown error word {word}"


def require_cuda(device, what: str = "this operation") -> None:
    """There is no CPU execution path: anything that is to compute must live on a CUDA device."""
    if torch.device(device).type != "cuda":
        raise KernelError(f"{what} is on {device}: this library computes on CUDA devices only "
                          "(there is no CPU execution path)")
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device is available; this library has no CPU execution path")


launches = 0  # kernels of this library launched by this process (the measurement reads it)

_sm_counts: dict = {}


def sm_count(device) -> int:
    """Streaming multiprocessors of `device` (asked once): what grids and split counts are sized by."""
    device = torch.device(device)
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index not in _sm_counts:
        _sm_counts[index] = int(torch.cuda.get_device_properties(index).multi_processor_count)
    return _sm_counts[index]


def _check(code: int, what: str) -> None:
    global launches
    launches += 1
    if code != 0:
        raise KernelError(f"{what}: CUDA error {code} at launch")


def _stream() -> _P:
    """The current stream's raw handle on the current device (the short way: this runs once per kernel launch)."""
    return _P(torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice()))


def _ptr(t: Optional[torch.Tensor]) -> _P:
    return _P(0) if t is None else _P(t.data_ptr())


def _dev(name: str, t: torch.Tensor, dtype=None, contiguous: bool = True) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} is on {t.device}: the kernels of this library run on CUDA devices only")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} has dtype {t.dtype}, expected {dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} is not contiguous")


def _is_bf16(dtype: torch.dtype) -> int:
    if dtype == torch.bfloat16:
        return 1
    if dtype == torch.float32:
        return 0
    raise KernelError(f"activation dtype {dtype} is not supported (bfloat16 or float32)")


class KvSiteArgs:
    """What the kernels need to address one schedule entry's keys and values (see `cache.KvSite`)."""
    __slots__ = ("storage", "table", "page_elems", "table_stride", "kv_heads", "head_dim")

    def __init__(self, storage: torch.Tensor, table: torch.Tensor, kv_heads: int, head_dim: int):
        # storage: [pages, 2, kv_heads, PAGE, head_dim]; table: [slots, max_pages] int32
        self.storage = storage
        self.table = table
        self.page_elems = storage.stride(0)
        self.table_stride = table.stride(0)
        self.kv_heads = kv_heads
        self.head_dim = head_dim


def embed_gather(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, err: torch.Tensor) -> None:
    """out[t] = float32(table[ids[t]]); ids int32 [T], table [V, W], out float32 [T, W]."""
    _dev("ids", ids, torch.int32)
    _dev("table", table)
    _dev("out", out, torch.float32)
    n, (vocab, width) = ids.numel(), table.shape
    if out.shape != (n, width):
        raise KernelError(f"embed_gather: out is {tuple(out.shape)}, expected {(n, width)}")
    _check(library("embed").qf_embed_gather(_I(_is_bf16(table.dtype)), _ptr(ids), _ptr(table), _ptr(out), _I(n),
                                            _I(vocab), _I(width), _ptr(err), _stream()), "embed_gather")


def gather_rows(hidden: torch.Tensor, delta: Optional[torch.Tensor], rows: torch.Tensor, out: torch.Tensor,
                err: torch.Tensor) -> None:
    """out[r] = hidden[rows[r]] + delta[rows[r]] in float32; delta may be None."""
    _dev("hidden", hidden, torch.float32)
    _dev("rows", rows, torch.int32)
    _dev("out", out, torch.float32)
    n_in, width = hidden.shape
    is_bf16 = 0
    if delta is not None:
        _dev("delta", delta)
        is_bf16 = _is_bf16(delta.dtype)
        if delta.shape != hidden.shape:
            raise KernelError("gather_rows: delta and hidden differ in shape")
    if out.shape != (rows.numel(), width):
        raise KernelError("gather_rows: out has the wrong shape")
    _check(library("embed").qf_gather_rows(_I(is_bf16), _ptr(hidden), _ptr(delta), _ptr(rows), _ptr(out),
                                           _I(rows.numel()), _I(n_in), _I(width), _ptr(err), _stream()), "gather_rows")


def gather_rows_norm(hidden: torch.Tensor, delta: Optional[torch.Tensor], rows: torch.Tensor, weight: torch.Tensor,
                     eps: float, out: torch.Tensor, err: torch.Tensor) -> None:
    """out[r] = rmsnorm(hidden[rows[r]] + delta[rows[r]]) * weight, the sums in float32; delta may be None. hidden float32
    [T, W]; delta, weight and out share a dtype."""
    _dev("hidden", hidden, torch.float32)
    _dev("rows", rows, torch.int32)
    _dev("weight", weight)
    _dev("out", out, weight.dtype)
    n_in, width = hidden.shape
    if delta is not None:
        _dev("delta", delta, weight.dtype)
        if delta.shape != hidden.shape:
            raise KernelError("gather_rows_norm: delta and hidden differ in shape")
    if out.shape != (rows.numel(), width) or weight.numel() != width:
        raise KernelError("gather_rows_norm: out must be [rows, width], weight [width]")
    _check(library("embed").qf_gather_rows_norm(_I(_is_bf16(weight.dtype)), _ptr(hidden), _ptr(delta), _ptr(rows),
                                                _ptr(weight), _ptr(out), _I(rows.numel()), _I(n_in), _I(width), _F(eps),
                                                _ptr(err), _stream()), "gather_rows_norm")


def add_rms_norm(hidden: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                 out: torch.Tensor) -> None:
    """hidden += delta (if given); out = rmsnorm(hidden) * weight. hidden float32 [R, W]; out, weight, delta share a dtype."""
    _dev("hidden", hidden, torch.float32)
    _dev("weight", weight)
    _dev("out", out, weight.dtype)
    rows, width = hidden.shape
    if weight.shape != (width,) or out.shape != hidden.shape:
        raise KernelError("add_rms_norm: shapes of weight/out do not match hidden")
    if delta is not None:
        _dev("delta", delta, weight.dtype)
        if delta.shape != hidden.shape:
            raise KernelError("add_rms_norm: delta and hidden differ in shape")
    _check(library("norm").qf_add_rms_norm(_I(_is_bf16(weight.dtype)), _ptr(hidden), _ptr(delta), _ptr(weight),
                                           _ptr(out), _I(rows), _I(width), _F(eps), _stream()), "add_rms_norm")


def gemm_f32(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """out = x @ weight.T (+ bias) in true float32 (FFMA; no TF32). x [M, K], weight [N, K], out [M, N]; rows may be strided."""
    for name, t in (("x", x), ("weight", weight), ("out", out)):
        _dev(name, t, torch.float32, contiguous=False)
        if t.dim() != 2 or t.stride(1) != 1:
            raise KernelError(f"gemm_f32: {name} must be 2-d with unit inner stride")
    (m, k), (n, k2) = x.shape, weight.shape
    if k != k2 or out.shape != (m, n):
        raise KernelError(f"gemm_f32: shapes {tuple(x.shape)} x {tuple(weight.shape)}^T -> {tuple(out.shape)} do not agree")
    if bias is not None:
        _dev("bias", bias, torch.float32)
        if bias.shape != (n,):
            raise KernelError("gemm_f32: bias has the wrong shape")
    _check(library("gemm_f32").qf_gemm_f32(_ptr(x), _ptr(weight), _ptr(bias), _ptr(out), _I(m), _I(n), _I(k),
                                           _I(x.stride(0)), _I(weight.stride(0)), _I(out.stride(0)), _stream()),
           "gemm_f32")


def rope_cache_write(qkv: torch.Tensor, tok_seq: torch.Tensor, tok_pos: torch.Tensor, slots: torch.Tensor,
                     inv_freq: Optional[torch.Tensor], rot_dim: int, n_heads: int, q_out: torch.Tensor,
                     site: KvSiteArgs, write_cache: bool, err: torch.Tensor, bias: Optional[torch.Tensor] = None,
                     unit_norm_eps: Optional[float] = None, norm_dim: int = 0, has_kv: bool = True,
                     interleaved: bool = False, norm_first: bool = False, q_norm: Optional[torch.Tensor] = None,
                     k_norm: Optional[torch.Tensor] = None) -> None:
    """Rotate q and k heads of qkv [T, (NH + 2 KVH) D] by position, write q to q_out [T, NH D] and k, v into the cache.
    The rows of qkv may be the first columns of wider rows (unit inner stride).
    `unit_norm_eps`: after the rotation every q and k head is divided by its root mean square (float32), the mean taken
    over the head's first `norm_dim` components (0: all; a head padded with zeros beyond its own size names that size).
    `norm_first`: that division comes before the rotation instead, and `q_norm` / `k_norm` ([norm_dim], shared by the
    heads) then multiply the components. `interleaved`: the rotation pairs component 2j with 2j + 1 instead of j with
    j + rot_dim / 2.
    `has_kv` false: the rows hold queries only, [T, NH D] (a layer that reads another layer's keys and values)."""
    _rows("qkv", qkv)
    _dev("q_out", q_out, qkv.dtype)
    _dev("cache", site.storage, qkv.dtype)
    _dev("tok_seq", tok_seq, torch.int32)
    _dev("tok_pos", tok_pos, torch.int32)
    _dev("slots", slots, torch.int32)
    n = qkv.shape[0]
    d, kvh = site.head_dim, site.kv_heads
    if qkv.shape[1] < (n_heads + (2 * kvh if has_kv else 0)) * d or q_out.shape != (n, n_heads * d):
        raise KernelError("rope_cache_write: qkv/q_out widths do not match the head counts")
    if not has_kv and write_cache:
        raise KernelError("rope_cache_write: rows without keys and values cannot write a cache")
    if bias is not None:
        _dev("bias", bias, qkv.dtype)
        if bias.numel() != (n_heads + (2 * kvh if has_kv else 0)) * d:
            raise KernelError("rope_cache_write: bias must have one element per projection column")
    if inv_freq is not None:
        _dev("inv_freq", inv_freq, torch.float32)
        if inv_freq.numel() * 2 != rot_dim:
            raise KernelError("rope_cache_write: inv_freq must hold rot_dim / 2 frequencies")
    if unit_norm_eps is not None or not has_kv or interleaved:
        if not 0 <= norm_dim <= d:
            raise KernelError("rope_cache_write: norm_dim must lie within the head size")
        for name, w in (("q_norm", q_norm), ("k_norm", k_norm)):
            if w is not None:
                _dev(name, w, qkv.dtype)
                if not norm_first or unit_norm_eps is None or w.numel() != (norm_dim or d):
                    raise KernelError(f"rope_cache_write: {name} goes with a norm before the rotation and holds norm_dim weights")
        _check(library("rope_cache").qf_rope_norm_cache_write_ex(
            _I(_is_bf16(qkv.dtype)), _ptr(qkv), _ptr(bias), _I(qkv.stride(0)), _ptr(tok_seq), _ptr(tok_pos), _ptr(slots),
            _ptr(inv_freq), _I(rot_dim), _I(n_heads), _ptr(q_out), _ptr(site.storage), _ptr(site.table),
            _LL(site.page_elems), _I(site.table_stride), _I(kvh), _I(d), _I(1 if write_cache else 0), _I(1 if has_kv else 0),
            _I(norm_dim or d), _F(-1.0 if unit_norm_eps is None else unit_norm_eps), _I(n), _ptr(err), _I(int(interleaved)),
            _I(int(norm_first)), _ptr(q_norm), _ptr(k_norm), _stream()),
            "rope_cache_write")
        return
    if norm_first or q_norm is not None or k_norm is not None:
        raise KernelError("rope_cache_write: a norm before the rotation needs its eps (unit_norm_eps)")
    _check(library("rope_cache").qf_rope_cache_write(
        _I(_is_bf16(qkv.dtype)), _ptr(qkv), _ptr(bias), _I(qkv.stride(0)), _ptr(tok_seq), _ptr(tok_pos), _ptr(slots),
        _ptr(inv_freq), _I(rot_dim), _I(n_heads), _ptr(q_out), _ptr(site.storage), _ptr(site.table),
        _LL(site.page_elems), _I(site.table_stride), _I(kvh), _I(d), _I(1 if write_cache else 0), _I(n), _ptr(err),
        _stream()), "rope_cache_write")


GENERIC_DECODE_CHUNK = 256
GENERIC_MAX_HEAD_DIM = 512


def attention_generic(q: torch.Tensor, out: torch.Tensor, cu_q: torch.Tensor, tok_pos: torch.Tensor,
                      slots: torch.Tensor, site: KvSiteArgs, n_heads: int, n_seqs: int, max_q_len: int, scale: float,
                      window: int, err: torch.Tensor, scratch: Optional["DecodeScratch"] = None,
                      max_kv_len: Optional[int] = None, sinks: Optional[torch.Tensor] = None,
                      shared_values: bool = False, chunk: int = 0, softcap: float = 0.0,
                      blocks: Optional[KvSiteArgs] = None, pool: int = 0) -> None:
    """Causal grouped-query attention of the step's queries over each sequence's cache (any sizes, SIMT float32 math).
    `pool` > 0 with `blocks` (a second cache of the same head shape that holds one row per block of `pool` positions) and a
    window: a query also sees the row of every block that lies wholly before its window, in the same softmax.
    `chunk` > 0: a query sees only the keys of its own block of `chunk` positions (blocks counted from position 0 of the
    sequence). `softcap` > 0: a score s (after the scale) becomes softcap * tanh(s / softcap).
    `sinks` (float32 [n_heads]): a logit per head that joins the softmax's denominator once, with no key and no value.
    `shared_values`: the values are the keys themselves (a cache whose pages hold one plane).
    A step of one token per sequence whose longest sequence exceeds one chunk of 256 keys is cut into chunks of keys
    when `scratch` and `max_kv_len` (a bound on any sequence's length after the step) are given: a block per chunk,
    then a fold in rising order; which chunks a row has depends on its own position only."""
    _dev("q", q)
    _dev("out", out, q.dtype)
    _dev("cache", site.storage, q.dtype)
    d = site.head_dim
    if d > GENERIC_MAX_HEAD_DIM:
        raise KernelError(f"attention_generic: head_dim {d} > {GENERIC_MAX_HEAD_DIM} is not supported")
    if q.shape[1] != n_heads * d or out.shape != q.shape:
        raise KernelError("attention_generic: q/out widths do not match the head count")
    if sinks is not None:
        _dev("sinks", sinks, torch.float32)
        if sinks.numel() != n_heads:
            raise KernelError("attention_generic: sinks must hold one float32 per query head")
    if pool > 0:
        if blocks is None or window <= 0 or shared_values or (blocks.kv_heads, blocks.head_dim) != (site.kv_heads, d):
            raise KernelError("attention_generic: rows of whole blocks need a window and a second cache of the same head shape")
        _dev("block rows", blocks.storage, q.dtype)
    elif (scratch is not None and max_kv_len is not None and max_q_len == 1 and q.shape[0] == n_seqs
            and max_kv_len > GENERIC_DECODE_CHUNK):
        n_chunks = -(-int(max_kv_len) // GENERIC_DECODE_CHUNK)
        scratch.ensure(n_seqs, n_heads, n_chunks, d, 0)
        _check(library("attention_generic").qf_attention_generic_decode_masked(
            _I(_is_bf16(q.dtype)), _ptr(q), _ptr(out), _ptr(cu_q), _ptr(tok_pos), _ptr(slots), _ptr(site.storage),
            _ptr(site.table), _LL(site.page_elems), _I(site.table_stride), _I(site.kv_heads), _I(d), _I(n_heads),
            _I(n_seqs), _I(int(max_kv_len)), _F(scale), _I(window), _ptr(scratch.part_o), _ptr(scratch.part_ml), _ptr(err),
            _ptr(sinks), _I(int(bool(shared_values))), _I(int(chunk)), _F(softcap), _stream()), "attention_generic")
        return
    _check(library("attention_generic").qf_attention_generic_pooled(
        _I(_is_bf16(q.dtype)), _ptr(q), _ptr(out), _ptr(cu_q), _ptr(tok_pos), _ptr(slots), _ptr(site.storage),
        _ptr(site.table), _LL(site.page_elems), _I(site.table_stride), _I(site.kv_heads), _I(d), _I(n_heads),
        _I(n_seqs), _I(max_q_len), _F(scale), _I(window), _ptr(err), _ptr(sinks), _I(int(bool(shared_values))),
        _I(int(chunk)), _F(softcap), _ptr(blocks.storage if pool > 0 else None), _ptr(blocks.table if pool > 0 else None),
        _LL(blocks.page_elems if pool > 0 else 0), _I(blocks.table_stride if pool > 0 else 0), _I(int(pool)), _stream()),
        "attention_generic")


FAST_ATTENTION_HEAD_DIMS = (32, 64, 96, 128)


def attention_prefill(q: torch.Tensor, out: torch.Tensor, cu_q: torch.Tensor, tok_pos: torch.Tensor,
                      slots: torch.Tensor, site: KvSiteArgs, n_heads: int, n_seqs: int, max_q_len: int, scale: float,
                      window: int, err: torch.Tensor, max_kv_len: Optional[int] = None,
                      sinks: Optional[torch.Tensor] = None, shared_values: bool = False, chunk: int = 0,
                      softcap: float = 0.0, blocks: Optional[KvSiteArgs] = None, pool: int = 0) -> None:
    """Tensor-core flash attention of spans of new tokens over the cache: bfloat16, head sizes 32/64/96/128.
    `sinks`, `shared_values`, `chunk`, `softcap`, `blocks` and `pool`: as in `attention_generic` (the cap with the hardware's
    approximate tanh).
    `max_kv_len`: an upper bound of any sequence's length after the step (None: unknown, taken as long); it only
    steers whether a tile of rows shares its pages among two groups of warps."""
    _dev("q", q, torch.bfloat16)
    _dev("out", out, torch.bfloat16)
    _dev("cache", site.storage, torch.bfloat16)
    d = site.head_dim
    if d not in FAST_ATTENTION_HEAD_DIMS:
        raise KernelError(f"attention_prefill: head_dim {d} has no tensor-core kernel (have {FAST_ATTENTION_HEAD_DIMS}); "
                          "use attention_generic")
    if q.shape[1] != n_heads * d or out.shape != q.shape:
        raise KernelError("attention_prefill: q/out widths do not match the head count")
    if sinks is not None:
        _dev("sinks", sinks, torch.float32)
        if sinks.numel() != n_heads:
            raise KernelError("attention_prefill: sinks must hold one float32 per query head")
    if pool > 0:
        if blocks is None or window <= 0 or shared_values or (blocks.kv_heads, blocks.head_dim) != (site.kv_heads, d):
            raise KernelError("attention_prefill: rows of whole blocks need a window and a second cache of the same head shape")
        _dev("block rows", blocks.storage, torch.bfloat16)
    _check(library("attention_prefill").qf_attention_prefill_pooled(
        _ptr(q), _ptr(out), _ptr(cu_q), _ptr(tok_pos), _ptr(slots), _ptr(site.storage), _ptr(site.table),
        _LL(site.page_elems), _I(site.table_stride), _I(site.kv_heads), _I(d), _I(n_heads), _I(n_seqs), _I(q.shape[0]),
        _I(max_q_len), _I(1 << 30 if max_kv_len is None else int(max_kv_len)), _F(scale), _I(window), _ptr(err),
        _ptr(sinks), _I(int(bool(shared_values))), _I(int(chunk)), _F(softcap), _ptr(blocks.storage if pool > 0 else None),
        _ptr(blocks.table if pool > 0 else None), _LL(blocks.page_elems if pool > 0 else 0),
        _I(blocks.table_stride if pool > 0 else 0), _I(int(pool)), _stream()), "attention_prefill")


TC_ATTENTION_HEAD_DIMS = (64, 128)


def attention_prefill_tc(q: torch.Tensor, out: torch.Tensor, cu_q: torch.Tensor, tok_pos: torch.Tensor,
                         slots: torch.Tensor, site: KvSiteArgs, n_heads: int, n_seqs: int, max_q_len: int, scale: float,
                         window: int, err: torch.Tensor, max_kv_len: Optional[int] = None,
                         sinks: Optional[torch.Tensor] = None, shared_values: bool = False) -> None:
    """The same attention on the fifth-generation tensor cores (tcgen05, accumulators in tensor memory): blocks of
    128 query rows; bfloat16, head sizes 64 and 128, cache pages without gaps. `max_kv_len` as in `attention_prefill`:
    with few tiles of many pages, two blocks of a cluster share a tile."""
    _dev("q", q, torch.bfloat16)
    _dev("out", out, torch.bfloat16)
    _dev("cache", site.storage, torch.bfloat16)
    d = site.head_dim
    if d not in TC_ATTENTION_HEAD_DIMS:
        raise KernelError(f"attention_prefill_tc: head_dim {d} has no tcgen05 kernel (have {TC_ATTENTION_HEAD_DIMS}); "
                          "use attention_prefill")
    if q.shape[1] != n_heads * d or out.shape != q.shape:
        raise KernelError("attention_prefill_tc: q/out widths do not match the head count")
    if site.page_elems != (1 if shared_values else 2) * site.kv_heads * site.storage.shape[-2] * d:
        raise KernelError("attention_prefill_tc: the cache pages have gaps; use attention_prefill")
    if sinks is not None:
        _dev("sinks", sinks, torch.float32)
        if sinks.numel() != n_heads:
            raise KernelError("attention_prefill_tc: sinks must hold one float32 per query head")
    _check(library("attention_prefill_tc").qf_attention_prefill_tc_ex(
        _ptr(q), _ptr(out), _ptr(cu_q), _ptr(tok_pos), _ptr(slots), _ptr(site.storage), _ptr(site.table),
        _LL(site.page_elems), _I(site.table_stride), _I(site.kv_heads), _I(d), _I(n_heads), _I(n_seqs), _I(q.shape[0]),
        _I(max_q_len), _I(1 << 30 if max_kv_len is None else int(max_kv_len)), _F(scale), _I(window), _ptr(err),
        _ptr(sinks), _I(int(bool(shared_values))), _stream()), "attention_prefill_tc")


class DecodeScratch:
    """Scratch of the split-K decode attention: float32 partial numerators and (max, sum) pairs per
    (sequence, head, split), and the ticket counters (kept zero between calls by the kernel itself).
    One instance is shared by all layers of a model: they run one after another on one stream."""

    def __init__(self, device):
        self.device = device
        self.part_o = self.part_ml = self.counters = None
        self.plans: dict = {}   # attention shape -> int32 [records, 4]: which block takes which run of which sequence

    def plan(self, key: tuple, records: int) -> torch.Tensor:
        held = self.plans.get(key)
        if held is None or held.shape[0] < records:
            held = self.plans[key] = torch.empty((records, 4), dtype=torch.int32, device=self.device)
        return held

    def ensure(self, n_seqs: int, n_heads: int, n_splits: int, head_dim: int, n_counters: int) -> None:
        rows = n_seqs * n_heads * n_splits
        if self.part_o is None or self.part_o.numel() < rows * head_dim:
            self.part_o = torch.empty(rows * head_dim, dtype=torch.float32, device=self.device)
        if self.part_ml is None or self.part_ml.numel() < rows * 2:
            self.part_ml = torch.empty(rows * 2, dtype=torch.float32, device=self.device)
        if n_counters and (self.counters is None or self.counters.numel() < n_counters):
            self.counters = torch.zeros(n_counters, dtype=torch.int32, device=self.device)


def attention_decode_warps(head_dim: int) -> int:
    """Warps of a block of the decode attention at this head size (each takes one page at a time): the fewest pages
    that a run of a sequence should hold."""
    return int(library("attention_decode").qf_attention_decode_warps(_I(head_dim)))


def attention_decode_plan(cu_q: torch.Tensor, tok_pos: torch.Tensor, slots: torch.Tensor, kv_heads: int, head_dim: int,
                          n_heads: int, n_seqs: int, window: int, n_splits: int, scratch: DecodeScratch,
                          chunk: int = 0) -> torch.Tensor:
    """The plan of one decode step for attention of this shape: which block takes which run of which sequence, worked
    out on the device from the batch's lengths (sequences of unequal lengths get blocks of about equal work; a batch
    that fills the SMs unsplit stays unsplit). One plan serves every layer of the step with this shape. `n_splits` is
    the most runs one sequence may get. The tensor belongs to `scratch` and is overwritten by the next plan of the
    same shape."""
    for name, t in (("cu_q", cu_q), ("tok_pos", tok_pos), ("slots", slots)):
        _dev(name, t, torch.int32)
    if not 1 <= n_splits <= 128:
        raise KernelError(f"attention_decode: n_splits {n_splits} outside 1..128")
    if kv_heads <= 0 or n_heads % kv_heads:
        raise KernelError(f"attention_decode: {n_heads} heads do not divide into {kv_heads} groups")
    lib = library("attention_decode")
    lib.qf_attention_decode_plan_size.restype = ctypes.c_longlong
    records = int(lib.qf_attention_decode_plan_size(_I(n_seqs), _I(kv_heads), _I(n_heads), _I(head_dim), _I(n_splits)))
    if records <= 0:
        raise KernelError(f"attention_decode: head_dim {head_dim} has no tensor-core kernel (have {FAST_ATTENTION_HEAD_DIMS})")
    plan = scratch.plan((n_seqs, kv_heads, n_heads, head_dim, window, n_splits, chunk), records)
    _check(lib.qf_attention_decode_plan_masked(_ptr(cu_q), _ptr(tok_pos), _ptr(slots), _I(n_seqs), _I(kv_heads), _I(head_dim),
                                               _I(n_heads), _I(window), _I(n_splits), _ptr(plan), _I(int(chunk)), _stream()),
           "attention_decode_plan")
    return plan


def attention_decode(q: torch.Tensor, out: torch.Tensor, cu_q: torch.Tensor, tok_pos: torch.Tensor,
                     slots: torch.Tensor, site: KvSiteArgs, n_heads: int, n_seqs: int, scale: float, window: int,
                     n_splits: int, scratch: DecodeScratch, err: torch.Tensor, plan: Optional[torch.Tensor] = None,
                     fold_later: bool = False, sinks: Optional[torch.Tensor] = None, shared_values: bool = False,
                     chunk: int = 0, softcap: float = 0.0) -> None:
    """Split-K flash decoding: ONE new token per sequence over its cache; bfloat16, head sizes 32/64/96/128.
    `n_splits` is the most blocks that share one (sequence, kv head); `plan` (attention_decode_plan with the same
    shape, made in this step; made here when absent) says how many of them each sequence gets. With `fold_later` the
    kernel stops at the runs' partial results in `scratch` and writes no `out` (which may be None): `fold_project`
    folds them on its way into the output projection. `sinks`, `shared_values`, `chunk`, `softcap`: as in
    `attention_generic` (sinks not with `fold_later`; a given `plan` must have been made with the same `chunk`; the cap
    with the hardware's approximate tanh)."""
    _dev("q", q, torch.bfloat16)
    if sinks is not None:
        _dev("sinks", sinks, torch.float32)
        if sinks.numel() != n_heads or fold_later:
            raise KernelError("attention_decode: sinks must hold one float32 per query head, and do not go with fold_later")
    if not fold_later:
        _dev("out", out, torch.bfloat16)
    _dev("cache", site.storage, torch.bfloat16)
    d = site.head_dim
    if d not in FAST_ATTENTION_HEAD_DIMS:
        raise KernelError(f"attention_decode: head_dim {d} has no tensor-core kernel (have {FAST_ATTENTION_HEAD_DIMS}); "
                          "use attention_generic")
    if q.shape != (n_seqs, n_heads * d) or (not fold_later and out.shape != q.shape):
        raise KernelError("attention_decode: wants exactly one token per sequence, q [n_seqs, n_heads * head_dim]")
    if not 1 <= n_splits <= 128:
        raise KernelError(f"attention_decode: n_splits {n_splits} outside 1..128")
    if plan is None:
        plan = attention_decode_plan(cu_q, tok_pos, slots, site.kv_heads, d, n_heads, n_seqs, window, n_splits, scratch, chunk)
    group = n_heads // site.kv_heads
    n_counters = n_seqs * site.kv_heads * ((group + 15) // 16)
    partials = n_splits > 1 or fold_later
    if partials:
        scratch.ensure(n_seqs, n_heads, n_splits, d, n_counters)
    _check(library("attention_decode").qf_attention_decode_masked(
        _ptr(q), _ptr(None if fold_later else out), _ptr(cu_q), _ptr(plan), _ptr(site.storage), _ptr(site.table),
        _LL(site.page_elems), _I(site.table_stride), _I(site.kv_heads), _I(d), _I(n_heads), _I(n_seqs), _F(scale),
        _I(window), _I(n_splits), _I(1 if fold_later else 0), _ptr(scratch.part_o if partials else None),
        _ptr(scratch.part_ml if partials else None), _ptr(scratch.counters if partials else None), _ptr(err),
        _ptr(sinks), _I(int(bool(shared_values))), _I(int(chunk)), _F(softcap), _stream()), "attention_decode")


class _FoldProjectArgs(ctypes.Structure):
    _fields_ = [("part_o", _P), ("part_ml", _P), ("runs", _P), ("w", _P), ("hidden", _P), ("rows", _I), ("n", _I),
                ("ldw", _I), ("n_heads", _I), ("head_dim", _I), ("max_splits", _I)]


def fold_project_takes(rows: int, weight: torch.Tensor, hidden: torch.Tensor, n_heads: int, head_dim: int) -> bool:
    """Whether `fold_project` takes the output projection `weight` [N, n_heads * head_dim] for a step of `rows` rows."""
    if weight.dtype != torch.bfloat16 or hidden.dtype != torch.float32 or weight.dim() != 2 or weight.stride(1) != 1:
        return False
    if weight.shape[1] != n_heads * head_dim or not hidden.is_contiguous() or hidden.shape != (rows, weight.shape[0]):
        return False
    return bool(library("fold_project").qf_fold_project_takes(
        _I(rows), _I(weight.shape[0]), _I(weight.stride(0)), _I(n_heads), _I(head_dim), _ptr(weight), _ptr(hidden)))


FOLD_PROJECT_MAX_REDUCTIONS = 150_000


def fold_project_pays(rows: int, weight: torch.Tensor) -> bool:
    """Whether `fold_project` is the faster way for this projection. What it saves is the attention kernel's life after
    its pages (about 3 microseconds); what it costs grows with the 16-byte reductions into the stream, rows x N / 4 from
    each of its K / 32 blocks. Measured: 50,000 of them (8 rows, 896 x 896) gain 2.2 microseconds per layer, 524,000 (16
    rows, 2048 x 2048) lose 1."""
    return rows * weight.shape[0] * (weight.shape[1] // 32) // 4 <= FOLD_PROJECT_MAX_REDUCTIONS


def fold_project(plan: torch.Tensor, scratch: DecodeScratch, weight: torch.Tensor, hidden: torch.Tensor, n_heads: int,
                 head_dim: int, n_splits: int) -> None:
    """hidden[r, :] += fold(the partial results of sequence r) @ weight^T, after `attention_decode(..., fold_later=True)`
    with the same `plan`, `scratch` and `n_splits` in a step whose row r is sequence r (one token per sequence).
    bfloat16 weight [N, n_heads * head_dim], float32 hidden [rows, N]; the blocks' shares are added with atomic
    reductions, in no fixed order."""
    _dev("weight", weight, torch.bfloat16, contiguous=False)
    _dev("hidden", hidden, torch.float32)
    rows = hidden.shape[0]
    if not fold_project_takes(rows, weight, hidden, n_heads, head_dim):
        raise KernelError(f"fold_project: does not take {rows} rows, weight {tuple(weight.shape)}, {n_heads} heads of {head_dim}")
    if scratch.part_o is None or scratch.part_o.numel() < rows * n_heads * n_splits * head_dim:
        raise KernelError("fold_project: the scratch does not hold this step's partial results")
    a = _FoldProjectArgs(scratch.part_o.data_ptr(), scratch.part_ml.data_ptr(), plan.data_ptr(), weight.data_ptr(),
                         hidden.data_ptr(), rows, weight.shape[0], weight.stride(0), n_heads, head_dim, n_splits)
    _check(library("fold_project").qf_fold_project(ctypes.byref(a), _stream()), "fold_project")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i]."""
    _dev("gate_up", gate_up)
    _dev("out", out, gate_up.dtype)
    rows, two_i = gate_up.shape
    if two_i % 2 or out.shape != (rows, two_i // 2):
        raise KernelError("swiglu: out must be [rows, width / 2]")
    _check(library("activation").qf_swiglu(_I(_is_bf16(gate_up.dtype)), _ptr(gate_up), _ptr(out), _I(rows),
                                           _I(two_i // 2), _stream()), "swiglu")


class SampleScratch:
    """Scratch of the sampling kernel when several blocks share a row: each block's best (score, id) and the
    rows' ticket counters (kept zero between calls by the kernel itself)."""

    def __init__(self):
        self.part_v = self.part_i = self.counters = None

    def ensure(self, rows: int, chunks: int, device) -> None:
        if self.part_v is None or self.part_v.numel() < rows * chunks or self.part_v.device != device:
            self.part_v = torch.empty(rows * chunks, dtype=torch.float32, device=device)
            self.part_i = torch.empty(rows * chunks, dtype=torch.int32, device=device)
        if self.counters is None or self.counters.numel() < rows or self.counters.device != device:
            self.counters = torch.zeros(rows, dtype=torch.int32, device=device)


_sample_scratch = SampleScratch()


def sample(logits: torch.Tensor, temperature: float, seed: int, seq_ids: Optional[torch.Tensor],
           steps: Optional[torch.Tensor], out: torch.Tensor, scratch: Optional[SampleScratch] = None) -> None:
    """out[r] = argmax (temperature <= 0) or a Gumbel-max draw keyed by (seed, seq_ids[r], steps[r]).
    `scratch`: whoever captures the call into a CUDA graph passes a scratch of its own, which then lives as long
    as the graph; other callers share one that grows as needed."""
    _dev("logits", logits, torch.float32, contiguous=False)
    _dev("out", out, torch.int32)
    if logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be 2-d with unit inner stride")
    rows, vocab = logits.shape
    if out.numel() != rows:
        raise KernelError("sample: out must have one element per row")
    if temperature > 0:
        if seq_ids is None or steps is None:
            raise KernelError("sample: sampling needs seq_ids and steps")
        _dev("seq_ids", seq_ids, torch.int64)
        _dev("steps", steps, torch.int32)
        if seq_ids.numel() != rows or steps.numel() != rows:
            raise KernelError("sample: seq_ids and steps must have one element per row")
    # enough blocks to fill the GPU (eight per SM) when there are few rows, at least 2048 tokens of the vocabulary each
    chunks = max(1, min(-(-vocab // 2048), -(-8 * sm_count(logits.device) // rows), 64))
    scratch = scratch or _sample_scratch
    if chunks > 1:
        scratch.ensure(rows, chunks, logits.device)
    _check(library("sampling").qf_sample(_ptr(logits), _I(rows), _I(vocab), _LL(logits.stride(0)),
                                         _F(max(float(temperature), 0.0)), _ULL(seed & 0xFFFFFFFFFFFFFFFF),
                                         _ptr(seq_ids), _ptr(steps), _ptr(out), _I(chunks),
                                         _ptr(scratch.part_v if chunks > 1 else None),
                                         _ptr(scratch.part_i if chunks > 1 else None),
                                         _ptr(scratch.counters if chunks > 1 else None), _stream()), "sample")


def decode_advance(sampled: torch.Tensor, token_ids: torch.Tensor, tok_pos: torch.Tensor, slots: torch.Tensor,
                   steps: torch.Tensor, budgets: torch.Tensor, stop_ids: torch.Tensor, n_stop: int,
                   out_tokens: torch.Tensor, cursor: torch.Tensor) -> None:
    """Record each live row's sampled token in out_tokens[cursor], feed it back as the next input, advance
    position and step count, retire rows that stopped (slot := -1); cursor += 1. All int32, on the device."""
    for name, t in (("sampled", sampled), ("token_ids", token_ids), ("tok_pos", tok_pos), ("slots", slots),
                    ("steps", steps), ("budgets", budgets), ("stop_ids", stop_ids), ("out_tokens", out_tokens),
                    ("cursor", cursor)):
        _dev(name, t, torch.int32)
    n = token_ids.numel()
    if out_tokens.dim() != 2 or out_tokens.shape[1] != n or n_stop > stop_ids.numel():
        raise KernelError("decode_advance: out_tokens must be [max_steps, rows]; n_stop within stop_ids")
    _check(library("decode_state").qf_decode_advance(
        _ptr(sampled), _ptr(token_ids), _ptr(tok_pos), _ptr(slots), _ptr(steps), _ptr(budgets), _ptr(stop_ids),
        _I(n_stop), _ptr(out_tokens), _ptr(cursor), _I(out_tokens.shape[0]), _I(n), _stream()), "decode_advance")


def decode_advance_embed(sampled: torch.Tensor, token_ids: torch.Tensor, tok_pos: torch.Tensor, slots: torch.Tensor,
                         steps: torch.Tensor, budgets: torch.Tensor, stop_ids: torch.Tensor, n_stop: int,
                         out_tokens: torch.Tensor, cursor: torch.Tensor, table: torch.Tensor, hidden: torch.Tensor,
                         ticket: torch.Tensor, err: torch.Tensor) -> None:
    """`decode_advance`, and the next step's embedding with it: hidden[r] = float32(table[the row's next input token]).
    `ticket` is one int32 that is zero before the first call."""
    for name, t in (("sampled", sampled), ("token_ids", token_ids), ("tok_pos", tok_pos), ("slots", slots),
                    ("steps", steps), ("budgets", budgets), ("stop_ids", stop_ids), ("out_tokens", out_tokens),
                    ("cursor", cursor), ("ticket", ticket)):
        _dev(name, t, torch.int32)
    _dev("table", table)
    _dev("hidden", hidden, torch.float32)
    n = token_ids.numel()
    if out_tokens.dim() != 2 or out_tokens.shape[1] != n or n_stop > stop_ids.numel():
        raise KernelError("decode_advance_embed: out_tokens must be [max_steps, rows]; n_stop within stop_ids")
    if table.dim() != 2 or hidden.shape != (n, table.shape[1]):
        raise KernelError("decode_advance_embed: hidden must be [rows, width of the table]")
    _check(library("decode_state").qf_decode_advance_embed(
        _ptr(sampled), _ptr(token_ids), _ptr(tok_pos), _ptr(slots), _ptr(steps), _ptr(budgets), _ptr(stop_ids),
        _I(n_stop), _ptr(out_tokens), _ptr(cursor), _I(out_tokens.shape[0]), _I(n), _I(_is_bf16(table.dtype)),
        _ptr(table), _I(table.shape[0]), _I(table.shape[1]), _ptr(hidden), _ptr(ticket), _ptr(err), _stream()),
        "decode_advance_embed")


# ---------------------------------------------------------------------------------------------- fused skinny products

SKINNY_MAX_ROWS = 16
EPI_PLAIN, EPI_RESIDUAL, EPI_SWIGLU, EPI_QKV = 0, 1, 2, 3


class _SkinnyArgs(ctypes.Structure):
    _fields_ = [
        ("w", _P), ("bias", _P), ("n", _I), ("k", _I), ("ldw", _I), ("m", _I),
        ("x", _P), ("ldx", _I), ("hidden", _P), ("norm_w", _P), ("eps", _F),
        ("out", _P), ("ldo", _I), ("out_f32", _I), ("residual", _P), ("inter", _I),
        ("n_heads", _I), ("kv_heads", _I), ("head_dim", _I), ("rot_dim", _I), ("write_cache", _I),
        ("inv_freq", _P), ("tok_pos", _P), ("tok_seq", _P), ("slots", _P), ("q_out", _P), ("kv_base", _P),
        ("table", _P), ("page_elems", _LL), ("table_stride", _I), ("err", _P), ("gate_limit", _F), ("gate_alpha", _F),
    ]


_own_err_words = {}


def _err_word_for(device) -> torch.Tensor:
    """A device error word for calls that bring none of their own (kernel tests)."""
    key = str(device)
    if key not in _own_err_words:
        _own_err_words[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _own_err_words[key]


_skinny_answers: dict = {}


def skinny_gemm_takes(m: int, weight: torch.Tensor, epilogue: int = EPI_PLAIN, norm: bool = False, *,
                      ldx: Optional[int] = None, n_heads: int = 0, kv_heads: int = 0, head_dim: int = 0,
                      rot_dim: int = 0) -> bool:
    """Whether `skinny_gemm` runs `m` token rows against `weight` [N, K] with this epilogue and prologue. The answer
    is the library's own (`qf_skinny_gemm_takes` runs the planning of the launch without launching), so a shape
    that gets a yes here is never refused later. `ldx`: elements between input rows (default K); `rot_dim`: > 0 when
    the QKV epilogue is to rotate that many components of each head."""
    if not (weight.is_cuda and weight.dtype == torch.bfloat16 and weight.dim() == 2 and weight.stride(1) == 1):
        return False
    n, k = weight.shape
    key = (weight.device.index, int(m), n, k, weight.stride(0), epilogue, bool(norm), k if ldx is None else ldx,
           n_heads, kv_heads, head_dim, rot_dim)
    answer = _skinny_answers.get(key)
    if answer is None:
        with torch.cuda.device(weight.device):
            answer = library("skinny_gemm").qf_skinny_gemm_takes(
                _I(epilogue), _I(int(bool(norm))), _I(int(m)), _I(n), _I(k), _I(weight.stride(0)), _I(key[7]),
                _I(n // 2 if epilogue == EPI_SWIGLU else 0), _I(n_heads), _I(kv_heads), _I(head_dim),
                _I(1 if rot_dim > 0 else 0), _I(rot_dim)) != 0
        _skinny_answers[key] = answer
    return answer


def skinny_gemm_pays(m: int, weight: torch.Tensor) -> bool:
    """Whether the weight-streaming kernel is the faster way to run `m` token rows against `weight`, by measurement on
    a B200 (`python -m qwenforge_b200.measure products`): for weights of 100 MB and more it loses to the norm kernel,
    the library product and the elementwise kernel together (Qwen2.5-7B's feed-forward, 272 and 136 MB: 57 and 41
    microseconds against 52 and 30 at 8 rows, 62 and 51 against 52 and 31 at 16), and from 9 rows on already for
    weights above 64 MB (Qwen2.5-3B's gate/up, 90 MB: 24.4 against 22.3). Everything smaller it wins, the smaller the
    clearer (0.5B at 8 rows: 2.9 / 5.9 / 4.8 / 4.4 microseconds against 5.1 / 8.6 / 11.0 / 8.3)."""
    size = weight.numel() * weight.element_size()
    return size < 100e6 and (m <= 8 or size < 64e6)


def _skinny_args(epilogue: int, weight: torch.Tensor, *, x: Optional[torch.Tensor] = None,
                 hidden: Optional[torch.Tensor] = None, norm_weight: Optional[torch.Tensor] = None, eps: float = 0.0,
                 bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                 residual: Optional[torch.Tensor] = None, qkv: Optional[dict] = None,
                 err: Optional[torch.Tensor] = None, clamp=None):
    """Checks one fused product's tensors and fills the kernels' argument block; returns (block, norm flag).
    clamp = (limit, alpha) with EPI_SWIGLU: the clamped gate in the silu gate's place (see `clamped_glu`)."""
    _dev("weight", weight, torch.bfloat16, contiguous=False)
    a = _SkinnyArgs()
    a.w, a.n, a.k, a.ldw = weight.data_ptr(), weight.shape[0], weight.shape[1], weight.stride(0)
    if bias is not None:
        _dev("bias", bias, torch.bfloat16)
        a.bias = bias.data_ptr()
    norm = hidden is not None
    if norm:
        _dev("hidden", hidden, torch.float32)
        _dev("norm_weight", norm_weight, torch.bfloat16)
        if hidden.shape[1] != a.k or norm_weight.numel() != a.k:
            raise KernelError("skinny_gemm: hidden/norm_weight widths do not match the weight's K")
        a.hidden, a.norm_w, a.eps, a.m = hidden.data_ptr(), norm_weight.data_ptr(), eps, hidden.shape[0]
    else:
        _dev("x", x, torch.bfloat16, contiguous=False)
        if x.shape[1] != a.k or x.stride(1) != 1:
            raise KernelError("skinny_gemm: x width does not match the weight's K")
        a.x, a.ldx, a.m = x.data_ptr(), x.stride(0), x.shape[0]
    if epilogue == EPI_PLAIN:
        _dev("out", out, None, contiguous=False)
        if out.shape != (a.m, a.n) or out.dtype not in (torch.bfloat16, torch.float32):
            raise KernelError("skinny_gemm: out must be [m, N] bf16 or float32")
        a.out, a.ldo, a.out_f32 = out.data_ptr(), out.stride(0), int(out.dtype == torch.float32)
    elif epilogue == EPI_RESIDUAL:
        _dev("residual", residual, torch.float32)
        if residual.shape != (a.m, a.n):
            raise KernelError("skinny_gemm: residual must be [m, N] float32")
        a.residual = residual.data_ptr()
    elif epilogue == EPI_SWIGLU:
        _dev("out", out, torch.bfloat16)
        a.inter = a.n // 2
        if out.shape != (a.m, a.inter):
            raise KernelError("skinny_gemm: out must be [m, N / 2] bf16")
        a.out, a.ldo = out.data_ptr(), out.stride(0)
        if clamp is not None:
            if not float(clamp[0]) > 0:
                raise KernelError("skinny_gemm: the clamped gate needs a positive limit")
            a.gate_limit, a.gate_alpha = float(clamp[0]), float(clamp[1])
    elif epilogue == EPI_QKV:
        site = qkv["site"]
        _dev("q_out", qkv["q_out"], torch.bfloat16)
        _dev("cache", site.storage, torch.bfloat16)
        a.n_heads, a.kv_heads, a.head_dim = qkv["n_heads"], site.kv_heads, site.head_dim
        a.rot_dim, a.write_cache = qkv["rot_dim"], int(bool(qkv["write_cache"]))
        a.inv_freq = 0 if qkv["inv_freq"] is None else qkv["inv_freq"].data_ptr()
        a.tok_pos, a.tok_seq, a.slots = qkv["tok_pos"].data_ptr(), qkv["tok_seq"].data_ptr(), qkv["slots"].data_ptr()
        a.q_out, a.kv_base, a.table = qkv["q_out"].data_ptr(), site.storage.data_ptr(), site.table.data_ptr()
        a.page_elems, a.table_stride, a.err = site.page_elems, site.table_stride, qkv["err"].data_ptr()
        if qkv["q_out"].shape != (a.m, a.n_heads * a.head_dim):
            raise KernelError("skinny_gemm: q_out must be [m, n_heads * head_dim]")
    else:
        raise KernelError(f"skinny_gemm: unknown epilogue {epilogue}")
    if not a.err:
        a.err = (err if err is not None else _err_word_for(weight.device)).data_ptr()
    return a, norm


def skinny_gemm(epilogue: int, weight: torch.Tensor, **tensors) -> None:
    """One fused product for up to 16 token rows. Input rows are either `x` [m, K] bf16, or the float32 residual
    stream `hidden` [m, K] normalised on the fly with `norm_weight`, `eps`. Keywords: x | hidden, norm_weight, eps;
    bias; out (PLAIN, SWIGLU); residual (RESIDUAL); err; see csrc/skinny_gemm.cu for the epilogues.
    qkv (EPI_QKV): dict(n_heads, site=KvSiteArgs, inv_freq, rot_dim, tok_pos, tok_seq, slots, q_out, write_cache, err)."""
    a, norm = _skinny_args(epilogue, weight, **tensors)
    code = library("skinny_gemm").qf_skinny_gemm(_I(epilogue), _I(int(norm)), ctypes.byref(a), _stream())
    if code == 1:  # cudaErrorInvalidValue: a shape the kernel does not take
        raise KernelError(f"skinny_gemm: shape m={a.m} n={a.n} k={a.k} (epilogue {epilogue}) is not supported; "
                          "use the unfused kernels")
    _check(code, "skinny_gemm")


WIDE_MAX_ROWS = 64
_wide_answers: dict = {}


def wide_gemm_takes(epilogue: int, weight: torch.Tensor, **tensors) -> bool:
    """Whether `wide_gemm` runs this product (up to 64 token rows `x`; the library's own planning, launching nothing)."""
    x = tensors.get("x")
    if x is None or not (weight.is_cuda and weight.dtype == torch.bfloat16 and x.dtype == torch.bfloat16):
        return False
    qkv = tensors.get("qkv") or {}
    site = qkv.get("site")
    key = (weight.device.index, epilogue, tuple(weight.shape), weight.stride(0), tuple(x.shape), x.stride(0),
           weight.data_ptr() % 16, x.data_ptr() % 16, tensors.get("bias") is not None, qkv.get("n_heads"),
           None if site is None else (site.kv_heads, site.head_dim), qkv.get("rot_dim"), qkv.get("inv_freq") is not None)
    answer = _wide_answers.get(key)
    if answer is None:
        try:
            a, _ = _skinny_args(epilogue, weight, **tensors)
        except KernelError:
            return False
        with torch.cuda.device(weight.device):
            answer = library("wide_gemm").qf_wide_gemm_takes(_I(epilogue), ctypes.byref(a)) != 0
        _wide_answers[key] = answer
    return answer


def wide_gemm_takes_rows(epilogue: int, m: int, weight: torch.Tensor) -> bool:
    """`wide_gemm_takes` for planning, before the step's tensors exist: `m` contiguous, aligned token rows against
    `weight`, for the epilogues without further arguments (EPI_RESIDUAL, EPI_SWIGLU, EPI_PLAIN)."""
    if not (weight.is_cuda and weight.dtype == torch.bfloat16) or epilogue == EPI_QKV:
        return False
    key = (weight.device.index, epilogue, tuple(weight.shape), weight.stride(0), m, weight.data_ptr() % 16)
    answer = _wide_answers.get(key)
    if answer is None:
        a = _SkinnyArgs()
        a.w, a.n, a.k, a.ldw = weight.data_ptr(), weight.shape[0], weight.shape[1], weight.stride(0)
        a.x, a.ldx, a.m = 256, weight.shape[1], m          # only the alignment of the rows is looked at
        a.inter = a.n // 2 if epilogue == EPI_SWIGLU else 0
        with torch.cuda.device(weight.device):
            answer = library("wide_gemm").qf_wide_gemm_takes(_I(epilogue), ctypes.byref(a)) != 0
        _wide_answers[key] = answer
    return answer


def residual_product_way(m: int, weight: torch.Tensor) -> str:
    """How `m` token rows (64 at most) are multiplied by `weight` [N, K] and added into the residual stream fastest, by
    measurement on a B200 (`python -m qwenforge_b200.measure products`, Qwen2.5 0.5B / 3B / 7B sizes).
    Up to 16 rows the choice is between the two kernels that add in place: "skinny" (the mma.sync streamer) up to 8 rows
    while the weight is under 20 MB (0.5B: 3.0 and 4.8 microseconds against 3.4 and 5.5 on the tcgen05 streamer; 7B's
    26 MB output projection: 9.0 against 8.0), "wide" (the tcgen05 streamer) beyond (16 rows: 3.4 / 5.5 against 4.1 /
    6.6 at 0.5B, 14.9 against 16.2 at 3B's down product, 25.8 against 50 at 7B's).
    From 17 rows on the other way is the library product, whose result the next norm kernel adds at no cost: "wide" is
    the faster one only for products with a long K (a feed-forward's down product: 7.2 against 9 microseconds at 0.5B
    with 64 rows, 29.5 against 31.6 at 7B; an output projection: 4.6 against 3.1), so it needs K >= 2 N there.
    "unfused" (library product, addition by the next norm) is what remains."""
    size = weight.numel() * weight.element_size()
    skinny = m <= SKINNY_MAX_ROWS and skinny_gemm_takes(m, weight, EPI_RESIDUAL, False)
    wide = m <= WIDE_MAX_ROWS and wide_gemm_takes_rows(EPI_RESIDUAL, m, weight)
    if m > SKINNY_MAX_ROWS:
        return "wide" if wide and weight.shape[1] >= 2 * weight.shape[0] else "unfused"
    if skinny and (not wide or (m <= 8 and size < 20e6)):
        return "skinny"
    return "wide" if wide else "unfused"


def wide_gemm(epilogue: int, weight: torch.Tensor, **tensors) -> None:
    """One fused product for up to 64 token rows on the tcgen05 tensor cores (csrc/wide_gemm.cu): the keywords of
    `skinny_gemm`, with the input rows always given as `x` [m, K] bf16 (already normalised)."""
    a, norm = _skinny_args(epilogue, weight, **tensors)
    if norm:
        raise KernelError("wide_gemm: the input rows must be given as x (normalise them first)")
    code = library("wide_gemm").qf_wide_gemm(_I(epilogue), ctypes.byref(a), _stream())
    if code == 1:
        raise KernelError(f"wide_gemm: shape m={a.m} n={a.n} k={a.k} (epilogue {epilogue}) is not supported; "
                          "use the unfused kernels")
    if code == 801:
        raise KernelError("wide_gemm: the driver offers no tensor-map encoder (cuTensorMapEncodeTiled)")
    _check(code, "wide_gemm")


class FusedProduct:
    """One fused product, described but not run: the epilogue, the weight and the keywords of `skinny_gemm`. Parts hand
    these out so that whoever arranges them can run several as one chain (`skinny_chain`) or each alone (`run`)."""
    __slots__ = ("epilogue", "weight", "tensors")

    def __init__(self, epilogue: int, weight: torch.Tensor, **tensors):
        self.epilogue, self.weight, self.tensors = epilogue, weight, tensors

    def run(self) -> None:
        skinny_gemm(self.epilogue, self.weight, **self.tensors)


class _ChainProduct(ctypes.Structure):
    _fields_ = [("epilogue", _I), ("norm", _I), ("a", _SkinnyArgs)]


CHAIN_MAX_PRODUCTS = 4
_chain_answers: dict = {}


def _chain_array(products):
    array = (_ChainProduct * len(products))()
    for i, product in enumerate(products):
        a, norm = _skinny_args(product.epilogue, product.weight, **product.tensors)
        array[i].epilogue, array[i].norm, array[i].a = product.epilogue, int(norm), a
    return array


def skinny_chain_takes(products) -> bool:
    """Whether `skinny_chain` runs these products as ONE persistent kernel (the library's own planning, launching nothing)."""
    if not 1 <= len(products) <= CHAIN_MAX_PRODUCTS:
        return False
    key = tuple((p.epilogue, p.weight.shape, p.weight.stride(0), "hidden" in p.tensors,
                 (p.tensors.get("hidden") if "hidden" in p.tensors else p.tensors["x"]).shape[0],
                 p.tensors["x"].stride(0) if "x" in p.tensors else 0) for p in products) + (products[0].weight.device.index,)
    answer = _chain_answers.get(key)
    if answer is None:
        with torch.cuda.device(products[0].weight.device):
            answer = library("skinny_chain").qf_skinny_chain_takes(_I(len(products)), _chain_array(products)) != 0
        _chain_answers[key] = answer
    return answer


def skinny_chain(products, sync: torch.Tensor, err: torch.Tensor) -> None:
    """Runs up to four fused products, each reading what the one before wrote, as one persistent kernel whose blocks
    stream the weights of all of them without a pause (csrc/skinny_chain.cu). `sync`: two int32 words, zero when first
    used, that belong to this stream's chains."""
    _dev("sync", sync, torch.int32)
    _dev("err", err, torch.int32)
    if sync.numel() < 2:
        raise KernelError("skinny_chain: sync must hold two words")
    code = library("skinny_chain").qf_skinny_chain(_I(len(products)), _chain_array(products), _ptr(sync), _ptr(err), _stream())
    if code == 1:
        raise KernelError("skinny_chain: these products do not fit the chain kernel; run them one by one")
    _check(code, "skinny_chain")


def skinny_chain_repeated(products, repeats: int, steps, sync: torch.Tensor, err: torch.Tensor) -> None:
    """A measuring aid: the chain run `repeats` times over inside ONE launch. steps: per product the elements by which
    its weight, its bias and its norm weight advance per repeat (three lists; stacked tensors); all else is shared."""
    flat = (ctypes.c_longlong * 12)(*([0] * 12))
    for kind, values in enumerate(steps):
        for i, value in enumerate(values):
            flat[4 * kind + i] = int(value)
    code = library("skinny_chain").qf_skinny_chain_repeated(_I(len(products)), _chain_array(products), _I(repeats), flat,
                                                            _ptr(sync), _ptr(err), _stream())
    if code == 1:
        raise KernelError("skinny_chain: these products do not fit the chain kernel; run them one by one")
    _check(code, "skinny_chain_repeated")


def residual_add(hidden: torch.Tensor, delta: torch.Tensor) -> None:
    """hidden (float32) += delta, in place."""
    _dev("hidden", hidden, torch.float32)
    _dev("delta", delta)
    if delta.shape != hidden.shape:
        raise KernelError("residual_add: shapes differ")
    _check(library("norm").qf_residual_add(_I(_is_bf16(delta.dtype)), _ptr(hidden), _ptr(delta), _LL(hidden.numel()),
                                           _stream()), "residual_add")


# ---------------------------------------------------------------------------------------------- tcgen05 products

TC_PLAIN, TC_SWIGLU = 0, 1


def add_dyt_norm(hidden: torch.Tensor, a: Optional[torch.Tensor], b: Optional[torch.Tensor], weight: torch.Tensor,
                 bias: torch.Tensor, alpha: float, out: torch.Tensor) -> None:
    """hidden += (a + b) (each if given); out = tanh(alpha * hidden) * weight + bias: Dynamic Tanh in a norm's place, element by
    element, float32 inside. hidden float32 [R, W]; a, b, weight, bias, out share the activation dtype."""
    _dev("hidden", hidden, torch.float32)
    _dev("weight", weight)
    _dev("bias", bias, weight.dtype)
    _dev("out", out, weight.dtype)
    rows, width = hidden.shape
    if weight.shape != (width,) or bias.shape != (width,) or out.shape != hidden.shape:
        raise KernelError("add_dyt_norm: weight and bias must be [width], out must have hidden's shape")
    for name, t in (("a", a), ("b", b)):
        if t is not None:
            _dev(name, t, weight.dtype)
            if t.shape != hidden.shape:
                raise KernelError(f"add_dyt_norm: {name} and hidden differ in shape")
    _check(library("norm").qf_add_dyt_norm(_I(_is_bf16(weight.dtype)), _ptr(hidden), _ptr(a), _ptr(b), _ptr(weight), _ptr(bias),
                                           _F(alpha), _ptr(out), _I(rows), _I(width), _stream()), "add_dyt_norm")


def add_dyt_norm_shift(hidden: torch.Tensor, a: Optional[torch.Tensor], b: Optional[torch.Tensor], weight: torch.Tensor,
                       bias: torch.Tensor, alpha: float, out: torch.Tensor, taps: torch.Tensor, slots: torch.Tensor,
                       state: torch.Tensor, shifted: torch.Tensor) -> None:
    """`add_dyt_norm` for a step of one token per sequence with a token shift in the same kernel:
    shifted = taps[:, 0] * previous out of the row's slot (state[slot, :W], zeros for slot < 0) + taps[:, 1] * out, and
    state[slot, :W] <- out. What `causal_conv(out, taps, ..., single=True)` gives and keeps, bit for bit.
    taps float32 [W, 2]; slots int32 [R]; state float32 [slots, >= W]; shifted like out."""
    _dev("hidden", hidden, torch.float32)
    _dev("weight", weight)
    _dev("bias", bias, weight.dtype)
    _dev("out", out, weight.dtype)
    _dev("shifted", shifted, weight.dtype)
    _dev("taps", taps, torch.float32)
    _dev("slots", slots, torch.int32)
    _rows("state", state, torch.float32)
    rows, width = hidden.shape
    if weight.shape != (width,) or bias.shape != (width,) or out.shape != hidden.shape or shifted.shape != hidden.shape:
        raise KernelError("add_dyt_norm_shift: weight and bias must be [width], out and shifted must have hidden's shape")
    if taps.shape != (width, 2) or slots.numel() != rows or state.shape[1] < width:
        raise KernelError("add_dyt_norm_shift: taps must be [width, 2], slots [rows], state rows of at least width")
    for name, t in (("a", a), ("b", b)):
        if t is not None:
            _dev(name, t, weight.dtype)
            if t.shape != hidden.shape:
                raise KernelError(f"add_dyt_norm_shift: {name} and hidden differ in shape")
    _check(library("norm").qf_add_dyt_norm_shift(
        _I(_is_bf16(weight.dtype)), _ptr(hidden), _ptr(a), _ptr(b), _ptr(weight), _ptr(bias), _F(alpha), _ptr(out), _ptr(taps),
        _ptr(slots), _ptr(state), _LL(state.stride(0)), _ptr(shifted), _I(rows), _I(width), _stream()), "add_dyt_norm_shift")


def residual_add_pair(hidden: torch.Tensor, a: Optional[torch.Tensor], b: Optional[torch.Tensor]) -> None:
    """hidden += (a + b): the two pending outputs of one layer, summed with each other first (float32)."""
    _dev("hidden", hidden, torch.float32)
    first = a if a is not None else b
    if first is None:
        return
    for name, t in (("a", a), ("b", b)):
        if t is not None:
            _dev(name, t, first.dtype)
            if t.shape != hidden.shape:
                raise KernelError(f"residual_add_pair: {name} and hidden differ in shape")
    _check(library("norm").qf_residual_add_pair(_I(_is_bf16(first.dtype)), _ptr(hidden), _ptr(a), _ptr(b), _LL(hidden.numel()),
                                                _stream()), "residual_add_pair")


def stream_pair(hidden: torch.Tensor, a: Optional[torch.Tensor], b: Optional[torch.Tensor], other: torch.Tensor,
                out: torch.Tensor) -> None:
    """out[t] = [hidden[t] + (a[t] + b[t]) | other[t]] in out's dtype: two float32 streams side by side as a product's
    input; a, b are pending outputs (each if given, of out's dtype); hidden is not changed."""
    _dev("hidden", hidden, torch.float32)
    _dev("other", other, torch.float32)
    _dev("out", out)
    rows, width = hidden.shape
    if other.shape != hidden.shape or out.shape != (rows, 2 * width):
        raise KernelError("stream_pair: other must have hidden's shape, out twice its width")
    for name, t in (("a", a), ("b", b)):
        if t is not None:
            _dev(name, t, out.dtype)
            if t.shape != hidden.shape:
                raise KernelError(f"stream_pair: {name} and hidden differ in shape")
    _check(library("norm").qf_stream_pair(_I(_is_bf16(out.dtype)), _ptr(hidden), _ptr(a), _ptr(b), _ptr(other), _ptr(out), _I(rows),
                                          _I(width), _stream()), "stream_pair")


def head_gate(x: torch.Tensor, gate: torch.Tensor, n_heads: int) -> None:
    """x[t, h, :] *= sigmoid(gate[t, h]) in place: x [T, n_heads * D]; gate [T, n_heads], which may be columns of wider rows."""
    _dev("x", x)
    _rows("gate", gate, x.dtype)
    rows, width = x.shape
    if width % n_heads or gate.shape != (rows, n_heads):
        raise KernelError("head_gate: x must be [T, n_heads * D] and gate [T, n_heads]")
    _check(library("activation").qf_head_gate(_I(_is_bf16(x.dtype)), _ptr(x), _ptr(gate), _I(gate.stride(0)), _I(rows), _I(n_heads),
                                              _I(width // n_heads), _stream()), "head_gate")


def pool_cache_write(cu_q: torch.Tensor, tok_pos: torch.Tensor, slots: torch.Tensor, site: KvSiteArgs, blocks: KvSiteArgs,
                     pool: int, max_q_len: int, err: torch.Tensor) -> None:
    """For every block of `pool` positions that this step completed (its last position is among the step's tokens, whose
    keys and values are in the cache already): row b of `blocks` <- the mean of the block's keys and the mean of its values
    as `site` holds them (float32 sums, rounded to the cache's dtype)."""
    for name, t in (("cu_q", cu_q), ("tok_pos", tok_pos), ("slots", slots)):
        _dev(name, t, torch.int32)
    _dev("cache", site.storage)
    _dev("block rows", blocks.storage, site.storage.dtype)
    if pool <= 0 or (blocks.kv_heads, blocks.head_dim) != (site.kv_heads, site.head_dim):
        raise KernelError("pool_cache_write: pool must be positive and both caches of one head shape")
    _check(library("rope_cache").qf_pool_cache_write(
        _I(_is_bf16(site.storage.dtype)), _ptr(cu_q), _ptr(tok_pos), _ptr(slots), _I(slots.numel()), _ptr(site.storage),
        _ptr(site.table), _LL(site.page_elems), _I(site.table_stride), _ptr(blocks.storage), _ptr(blocks.table),
        _LL(blocks.page_elems), _I(blocks.table_stride), _I(site.kv_heads), _I(site.head_dim), _I(int(pool)),
        _I(int(max_q_len) // int(pool) + 1), _ptr(err), _stream()), "pool_cache_write")


def tc_gemm_takes(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether the tcgen05 kernel takes x [M, K] against weight [N, K]: bf16, K and the row strides multiples of 8."""
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.stride(1) == 1 and weight.stride(1) == 1
            and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and weight.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


class _TcQkvArgs(ctypes.Structure):
    _fields_ = [("bias", ctypes.c_void_p), ("angles", ctypes.c_void_p), ("tok_pos", ctypes.c_void_p), ("tok_seq", ctypes.c_void_p),
                ("slots", ctypes.c_void_p), ("q_out", ctypes.c_void_p), ("kv_base", ctypes.c_void_p), ("table", ctypes.c_void_p),
                ("page_elems", ctypes.c_longlong), ("table_stride", _I), ("n_heads", _I), ("kv_heads", _I), ("head_dim", _I),
                ("write_cache", _I)]


def rope_table(tok_pos: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """The rotation angles of a step's tokens, [tokens, rot_dim / 2, 2] float32 (cos, sin): made once, read by every layer."""
    _dev("tok_pos", tok_pos, torch.int32)
    _dev("inv_freq", inv_freq, torch.float32)
    table = torch.empty((tok_pos.numel(), inv_freq.numel(), 2), dtype=torch.float32, device=tok_pos.device)
    _check(library("rope_cache").qf_rope_table(_ptr(tok_pos), _ptr(inv_freq), _I(tok_pos.numel()), _I(inv_freq.numel()), _ptr(table),
                                               _stream()), "rope_table")
    return table


TC_QKV_HEAD_DIMS = (32, 64, 128)


def tc_gemm_qkv_takes(x: torch.Tensor, weight: torch.Tensor, head_dim: int) -> bool:
    """Whether `tc_gemm_qkv` takes these operands: what `tc_gemm_takes` asks, and whole heads per tile of 128 columns."""
    return head_dim in TC_QKV_HEAD_DIMS and tc_gemm_takes(x, weight)


def tc_gemm_qkv(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], angles: Optional[torch.Tensor],
                tok_seq: torch.Tensor, tok_pos: torch.Tensor, slots: torch.Tensor, n_heads: int, q_out: torch.Tensor,
                site: KvSiteArgs, write_cache: bool, err: torch.Tensor) -> None:
    """The query/key/value product of many token rows on the tcgen05 tensor cores with its bias, the rotation of q and k
    heads by the tokens' angles (`rope_table`; None: no rotation) and the writes in its epilogue: q to `q_out`
    [tokens, n_heads * head_dim], k and v to each token's place in its sequence's cache page."""
    _dev("x", x, torch.bfloat16, contiguous=False)
    _dev("weight", weight, torch.bfloat16, contiguous=False)
    _dev("q_out", q_out, torch.bfloat16)
    _dev("cache", site.storage, torch.bfloat16)
    d = site.head_dim
    m, k = x.shape
    if weight.shape != ((n_heads + 2 * site.kv_heads) * d, k) or q_out.shape != (m, n_heads * d):
        raise KernelError("tc_gemm_qkv: weight must be [(n_heads + 2 kv_heads) * head_dim, K] and q_out [tokens, n_heads * head_dim]")
    if not tc_gemm_qkv_takes(x, weight, d):
        raise KernelError(f"tc_gemm_qkv: head_dim {d} or the operands' alignment is not taken (head sizes {TC_QKV_HEAD_DIMS})")
    if angles is not None and (angles.dtype != torch.float32 or angles.shape != (m, d // 2, 2) or not angles.is_contiguous()):
        raise KernelError("tc_gemm_qkv: angles must be float32 [tokens, head_dim / 2, 2] (the whole head is rotated)")
    a = _TcQkvArgs()
    a.bias = None if bias is None else bias.data_ptr()
    a.angles = None if angles is None else angles.data_ptr()
    a.tok_pos, a.tok_seq, a.slots = tok_pos.data_ptr(), tok_seq.data_ptr(), slots.data_ptr()
    a.q_out, a.kv_base, a.table = q_out.data_ptr(), site.storage.data_ptr(), site.table.data_ptr()
    a.page_elems, a.table_stride = site.page_elems, site.table_stride
    a.n_heads, a.kv_heads, a.head_dim, a.write_cache = n_heads, site.kv_heads, d, int(bool(write_cache))
    code = library("tc_gemm").qf_tc_gemm_qkv(_ptr(x), _I(x.stride(0)), _ptr(weight), _I(weight.stride(0)), _I(m), _I(k),
                                             ctypes.byref(a), _ptr(err), _stream())
    if code == 801:
        raise KernelError("tc_gemm_qkv: the driver offers no tensor-map encoder (cuTensorMapEncodeTiled)")
    _check(code, "tc_gemm_qkv")


def tc_gemm_is_persistent(epilogue: int, m: int, n: int) -> bool:
    """Whether `tc_gemm` runs x [m, K] against weight [n, K] in its persistent kernel (tiles for every SM)."""
    return library("tc_gemm").qf_tc_gemm_is_persistent(_I(epilogue), _I(m), _I(n)) != 0


def tc_gemm(epilogue: int, x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, err: Optional[torch.Tensor] = None) -> None:
    """out = x @ weight.T on the tcgen05 tensor cores (bf16 in, float32 accumulate in tensor memory, bf16 out).
    TC_SWIGLU: weight = [gate rows | up rows], out [M, N / 2] = silu(x gate^T) * (x up^T)."""
    _dev("x", x, torch.bfloat16, contiguous=False)
    _dev("weight", weight, torch.bfloat16, contiguous=False)
    _dev("out", out, torch.bfloat16, contiguous=False)
    m, k = x.shape
    n = weight.shape[0]
    cols = n // 2 if epilogue == TC_SWIGLU else n
    if weight.shape[1] != k or out.shape != (m, cols) or out.stride(1) != 1:
        raise KernelError(f"tc_gemm: shapes {tuple(x.shape)} x {tuple(weight.shape)}^T -> {tuple(out.shape)} do not agree")
    if not tc_gemm_takes(x, weight) or out.stride(0) % 8 or out.data_ptr() % 16:
        raise KernelError("tc_gemm: operands must be bf16 with K and row strides multiples of 8 and 16-byte aligned")
    err = err if err is not None else _err_word_for(x.device)
    code = library("tc_gemm").qf_tc_gemm(_I(epilogue), _ptr(x), _I(x.stride(0)), _ptr(weight), _I(weight.stride(0)), _ptr(out),
                                         _I(out.stride(0)), _I(m), _I(n), _I(k), _ptr(err), _stream())
    if code == 801:
        raise KernelError("tc_gemm: the driver offers no tensor-map encoder (cuTensorMapEncodeTiled)")
    _check(code, "tc_gemm")


# ---------------------------------------------------------------------------------------------- parts of other designs

def embed_positions(ids: torch.Tensor, tok_pos: torch.Tensor, table: torch.Tensor, positions: torch.Tensor,
                    out: torch.Tensor, err: torch.Tensor) -> None:
    """out[t] = float32(table[ids[t]]) + float32(positions[tok_pos[t]]): a token embedding plus a learned vector per
    absolute position. ids, tok_pos int32 [T]; table [V, W], positions [P, W] of one dtype; out float32 [T, W]."""
    _dev("ids", ids, torch.int32)
    _dev("tok_pos", tok_pos, torch.int32)
    _dev("table", table)
    _dev("positions", positions, table.dtype)
    _dev("out", out, torch.float32)
    n, (vocab, width) = ids.numel(), table.shape
    if out.shape != (n, width) or positions.shape[1] != width or tok_pos.numel() != n:
        raise KernelError("embed_positions: out must be [tokens, width], positions [places, width]")
    _check(library("embed").qf_embed_positions(_I(_is_bf16(table.dtype)), _ptr(ids), _ptr(tok_pos), _ptr(table),
                                               _ptr(positions), _ptr(out), _I(n), _I(vocab), _I(positions.shape[0]),
                                               _I(width), _ptr(err), _stream()), "embed_positions")


def sandwich_norm(hidden: torch.Tensor, y: torch.Tensor, post_weight: torch.Tensor, post_eps: float,
                  next_weight: Optional[torch.Tensor] = None, next_eps: float = 0.0,
                  out: Optional[torch.Tensor] = None, dest: Optional[torch.Tensor] = None, top: int = 1,
                  row_weight: Optional[torch.Tensor] = None) -> None:
    """hidden += rmsnorm(y) * post_weight; then, if `next_weight` is given, out = rmsnorm(hidden) * next_weight: a
    sublayer's output normalised on its way into the float32 stream, and the stream normalised for the next sublayer, in
    one pass. y, the weights and out share a dtype. With `dest` (int32 [rows * top]), row t of the sublayer's output is the
    sum of the `top` rows y[dest[t * top + k]] (times row_weight[that row], float32, if given), summed in float32 on the way
    in: what a mixture of experts leaves per token (`MoePlan.dest`)."""
    _dev("hidden", hidden, torch.float32)
    _dev("y", y)
    _dev("post_weight", post_weight, y.dtype)
    rows, width = hidden.shape
    if dest is not None:
        _dev("dest", dest, torch.int32)
        if dest.numel() != rows * top or y.dim() != 2 or y.shape[1] != width:
            raise KernelError("sandwich_norm: dest must name `top` rows of y [*, width] per row of the stream")
        if row_weight is not None:
            _dev("row_weight", row_weight, torch.float32)
            if row_weight.numel() != y.shape[0]:
                raise KernelError("sandwich_norm: row_weight must hold one float32 per row of y")
    elif y.shape != hidden.shape:
        raise KernelError("sandwich_norm: y must have the stream's shape")
    if post_weight.numel() != width:
        raise KernelError("sandwich_norm: post_weight must have the stream's width")
    if next_weight is not None:
        _dev("next_weight", next_weight, y.dtype)
        _dev("out", out, y.dtype)
        if out.shape != hidden.shape or next_weight.numel() != width:
            raise KernelError("sandwich_norm: out must have the stream's shape and next_weight its width")
    _check(library("norm").qf_sandwich_norm(_I(_is_bf16(y.dtype)), _ptr(hidden), _ptr(y), _ptr(post_weight), _F(post_eps),
                                            _ptr(next_weight), _F(next_eps), _ptr(out if next_weight is not None else None),
                                            _I(rows), _I(width), _ptr(dest), _I(top if dest is not None else 1),
                                            _ptr(row_weight if dest is not None else None), _stream()), "sandwich_norm")


def clamped_glu(gate_up: torch.Tensor, limit: float, alpha: float, out: torch.Tensor) -> None:
    """out[t, i] = g * sigmoid(alpha * g) * (u + 1) with g = min(gate_up[t, i], limit), u = clamp(gate_up[t, I + i], -limit, limit)."""
    _dev("gate_up", gate_up)
    _dev("out", out, gate_up.dtype)
    rows, two_i = gate_up.shape
    if two_i % 2 or out.shape != (rows, two_i // 2):
        raise KernelError("clamped_glu: out must be [rows, width / 2]")
    _check(library("activation").qf_clamped_glu(_I(_is_bf16(gate_up.dtype)), _ptr(gate_up), _ptr(out), _I(rows),
                                                _I(two_i // 2), _F(limit), _F(alpha), _stream()), "clamped_glu")


def latent_norm_cache(down: torch.Tensor, q_rank: int, q_norm: Optional[torch.Tensor], kv_norm: torch.Tensor, eps: float,
                      tok_seq: torch.Tensor, tok_pos: torch.Tensor, slots: torch.Tensor, q_latent: Optional[torch.Tensor],
                      site: KvSiteArgs, write_cache: bool, err: torch.Tensor,
                      latent_out: Optional[torch.Tensor] = None) -> None:
    """The two latents of a latent attention from their fused down-projection `down` (float32 [T, q_rank + kv_rank]):
    q_latent [T, q_rank] = rmsnorm(down[:, :q_rank]) * q_norm, and rmsnorm(down[:, q_rank:]) * kv_norm written to each
    token's own position in a one-plane cache of a single head of kv_rank elements (`site`; and to `latent_out` in token
    order, if given). q_rank 0: no query latent."""
    _dev("down", down, torch.float32, contiguous=False)
    _dev("kv_norm", kv_norm)
    _dev("cache", site.storage, kv_norm.dtype)
    for name, t in (("tok_seq", tok_seq), ("tok_pos", tok_pos), ("slots", slots)):
        _dev(name, t, torch.int32)
    n, kv_rank = down.shape[0], site.head_dim
    if down.stride(1) != 1 or down.shape[1] != q_rank + kv_rank or site.kv_heads != 1 or kv_norm.numel() != kv_rank:
        raise KernelError("latent_norm_cache: down must be [tokens, q_rank + kv_rank] and the cache hold one head of kv_rank")
    if q_rank:
        _dev("q_norm", q_norm, kv_norm.dtype)
        _dev("q_latent", q_latent, kv_norm.dtype)
        if q_latent.shape != (n, q_rank) or q_norm.numel() != q_rank:
            raise KernelError("latent_norm_cache: q_latent must be [tokens, q_rank]")
    if latent_out is not None:
        _dev("latent_out", latent_out, kv_norm.dtype)
        if latent_out.shape != (n, kv_rank):
            raise KernelError("latent_norm_cache: latent_out must be [tokens, kv_rank]")
    _check(library("latent_cache").qf_latent_norm_cache(
        _I(_is_bf16(kv_norm.dtype)), _ptr(down), _I(down.stride(0)), _I(q_rank), _I(kv_rank), _ptr(q_norm if q_rank else None),
        _ptr(kv_norm), _F(eps), _ptr(tok_seq), _ptr(tok_pos), _ptr(slots), _ptr(q_latent if q_rank else None),
        _ptr(latent_out), _ptr(site.storage), _ptr(site.table), _LL(site.page_elems), _I(site.table_stride),
        _I(1 if write_cache else 0), _I(n), _ptr(err), _stream()), "latent_norm_cache")


def _grouped(x, weight, out, a_group_cols, c_group_cols, rows, plan, a_rows=None, gated=False, row_scale=None, clamp=None,
             activation=None) -> None:
    groups, n, k = weight.shape
    if gated:
        n //= 2   # columns of the result
    limit, alpha = (float(clamp[0]), float(clamp[1])) if clamp is not None else (0.0, 0.0)
    if activation is not None and (gated or activation not in ACTIVATIONS):
        raise KernelError(f"grouped_gemm: activation {activation!r} is not known, or was asked of a gated product")
    code = library("grouped_gemm").qf_grouped_gemm_act(
        _I(_is_bf16(x.dtype)), _ptr(x), _LL(x.stride(0)), _LL(a_group_cols), _ptr(weight), _LL(weight.stride(0)),
        _LL(weight.stride(1)), _ptr(out), _LL(out.stride(0)), _LL(c_group_cols), _I(rows), _I(n), _I(k), _I(groups),
        _ptr(plan.tile_group if plan else None), _ptr(plan.tile_row0 if plan else None), _ptr(plan.offsets if plan else None),
        _ptr(plan.n_tiles if plan else None), _I(plan.max_tiles if plan else 0), _I(plan.tile_rows if plan else 0),
        _ptr(a_rows), _I(int(gated)), _ptr(row_scale), _F(limit), _F(alpha), _I(0 if activation is None else ACTIVATIONS[activation] + 1),
        _stream())
    if code == 1:
        raise KernelError("grouped_gemm: the plan's tiles do not fit these operands (tiles of 128 rows need bfloat16 operands "
                          "whose K and strides are multiples of 8), or the grid is too large")
    _check(code, "grouped_gemm")


def head_linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
    """A product per head in one launch: out[:, g*N:(g+1)*N] = x[:, g*K:(g+1)*K] @ weight[g].T for weight [G, N, K],
    x [T, G*K], out [T, G*N], all of the activation dtype."""
    _dev("x", x, None, contiguous=False)
    _dev("weight", weight, x.dtype, contiguous=False)
    _dev("out", out, x.dtype, contiguous=False)
    groups, n, k = weight.shape
    if x.shape[1] != groups * k or out.shape != (x.shape[0], groups * n) or weight.stride(2) != 1 or x.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError(f"head_linear: shapes {tuple(x.shape)} x {tuple(weight.shape)} -> {tuple(out.shape)} do not agree")
    _grouped(x, weight, out, k, n, x.shape[0], None)


GROUP_TILE_ROWS = 64          # rows of a tile of the grouped products (QF_GROUP_BM in csrc/common.cuh)
GROUP_LARGE_TILE_ROWS = 128   # and of the large tile, for bfloat16 operands with rows enough
MOE_FUSED_ROUTER_MAX = 4096   # tokens x experts up to which the plan's one block makes the router's logits itself
MOE_LONG_PLAN_TOKENS = 1024   # tokens from which the plan is made by three parallel launches instead of one block


class MoePlan:
    """One routing of a step's tokens over experts, on the device (csrc/moe.cu): `top` (token, expert) pairs per token,
    sorted by expert into rows. dest[t * top + j]: the row of token t's j-th choice; sorted_token / sorted_weight: each row's
    token and routing weight; offsets: every expert's first row; tile_*: the rows cut into tiles for `expert_linear`."""

    def __init__(self, n_tokens: int, n_experts: int, top: int, device, tile_rows: int = GROUP_TILE_ROWS):
        self.n_tokens, self.n_experts, self.top, self.tile_rows = n_tokens, n_experts, top, tile_rows
        self.pairs = pairs = n_tokens * top
        self.max_tiles = -(-pairs // tile_rows) + n_experts   # the most tiles any routing can have
        ints = torch.empty(3 * pairs + n_experts + 1 + 2 * self.max_tiles + 1, dtype=torch.int32, device=device)
        floats = torch.empty(2 * pairs, dtype=torch.float32, device=device)
        o = 0

        def take(count):
            nonlocal o
            piece = ints[o:o + count]
            o += count
            return piece

        self.pair_expert, self.sorted_token, self.dest = take(pairs), take(pairs), take(pairs)
        self.offsets, self.tile_group, self.tile_row0, self.n_tiles = take(n_experts + 1), take(self.max_tiles), take(self.max_tiles), take(1)
        self.pair_weight, self.sorted_weight = floats[:pairs], floats[pairs:]


def moe_tile_rows(n_tokens: int, n_experts: int, top: int, weight: torch.Tensor) -> int:
    """The tile height for the experts' products of a step: 128 where the experts have rows enough to fill such tiles
    (two of them each on average) and the operands allow the large tile, else 64."""
    if weight.dtype != torch.bfloat16 or n_tokens * top < 2 * GROUP_LARGE_TILE_ROWS * n_experts:
        return GROUP_TILE_ROWS
    aligned = all(s % 8 == 0 for s in (weight.stride(0), weight.stride(1), weight.shape[2])) and weight.data_ptr() % 16 == 0
    return GROUP_LARGE_TILE_ROWS if aligned else GROUP_TILE_ROWS


def moe_plan(logits: Optional[torch.Tensor], top: int, softmax_scores: bool = False, renormalize: bool = False,
             tile_rows: int = GROUP_TILE_ROWS, x: Optional[torch.Tensor] = None, router: Optional[torch.Tensor] = None,
             bias: Optional[torch.Tensor] = None, correction: Optional[torch.Tensor] = None, groups=None) -> MoePlan:
    """Route: logits float32 [T, E] -> the `top` experts with the largest scores per token (sigmoid of the logit, or the
    softmax over the experts) and the sorted rows (see `MoePlan`), cut into tiles of `tile_rows`. Everything stays on the
    device. With `logits` None, the kernel makes the logits itself from `x` [T, W] and `router` [E, W] (float32 sums; for
    steps of few tokens, T * E <= MOE_FUSED_ROUTER_MAX). `bias` (float32 [E]) is added to the logits before the choice.
    `correction` (float32 [E]) and `groups` = (count, keep), with sigmoid scores: the choice goes by score + correction, and
    only among the experts of the `keep` best of `count` equal groups of neighbouring experts, a group's score being the sum
    of its two largest choice scores; the weights are the scores without the correction."""
    if bias is not None:
        _dev("bias", bias, torch.float32)
    group_count, group_keep = (0, 0)
    if correction is not None or groups is not None:
        group_count, group_keep = (int(groups[0]), int(groups[1])) if groups is not None else (1, 1)
        if softmax_scores:
            raise KernelError("moe_plan: a correction or groups go with sigmoid scores")
        if correction is not None:
            _dev("correction", correction, torch.float32)
    if logits is not None:
        _dev("logits", logits, torch.float32)
        n_tokens, n_experts = logits.shape
        width = 0
    else:
        _dev("x", x)
        _dev("router", router, x.dtype)
        (n_tokens, width), n_experts = x.shape, router.shape[0]
        if router.shape[1] != width or n_tokens * n_experts > MOE_FUSED_ROUTER_MAX:
            raise KernelError("moe_plan: x [T, W] and router [E, W] with T * E <= %d, or give the logits" % MOE_FUSED_ROUTER_MAX)
    if bias is not None and bias.numel() != n_experts:
        raise KernelError("moe_plan: bias must hold one float32 per expert")
    if correction is not None and correction.numel() != n_experts:
        raise KernelError("moe_plan: correction must hold one float32 per expert")
    if group_count and (not 1 <= group_keep <= group_count <= 64 or n_experts % group_count or group_keep * (n_experts // group_count) < top):
        raise KernelError(f"moe_plan: {group_keep} of {group_count} groups over {n_experts} experts cannot yield {top} choices "
                          "(up to 64 equal groups)")
    plan = MoePlan(n_tokens, n_experts, top, (logits if logits is not None else x).device, tile_rows)
    if logits is not None and n_tokens >= MOE_LONG_PLAN_TOKENS and n_experts <= 4096:
        expert_rows = torch.zeros(n_experts, dtype=torch.int32, device=logits.device)
        code = library("moe").qf_moe_plan_long_grouped(
            _ptr(logits), _I(n_tokens), _I(n_experts), _I(top), _I(int(softmax_scores)), _I(int(renormalize)),
            _ptr(plan.pair_expert), _ptr(plan.pair_weight), _ptr(plan.sorted_token), _ptr(plan.sorted_weight), _ptr(plan.dest),
            _ptr(plan.offsets), _ptr(plan.tile_group), _ptr(plan.tile_row0), _ptr(plan.n_tiles), _I(plan.max_tiles),
            _I(tile_rows), _ptr(expert_rows), _ptr(bias), _ptr(correction), _I(group_count), _I(group_keep), _stream())
        if code == 1:
            raise KernelError(f"moe_plan: {top} of {n_experts} experts is not supported (top <= 16)")
        _check(code, "moe_plan")
        return plan
    code = library("moe").qf_moe_plan_grouped(_ptr(logits), _I(n_tokens), _I(n_experts), _I(top), _I(int(softmax_scores)),
                                      _I(int(renormalize)), _ptr(plan.pair_expert), _ptr(plan.pair_weight),
                                      _ptr(plan.sorted_token), _ptr(plan.sorted_weight), _ptr(plan.dest), _ptr(plan.offsets),
                                      _ptr(plan.tile_group), _ptr(plan.tile_row0), _ptr(plan.n_tiles), _I(plan.max_tiles),
                                      _I(tile_rows), _ptr(x if logits is None else None), _ptr(router if logits is None else None),
                                      _I(width), _I(_is_bf16(x.dtype) if logits is None else 0), _ptr(bias), _ptr(correction),
                                      _I(group_count), _I(group_keep), _stream())
    if code == 1:
        raise KernelError(f"moe_plan: {top} of {n_experts} experts is not supported (top <= 16, experts <= 8192)")
    _check(code, "moe_plan")
    return plan


def moe_gather(x: torch.Tensor, plan: MoePlan, out: torch.Tensor, scale_input: bool) -> None:
    """out[row] = x[token of the row] (times the row's routing weight with `scale_input`); out [T * top, W]."""
    _dev("x", x)
    _dev("out", out, x.dtype)
    if out.shape != (plan.pairs, x.shape[1]) or x.shape[0] != plan.n_tokens:
        raise KernelError("moe_gather: out must be [tokens * top, width]")
    _check(library("moe").qf_moe_gather(_I(_is_bf16(x.dtype)), _ptr(x), _ptr(plan.sorted_token), _ptr(plan.sorted_weight),
                                        _ptr(out), _I(plan.pairs), _I(x.shape[1]), _I(int(scale_input)), _stream()), "moe_gather")


def moe_combine(y: torch.Tensor, plan: MoePlan, out: torch.Tensor, scale_output: bool, extra: Optional[torch.Tensor] = None,
                extra_gate: Optional[torch.Tensor] = None, gate_input: Optional[torch.Tensor] = None,
                gate_weight: Optional[torch.Tensor] = None) -> None:
    """out[t] = the sum over token t's choices, in their order, of y[row of the choice] (times the routing weight with
    `scale_output`), summed in float32; y [T * top, W], out [T, W]. `extra` [T, W] is an output that every token gets beside
    its chosen ones; it is added times sigmoid(extra_gate[t]) where `extra_gate` (float32, one logit per token) is given, or
    times sigmoid(gate_input[t] . gate_weight) where the kernel is to form that logit itself (gate_input [T, K], gate_weight
    [K], float32 sums)."""
    _dev("y", y)
    _dev("out", out, y.dtype)
    if y.shape[0] != plan.pairs or out.shape != (plan.n_tokens, y.shape[1]):
        raise KernelError("moe_combine: y must be [tokens * top, width], out [tokens, width]")
    if extra is not None:
        _dev("extra", extra, y.dtype)
        if extra.shape != out.shape:
            raise KernelError("moe_combine: extra must have out's shape")
    if extra_gate is not None:
        _dev("extra_gate", extra_gate, torch.float32)
        if extra is None or extra_gate.numel() != plan.n_tokens:
            raise KernelError("moe_combine: extra_gate holds one float32 per token and goes with extra")
    gate_k = 0
    if gate_weight is not None:
        _dev("gate_input", gate_input, y.dtype)
        _dev("gate_weight", gate_weight, y.dtype)
        gate_k = gate_weight.numel()
        if extra is None or extra_gate is not None or gate_input.shape != (plan.n_tokens, gate_k):
            raise KernelError("moe_combine: gate_weight [K] goes with extra and gate_input [tokens, K], and not with extra_gate")
    _check(library("moe").qf_moe_combine_shared(_I(_is_bf16(y.dtype)), _ptr(y), _ptr(plan.dest), _ptr(plan.sorted_weight), _ptr(out),
                                                _I(plan.n_tokens), _I(plan.top), _I(y.shape[1]), _I(int(scale_output)), _ptr(extra),
                                                _ptr(extra_gate), _ptr(gate_input if gate_k else None),
                                                _ptr(gate_weight if gate_k else None), _I(gate_k), _stream()), "moe_combine")


def expert_linear(x: torch.Tensor, weight: torch.Tensor, plan: MoePlan, out: torch.Tensor, gather: bool = False,
                  activation: Optional[str] = None) -> None:
    """out[row] = x[row] @ weight[expert of the row].T for rows sorted by expert (`plan`): x [T * top, K], weight [E, N, K],
    out [T * top, N], all of the activation dtype; one launch, no count on the host. With `gather`, x is the tokens' own
    rows [T, K] and row r reads x[token of r]: the sorted rows are never stored. With `activation` (a name of `ACTIVATIONS`)
    the product's epilogue applies it to the float32 sums before they are stored."""
    _dev("x", x)
    _dev("weight", weight, x.dtype)
    _dev("out", out, x.dtype)
    groups, n, k = weight.shape
    if groups != plan.n_experts or x.shape != ((plan.n_tokens if gather else plan.pairs), k) or out.shape != (plan.pairs, n):
        raise KernelError(f"expert_linear: shapes {tuple(x.shape)} x {tuple(weight.shape)} -> {tuple(out.shape)} do not agree")
    _grouped(x, weight, out, 0, 0, plan.pairs, plan, plan.sorted_token if gather else None, activation=activation)


def expert_gate_takes(x: torch.Tensor, weight: torch.Tensor, plan: MoePlan) -> bool:
    """Whether `expert_gate_up` takes these operands: bfloat16, tiles of 64 rows, K and the strides multiples of 8, 16-byte
    aligned bases."""
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and plan.tile_rows == GROUP_TILE_ROWS and weight.shape[1] % 2 == 0
            and all(v % 8 == 0 for v in (x.stride(0), weight.stride(0), weight.stride(1), weight.shape[2]))
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def expert_gate_up(x: torch.Tensor, weight: torch.Tensor, plan: MoePlan, out: torch.Tensor,
                   row_scale: Optional[torch.Tensor] = None, gather: bool = False, clamp=None) -> None:
    """An expert's gate/up product and its gate in one kernel: out[row] = silu(s g) * (s u) with [g | u] = x[row] @
    weight[expert of the row].T, weight [E, 2 F, K] (gate rows then up rows), out [T * top, F], s = row_scale[row] (float32) or
    1. `gather` as in `expert_linear`. bfloat16 on the tensor cores only (`expert_gate_takes`).
    clamp = (limit, alpha), limit > 0: the clamped gate instead, min(g, limit) sigmoid(alpha min(g, limit)) (clamp(u, -limit,
    limit) + 1), on the float32 sums."""
    if clamp is not None and not float(clamp[0]) > 0:
        raise KernelError("expert_gate_up: the clamped gate needs a positive limit")
    _dev("x", x, torch.bfloat16)
    _dev("weight", weight, torch.bfloat16)
    _dev("out", out, torch.bfloat16)
    groups, n2, k = weight.shape
    if not expert_gate_takes(x, weight, plan):
        raise KernelError("expert_gate_up: bfloat16 operands with K and strides multiples of 8 and a plan of 64-row tiles")
    if groups != plan.n_experts or x.shape != ((plan.n_tokens if gather else plan.pairs), k) or out.shape != (plan.pairs, n2 // 2):
        raise KernelError(f"expert_gate_up: shapes {tuple(x.shape)} x {tuple(weight.shape)} -> {tuple(out.shape)} do not agree")
    if row_scale is not None:
        _dev("row_scale", row_scale, torch.float32)
    _grouped(x, weight, out, 0, 0, plan.pairs, plan, plan.sorted_token if gather else None, True, row_scale, clamp)


def scaled_swiglu(gate_up: torch.Tensor, row_scale: torch.Tensor, out: torch.Tensor) -> None:
    """out[r, i] = silu(s_r * gate_up[r, i]) * (s_r * gate_up[r, I + i]): SwiGLU of rows whose input was to be multiplied by
    s_r (float32 [rows]), on the product of the unscaled rows."""
    _dev("gate_up", gate_up)
    _dev("row_scale", row_scale, torch.float32)
    _dev("out", out, gate_up.dtype)
    rows, two_i = gate_up.shape
    if two_i % 2 or out.shape != (rows, two_i // 2) or row_scale.numel() != rows:
        raise KernelError("scaled_swiglu: out must be [rows, width / 2], row_scale [rows]")
    _check(library("activation").qf_scaled_swiglu(_I(_is_bf16(gate_up.dtype)), _ptr(gate_up), _ptr(row_scale), _ptr(out),
                                                  _I(rows), _I(two_i // 2), _stream()), "scaled_swiglu")


def tc_gemm_grouped_takes(x: torch.Tensor, weight: torch.Tensor, plan: MoePlan, epilogue: int = TC_PLAIN) -> bool:
    """Whether `tc_gemm_grouped` takes these operands: bfloat16, a plan cut into tiles of 128 rows, K and the strides
    multiples of 8, 16-byte aligned bases, and for TC_SWIGLU an expert size that is a multiple of 8."""
    if plan.tile_rows != GROUP_LARGE_TILE_ROWS or weight.dim() != 3 or not weight.is_contiguous() or plan.max_tiles > 65535:
        return False
    if epilogue == TC_SWIGLU and (weight.shape[1] % 2 or (weight.shape[1] // 2) % 8):
        return False
    return tc_gemm_takes(x, weight.view(-1, weight.shape[2]))


def tc_gemm_grouped(epilogue: int, x: torch.Tensor, weight: torch.Tensor, plan: MoePlan, out: torch.Tensor,
                    row_scale: Optional[torch.Tensor] = None, err: Optional[torch.Tensor] = None,
                    clamp: Optional[tuple] = None) -> None:
    """The experts' products on the tcgen05 tensor cores: out[row] = x[row] @ weight[expert of the row].T for rows sorted by
    expert (`plan`, tiles of 128 rows); x [T * top, K], weight [E, N, K], out [T * top, N]. TC_SWIGLU: weight[e] = [gate rows |
    up rows], out [T * top, N / 2] = silu(s g) * (s u) with s = row_scale[row] (float32, or 1 when None); with
    `clamp` = (limit, alpha) the gate is the clamped one instead: min(g, limit) * sigmoid(alpha * min(g, limit)) *
    (clamp(u, -limit, limit) + 1)."""
    _dev("x", x, torch.bfloat16, contiguous=False)
    _dev("weight", weight, torch.bfloat16)
    _dev("out", out, torch.bfloat16, contiguous=False)
    groups, n, k = weight.shape
    cols = n // 2 if epilogue == TC_SWIGLU else n
    if x.shape != (plan.pairs, k) or out.shape != (plan.pairs, cols) or groups != plan.n_experts or out.stride(1) != 1:
        raise KernelError(f"tc_gemm_grouped: shapes {tuple(x.shape)} x {tuple(weight.shape)} -> {tuple(out.shape)} do not agree")
    if not tc_gemm_grouped_takes(x, weight, plan, epilogue) or out.stride(0) % 8 or out.data_ptr() % 16:
        raise KernelError("tc_gemm_grouped: operands must be bf16 with K and row strides multiples of 8, 16-byte aligned, and the "
                          "plan cut into tiles of 128 rows")
    if row_scale is not None:
        _dev("row_scale", row_scale, torch.float32)
        if row_scale.numel() != plan.pairs or epilogue != TC_SWIGLU:
            raise KernelError("tc_gemm_grouped: row_scale is one float32 per row, for TC_SWIGLU")
    if clamp is not None and (epilogue != TC_SWIGLU or not clamp[0] > 0):
        raise KernelError("tc_gemm_grouped: the clamped gate goes with TC_SWIGLU and a positive limit")
    err = err if err is not None else _err_word_for(x.device)
    code = library("tc_gemm").qf_tc_gemm_grouped_gated(
        _I(epilogue), _ptr(x), _I(x.stride(0)), _ptr(weight), _I(weight.stride(1)), _I(groups), _ptr(out), _I(out.stride(0)),
        _I(plan.pairs), _I(n), _I(k), _ptr(plan.tile_group), _ptr(plan.tile_row0), _ptr(plan.offsets), _ptr(plan.n_tiles),
        _I(plan.max_tiles), _ptr(row_scale), _F(clamp[0] if clamp else 0.0), _F(clamp[1] if clamp else 0.0), _ptr(err), _stream())
    if code == 801:
        raise KernelError("tc_gemm_grouped: the driver offers no tensor-map encoder (cuTensorMapEncodeTiled)")
    _check(code, "tc_gemm_grouped")


# ---------------------------------------------------------------------------------------------------------------------
# Elementwise kernels of feed-forwards with a bias and of capped logits (csrc/activation.cu)
ACTIVATIONS = {"relu2": 0, "gelu_tanh": 1, "silu": 2, "relu": 3, "gelu": 4, "tanh": 5}


def bias_act(x: torch.Tensor, bias: Optional[torch.Tensor], kind: str, out: torch.Tensor) -> None:
    """out = act(x + bias), float32 inside. kind: relu2 (the square of relu), gelu_tanh, gelu (the exact form, through erf), silu, relu, tanh."""
    _dev("x", x)
    _dev("out", out, x.dtype)
    if kind not in ACTIVATIONS:
        raise KernelError(f"bias_act: unknown activation {kind!r}; known: {', '.join(ACTIVATIONS)}")
    rows, width = x.shape
    if out.shape != x.shape:
        raise KernelError("bias_act: out must have x's shape")
    if bias is not None:
        _dev("bias", bias, x.dtype)
        if bias.numel() != width:
            raise KernelError("bias_act: bias must hold one element per column")
    _check(library("activation").qf_bias_act(_I(_is_bf16(x.dtype)), _ptr(x), _ptr(bias), _ptr(out), _I(rows), _I(width),
                                             _I(ACTIVATIONS[kind]), _stream()), "bias_act")


def softcap_(x: torch.Tensor, cap: float) -> None:
    """x <- cap * tanh(x / cap) in place; float32 (logits)."""
    _dev("x", x, torch.float32)
    if cap <= 0:
        raise KernelError("softcap_: the cap must be positive")
    _check(library("activation").qf_softcap(_ptr(x), _LL(x.numel()), _F(cap), _stream()), "softcap_")


# ---------------------------------------------------------------------------------------------------------------------
# Recurrent mixers (csrc/recurrent.cu): a state of fixed size per sequence, S <- decay * S + take * k v^T, y = S^T q.
# `state` is a cache's fixed-size state of one schedule entry, float32 [slots, floats]; each kernel is told where in a
# slot's row its piece starts. A sequence whose slot is -1 (padding) runs from a zero state and stores nothing.
def _state(state: torch.Tensor, *pieces) -> None:
    _dev("state", state, torch.float32)
    if state.dim() != 2:
        raise KernelError("the recurrent state must be float32 [slots, floats]")
    for offset, size in pieces:
        if offset < 0 or offset + size > state.shape[1]:
            raise KernelError(f"a piece of {size} floats at {offset} does not fit a state of {state.shape[1]} floats per slot")


def _rows(name: str, t: torch.Tensor, dtype=None) -> None:
    _dev(name, t, dtype, contiguous=False)
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{name} must be 2-d with unit inner stride")


def stabilized_gates(pre: torch.Tensor, bias: torch.Tensor, cap: float, cu_q: torch.Tensor, slots: torch.Tensor,
                     state: torch.Tensor, m_offset: int, n_heads: int, decay: torch.Tensor, take: torch.Tensor,
                     floor: torch.Tensor) -> None:
    """The exponential gates of a matrix memory with a running maximum, per head. pre: float32 [T, 2 H], the input gate's
    and then the forget gate's pre-activations; bias float32 [2 H]. With a = cap tanh((pre_i + b_i) / cap),
    f = logsigmoid(cap tanh((pre_f + b_f) / cap)) and m the running maximum kept in `state` (H floats at m_offset, 0 at a
    sequence's start): m' = max(f + m, a), decay = exp(f + m - m'), take = exp(a - m'), floor = exp(-m'); all float32 [T, H]."""
    _rows("pre", pre, torch.float32)
    _dev("bias", bias, torch.float32)
    n = pre.shape[0]
    if pre.shape[1] != 2 * n_heads or bias.numel() != 2 * n_heads:
        raise KernelError("stabilized_gates: pre must be [T, 2 * heads], bias [2 * heads]")
    for name, t in (("decay", decay), ("take", take), ("floor", floor)):
        _dev(name, t, torch.float32)
        if t.shape != (n, n_heads):
            raise KernelError(f"stabilized_gates: {name} must be float32 [T, heads]")
    _state(state, (m_offset, n_heads))
    _check(library("recurrent").qf_stabilized_gates(
        _ptr(pre), _I(pre.stride(0)), _ptr(bias), _F(cap), _ptr(cu_q), _ptr(slots), _I(cu_q.numel() - 1), _ptr(state),
        _LL(state.stride(0)), _LL(m_offset), _I(n_heads), _ptr(decay), _ptr(take), _ptr(floor), _stream()), "stabilized_gates")


def decay_gates(dt_pre: torch.Tensor, dt_bias: torch.Tensor, rate_log: torch.Tensor, decay: torch.Tensor,
                take: torch.Tensor) -> None:
    """The gates of a state-space recurrence: dt = softplus(dt_pre + dt_bias), decay = exp(-exp(rate_log) * dt), take = dt.
    dt_pre float32 [T, H] (rows may be strided); dt_bias, rate_log float32 [H]; decay, take float32 [T, H]."""
    _rows("dt_pre", dt_pre, torch.float32)
    n, h = dt_pre.shape
    for name, t in (("dt_bias", dt_bias), ("rate_log", rate_log)):
        _dev(name, t, torch.float32)
        if t.numel() != h:
            raise KernelError(f"decay_gates: {name} must hold one float32 per head")
    for name, t in (("decay", decay), ("take", take)):
        _dev(name, t, torch.float32)
        if t.shape != (n, h):
            raise KernelError(f"decay_gates: {name} must be float32 [T, heads]")
    _check(library("recurrent").qf_decay_gates(_ptr(dt_pre), _I(dt_pre.stride(0)), _ptr(dt_bias), _ptr(rate_log), _I(n), _I(h),
                                               _ptr(decay), _ptr(take), _stream()), "decay_gates")


OUTER_STATE_MAX_DIM = 256


def outer_state_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, take: torch.Tensor,
                     cu_q: torch.Tensor, slots: torch.Tensor, state: torch.Tensor, s_offset: int, n_offset: int,
                     n_heads: int, n_groups: int, dim: int, vdim: int, q_scale: float, y: torch.Tensor,
                     nq: Optional[torch.Tensor]) -> None:
    """The recurrence of a matrix state per head, token after token of every sequence, all float32 inside:
        S <- decay_t S + take_t k_t v_t^T   (S: dim x vdim, kept in `state` at s_offset as [heads, dim, vdim]);  y_t = S^T (q_scale q_t)
    and, with `nq`, a vector n <- decay_t n + take_t k_t beside it (at n_offset, [heads, dim]) and nq_t = n . (q_scale q_t).
    q, k: [T, groups * dim] (head h reads group h // (heads / groups)), v: [T, heads * vdim], in the activation dtype, rows
    may be strided; decay, take: float32 [T, heads]; y: float32 [T, heads * vdim]; nq: float32 [T, heads] or None."""
    for name, t in (("q", q), ("k", k), ("v", v)):
        _rows(name, t, q.dtype)
    _is_bf16(q.dtype)
    n = q.shape[0]
    if n_groups <= 0 or n_heads % n_groups or q.shape[1] != n_groups * dim or k.shape != q.shape or v.shape != (n, n_heads * vdim):
        raise KernelError("outer_state_scan: q, k must be [T, groups * dim], v [T, heads * vdim]")
    if dim > OUTER_STATE_MAX_DIM:
        raise KernelError(f"outer_state_scan: a state of {dim} rows per head exceeds the kernel's {OUTER_STATE_MAX_DIM}")
    for name, t in (("decay", decay), ("take", take)):
        _dev(name, t, torch.float32)
        if t.shape != (n, n_heads):
            raise KernelError(f"outer_state_scan: {name} must be float32 [T, heads]")
    _dev("y", y, torch.float32)
    if y.shape != (n, n_heads * vdim):
        raise KernelError("outer_state_scan: y must be float32 [T, heads * vdim]")
    pieces = [(s_offset, n_heads * dim * vdim)]
    if nq is not None:
        _dev("nq", nq, torch.float32)
        if nq.shape != (n, n_heads):
            raise KernelError("outer_state_scan: nq must be float32 [T, heads]")
        pieces.append((n_offset, n_heads * dim))
    _state(state, *pieces)
    _check(library("recurrent").qf_outer_state_scan(
        _I(_is_bf16(q.dtype)), _ptr(q), _I(q.stride(0)), _ptr(k), _I(k.stride(0)), _ptr(v), _I(v.stride(0)), _ptr(decay),
        _ptr(take), _ptr(cu_q), _ptr(slots), _I(cu_q.numel() - 1), _ptr(state), _LL(state.stride(0)), _LL(s_offset),
        _LL(n_offset if nq is not None else -1), _I(n_heads), _I(n_groups), _I(dim), _I(vdim), _F(q_scale), _ptr(y), _ptr(nq),
        _stream()), "outer_state_scan")


GATES = {"sigmoid": 0, "silu": 1}


def gated_group_norm(y: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, n_parts: int,
                     n_heads: int, gate_kind: str, gate_first: bool, nq: Optional[torch.Tensor] = None,
                     floor: Optional[torch.Tensor] = None, floor_add: float = 0.0, skip: Optional[torch.Tensor] = None,
                     skip_x: Optional[torch.Tensor] = None) -> None:
    """What follows a recurrent mixer's scan, one pass per token, float32 inside. y: float32 [T, C] in `n_heads` heads.
      with nq, floor (float32 [T, heads]):  y <- y / (max(|nq|, floor) + floor_add)          per head
      with skip (float32 [heads]), skip_x [T, C]:  y <- y + skip[head] * skip_x              per head
      gate_first:  y <- y * act(gate);   y <- y / rms(y) over each of `n_parts` equal parts (eps inside the root);
      y <- y * weight;   not gate_first:  y <- y * act(gate).   act: sigmoid or silu.
    gate, skip_x: [T, C] in the activation dtype, rows may be strided; weight [C] and out [T, C] in the activation dtype."""
    _dev("y", y, torch.float32)
    _rows("gate", gate, out.dtype)
    _dev("weight", weight, out.dtype)
    _dev("out", out)
    _is_bf16(out.dtype)
    n, c = y.shape
    if gate.shape != (n, c) or out.shape != (n, c) or weight.numel() != c or n_parts <= 0 or c % n_parts or c % n_heads:
        raise KernelError("gated_group_norm: gate and out must be [T, C] like y, weight [C]; parts and heads must divide C")
    if gate_kind not in GATES:
        raise KernelError(f"gated_group_norm: unknown gate {gate_kind!r}")
    if (nq is None) != (floor is None) or (skip is None) != (skip_x is None):
        raise KernelError("gated_group_norm: nq goes with floor, skip with skip_x")
    if nq is not None:
        for name, t in (("nq", nq), ("floor", floor)):
            _dev(name, t, torch.float32)
            if t.shape != (n, n_heads):
                raise KernelError(f"gated_group_norm: {name} must be float32 [T, heads]")
    if skip is not None:
        _dev("skip", skip, torch.float32)
        _rows("skip_x", skip_x, out.dtype)
        if skip.numel() != n_heads or skip_x.shape != (n, c):
            raise KernelError("gated_group_norm: skip must be float32 [heads], skip_x [T, C]")
    _check(library("recurrent").qf_gated_group_norm(
        _I(_is_bf16(out.dtype)), _ptr(y), _ptr(gate), _I(gate.stride(0)), _ptr(weight), _F(eps), _ptr(out), _I(n), _I(c),
        _I(n_parts), _I(n_heads), _I(GATES[gate_kind]), _I(1 if gate_first else 0), _ptr(nq), _ptr(floor), _F(floor_add),
        _ptr(skip), _ptr(skip_x), _I(skip_x.stride(0) if skip_x is not None else 0), _stream()), "gated_group_norm")


CONV_MAX_TAPS = 16


def causal_conv_silu(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], cu_q: torch.Tensor,
                     tok_seq: torch.Tensor, slots: torch.Tensor, state: torch.Tensor, offset: int, out: torch.Tensor,
                     activation: str = "silu", single: bool = False) -> None:
    """A causal convolution per channel over each sequence's tokens, then silu (`activation` "none": the convolution
    alone): out[t, c] = silu(b[c] + sum_j w[c, j] *
    x[t - (taps - 1 - j), c]); inputs before the step's first token come from `state` (the sequence's last taps - 1 inputs,
    float32 [taps - 1, C] at `offset`, zeros at a sequence's start), which then takes the step's last taps - 1 inputs.
    x: [T, C] in the activation dtype (rows may be strided); weight [C, taps], bias [C] float32; out [T, C].
    `single`: the caller's promise that every sequence of the step brings exactly one token; the state then moves inside
    the same kernel."""
    _rows("x", x)
    _dev("out", out, x.dtype)
    _dev("weight", weight, torch.float32)
    _is_bf16(x.dtype)
    n, c = x.shape
    taps = weight.shape[1]
    if weight.shape[0] != c or out.shape != (n, c) or not 1 <= taps <= CONV_MAX_TAPS:
        raise KernelError(f"causal_conv_silu: weight must be [C, taps <= {CONV_MAX_TAPS}], out [T, C]")
    if bias is not None:
        _dev("bias", bias, torch.float32)
        if bias.numel() != c:
            raise KernelError("causal_conv_silu: bias must hold one float32 per channel")
    _state(state, (offset, (taps - 1) * c))
    if activation not in ("silu", "none"):
        raise KernelError(f"causal_conv_silu: activation {activation!r} is not known ('silu' or 'none')")
    _check(library("recurrent").qf_causal_conv(
        _I(_is_bf16(x.dtype)), _ptr(x), _I(x.stride(0)), _ptr(weight), _ptr(bias), _ptr(cu_q), _ptr(tok_seq), _ptr(slots),
        _I(cu_q.numel() - 1), _ptr(state), _LL(state.stride(0)), _LL(offset), _I(taps), _I(n), _I(c), _ptr(out),
        _I(1 if activation == "none" else 0), _I(1 if single and n == cu_q.numel() - 1 else 0), _stream()), "causal_conv_silu")


def causal_conv(x, weight, bias, cu_q, tok_seq, slots, state, offset, out, single: bool = False) -> None:
    """`causal_conv_silu` without the activation."""
    causal_conv_silu(x, weight, bias, cu_q, tok_seq, slots, state, offset, out, activation="none", single=single)


# ---------------------------------------------------------------------------------------------------------------------
# Outputs that enter the stream under a factor each; norms over runs of columns; rows drawn towards another layer's
# (csrc/norm.cu)
def add_rms_norm_scaled(hidden: torch.Tensor, a: torch.Tensor, scale_a: float, b: Optional[torch.Tensor], scale_b: float,
                        weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """hidden += scale_a * a + scale_b * b (b may be None), float32; out = rmsnorm(hidden) * weight. hidden float32 [R, W]; a, b,
    weight and out share the activation dtype."""
    _dev("hidden", hidden, torch.float32)
    _dev("weight", weight)
    _dev("out", out, weight.dtype)
    rows, width = hidden.shape
    if weight.shape != (width,) or out.shape != hidden.shape:
        raise KernelError("add_rms_norm_scaled: shapes of weight/out do not match hidden")
    for name, t in (("a", a), ("b", b)):
        if t is not None:
            _dev(name, t, weight.dtype)
            if t.shape != hidden.shape:
                raise KernelError(f"add_rms_norm_scaled: {name} and hidden differ in shape")
    if a is None:
        raise KernelError("add_rms_norm_scaled: the first output is required")
    _check(library("norm").qf_add_scaled_rms_norm(_I(_is_bf16(weight.dtype)), _ptr(hidden), _ptr(a), _F(scale_a), _ptr(b), _F(scale_b),
                                                  _ptr(weight), _ptr(out), _I(rows), _I(width), _F(eps), _stream()), "add_rms_norm_scaled")


def residual_add_scaled(hidden: torch.Tensor, a: torch.Tensor, scale_a: float, b: Optional[torch.Tensor] = None,
                        scale_b: float = 0.0) -> None:
    """hidden (float32) += scale_a * a + scale_b * b, in place; b may be None."""
    _dev("hidden", hidden, torch.float32)
    _dev("a", a)
    if a.shape != hidden.shape or (b is not None and (b.shape != hidden.shape or b.dtype != a.dtype)):
        raise KernelError("residual_add_scaled: shapes or dtypes differ")
    if b is not None:
        _dev("b", b, a.dtype)
    _check(library("norm").qf_residual_add_scaled(_I(_is_bf16(a.dtype)), _ptr(hidden), _ptr(a), _F(scale_a), _ptr(b), _F(scale_b),
                                                  _LL(hidden.numel()), _stream()), "residual_add_scaled")


def rms_norm_cols(x: torch.Tensor, runs, eps: float) -> None:
    """RMS norms over runs of columns of x [T, C] (rows may be strided), in place, float32 inside. `runs`: one or two of
    (first column, width, count, weight [width]): x[:, c0:c0 + width] <- x / sqrt(sum(x^2) / count + eps) * weight; `count` is
    how many of the run's columns carry numbers (columns of padding hold zeros)."""
    _rows("x", x)
    _is_bf16(x.dtype)
    runs = list(runs)
    if not 1 <= len(runs) <= 2:
        raise KernelError("rms_norm_cols: one or two runs of columns")
    flat = []
    for col0, width, count, weight in runs:
        _dev("weight", weight, x.dtype)
        if col0 < 0 or width <= 0 or col0 + width > x.shape[1] or weight.numel() != width or not 0 < count <= width:
            raise KernelError("rms_norm_cols: a run must lie within the row, with one weight per column")
        flat += [_I(col0), _I(width), _I(count), _ptr(weight)]
    if len(runs) == 1:
        flat += [_I(0), _I(0), _I(0), _P(0)]
    _check(library("norm").qf_rms_norm_cols(_I(_is_bf16(x.dtype)), _ptr(x), _I(x.stride(0)), _I(x.shape[0]), _I(len(runs)), *flat,
                                            _F(eps), _stream()), "rms_norm_cols")


def mix_rows(x: torch.Tensor, other: torch.Tensor, heads: int, size: int, x_head: int, other_head: int, weight: float) -> None:
    """x[t, h * x_head + c] <- (1 - weight) * x[...] + weight * other[t, h * other_head + c] for c < size, in place, float32
    inside; x and other: [T, >= heads * head] views with unit inner stride, of one dtype."""
    _rows("x", x)
    _rows("other", other, x.dtype)
    _is_bf16(x.dtype)
    if x.shape[0] != other.shape[0] or size > min(x_head, other_head) or (heads - 1) * x_head + size > x.shape[1] \
            or (heads - 1) * other_head + size > other.shape[1]:
        raise KernelError("mix_rows: the heads do not fit the rows")
    _check(library("norm").qf_mix_rows(_I(_is_bf16(x.dtype)), _ptr(x), _I(x.stride(0)), _ptr(other), _I(other.stride(0)), _I(x.shape[0]),
                                       _I(heads), _I(size), _I(x_head), _I(other_head), _F(weight), _stream()), "mix_rows")


def bias_glu(gate_up: torch.Tensor, bias: Optional[torch.Tensor], kind: str, out: torch.Tensor) -> None:
    """out = act(gate + bias[:I]) * (up + bias[I:]) from the fused product gate_up [T, 2 I] (gate columns first); float32
    inside; bias [2 I] or None; kind as in `bias_act`."""
    _dev("gate_up", gate_up)
    _dev("out", out, gate_up.dtype)
    if kind not in ACTIVATIONS:
        raise KernelError(f"bias_glu: unknown activation {kind!r}; known: {', '.join(ACTIVATIONS)}")
    rows, inter = out.shape
    if gate_up.shape != (rows, 2 * inter):
        raise KernelError("bias_glu: gate_up must be [rows, 2 * width of out]")
    if bias is not None:
        _dev("bias", bias, gate_up.dtype)
        if bias.numel() != 2 * inter:
            raise KernelError("bias_glu: bias must hold one element per column of gate_up")
    _check(library("activation").qf_bias_glu(_I(_is_bf16(gate_up.dtype)), _ptr(gate_up), _ptr(bias), _ptr(out), _I(rows), _I(inter),
                                             _I(ACTIVATIONS[kind]), _stream()), "bias_glu")


# ---------------------------------------------------------------------------------------------------------------------
# Recurrences with a decay per row of the state (csrc/recurrent.cu)
def shift_mix(h: torch.Tensor, mu: torch.Tensor, cu_q: torch.Tensor, tok_seq: torch.Tensor, slots: torch.Tensor,
              state: torch.Tensor, offset: int, out: torch.Tensor, single: bool = False) -> None:
    """Token shift into several mixes: out[t, s * W:(s + 1) * W] = h_t + (h_(t-1) - h_t) * mu[s], float32 inside, h before a
    sequence's first token of the step being its kept row (float32 [W] at `offset` of the slot's state; zeros at a sequence's
    start), which then takes the sequence's last h. h: [T, W] (rows may be strided); mu: float32 [S, W]; out [T, S * W].
    `single`: the caller's promise that every sequence of the step brings exactly one token."""
    _rows("h", h)
    _dev("out", out, h.dtype)
    _dev("mu", mu, torch.float32)
    _is_bf16(h.dtype)
    n, width = h.shape
    if mu.dim() != 2 or mu.shape[1] != width or out.shape != (n, mu.shape[0] * width):
        raise KernelError("shift_mix: mu must be float32 [mixes, width], out [T, mixes * width]")
    _state(state, (offset, width))
    n_seqs = cu_q.numel() - 1
    _check(library("recurrent").qf_shift_mix(_I(_is_bf16(h.dtype)), _ptr(h), _I(h.stride(0)), _ptr(mu), _I(mu.shape[0]), _ptr(cu_q),
                                             _ptr(tok_seq), _ptr(slots), _I(n_seqs), _ptr(state), _LL(state.stride(0)), _LL(offset),
                                             _I(n), _I(width), _ptr(out), _I(1 if single and n == n_seqs else 0), _stream()), "shift_mix")


DECAYS = {"double_exp": 0, "sigmoid_root": 1}


def channel_decay(pre: torch.Tensor, bias: Optional[torch.Tensor], kind: str, out: torch.Tensor, tau: float = 1.0) -> None:
    """A decay per channel from float32 pre-activations [T, C] (rows may be strided) and a float32 bias [C]:
    "double_exp": exp(-exp(pre + bias));  "sigmoid_root": sigmoid(pre + bias)^(1 / tau). out float32 [T, C]."""
    _rows("pre", pre, torch.float32)
    _dev("out", out, torch.float32)
    if kind not in DECAYS or out.shape != pre.shape or tau <= 0:
        raise KernelError("channel_decay: kind is 'double_exp' or 'sigmoid_root', out has pre's shape, tau is positive")
    if bias is not None:
        _dev("bias", bias, torch.float32)
        if bias.numel() != pre.shape[1]:
            raise KernelError("channel_decay: bias must hold one float32 per channel")
    _check(library("recurrent").qf_channel_decay(_ptr(pre), _I(pre.stride(0)), _ptr(bias), _I(pre.shape[0]), _I(pre.shape[1]),
                                                 _I(DECAYS[kind]), _F(1.0 / tau), _ptr(out), _stream()), "channel_decay")


def outer_state_scan_rows(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, cu_q: torch.Tensor,
                          slots: torch.Tensor, state: torch.Tensor, s_offset: int, n_heads: int, dim: int, vdim: int,
                          q_scale: float, y: torch.Tensor, bonus: Optional[torch.Tensor] = None, decay_from=None) -> None:
    """The recurrence of a matrix state per head with a decay per row of the state, float32 inside:
        S <- diag(decay_t) S + k_t v_t^T,   y_t = S^T (q_scale q_t)                         (bonus None: read after the update)
        y_t = (S + diag(bonus) k_t v_t^T)^T (q_scale q_t),  then the same update            (bonus float32 [heads, dim])
    q, k: [T, heads * dim], v: [T, heads * vdim] in the activation dtype (rows may be strided); decay float32 [T, heads * dim];
    y float32 [T, heads * vdim]; S in `state` at s_offset as [heads, dim, vdim].
    `decay_from` = (kind, bias float32 [heads * dim], tau): `decay` holds the decays' pre-activations instead, and the kernel forms
    the decays on its way in, with the arithmetic of `channel_decay` (kind "double_exp" or "sigmoid_root")."""
    for name, t in (("q", q), ("k", k), ("v", v)):
        _rows(name, t, q.dtype)
    _is_bf16(q.dtype)
    n = q.shape[0]
    if q.shape[1] != n_heads * dim or k.shape != q.shape or v.shape != (n, n_heads * vdim):
        raise KernelError("outer_state_scan_rows: q, k must be [T, heads * dim], v [T, heads * vdim]")
    if dim > OUTER_STATE_MAX_DIM:
        raise KernelError(f"outer_state_scan_rows: a state of {dim} rows per head exceeds the kernel's {OUTER_STATE_MAX_DIM}")
    _dev("decay", decay, torch.float32)
    _dev("y", y, torch.float32)
    if decay.shape != (n, n_heads * dim) or y.shape != (n, n_heads * vdim):
        raise KernelError("outer_state_scan_rows: decay must be float32 [T, heads * dim], y float32 [T, heads * vdim]")
    if bonus is not None:
        _dev("bonus", bonus, torch.float32)
        if bonus.numel() != n_heads * dim:
            raise KernelError("outer_state_scan_rows: bonus must be float32 [heads, dim]")
    kind, decay_bias, inv_tau = 0, None, 1.0
    if decay_from is not None:
        name, decay_bias, tau = decay_from
        if name not in DECAYS or tau <= 0:
            raise KernelError("outer_state_scan_rows: decay_from names 'double_exp' or 'sigmoid_root' and a positive tau")
        _dev("decay bias", decay_bias, torch.float32)
        if decay_bias.numel() != n_heads * dim:
            raise KernelError("outer_state_scan_rows: the decays' bias must be float32 [heads * dim]")
        kind, inv_tau = DECAYS[name] + 1, 1.0 / tau
    _state(state, (s_offset, n_heads * dim * vdim))
    _check(library("recurrent").qf_outer_state_scan_rows(
        _I(_is_bf16(q.dtype)), _ptr(q), _I(q.stride(0)), _ptr(k), _I(k.stride(0)), _ptr(v), _I(v.stride(0)), _ptr(decay), _ptr(cu_q),
        _ptr(slots), _I(cu_q.numel() - 1), _ptr(state), _LL(state.stride(0)), _LL(s_offset), _I(n_heads), _I(n_heads), _I(dim),
        _I(vdim), _F(q_scale), _ptr(y), _ptr(bonus), _ptr(decay_bias), _I(kind), _F(inv_tau), _stream()), "outer_state_scan_rows")


def rows_prepare(x: torch.Tensor, runs, eps: float, mix=None) -> None:
    """What stands between a q | k | v product and the rotation where q and k are normed over whole rows, in place and in one
    launch. `runs`: up to three of (first column, width, count, bias or None, weight or None): the run gets its bias, then (with
    count > 0) the RMS norm x / sqrt(sum(x^2) / count + eps) * weight. `mix` = (run index, other [T, ...], heads' size, head pitch
    in x, head pitch in other, weight): that run, after its bias, is drawn towards `other` head by head,
    (1 - weight) * x + weight * other. Float32 inside; x [T, C] with unit inner stride."""
    _rows("x", x)
    _is_bf16(x.dtype)
    runs = list(runs)
    if not 1 <= len(runs) <= 3:
        raise KernelError("rows_prepare: one to three runs of columns")
    n = len(runs)
    col0, width, count = ((_I * n)(*[int(r[i]) for r in runs]) for i in range(3))
    for c0, w, cnt, bias, weight in runs:
        if c0 < 0 or w <= 0 or c0 + w > x.shape[1] or not 0 <= cnt <= w or (cnt > 0 and weight is None):
            raise KernelError("rows_prepare: a run must lie within the row; a norm needs its weight")
        for name, t in (("bias", bias), ("weight", weight)):
            if t is not None:
                _dev(name, t, x.dtype)
                if t.numel() != w:
                    raise KernelError(f"rows_prepare: {name} must hold one element per column of its run")
    biases = (_P * n)(*[(0 if r[3] is None else r[3].data_ptr()) for r in runs])
    weights = (_P * n)(*[(0 if r[4] is None else r[4].data_ptr()) for r in runs])
    mix_run, other, ldo, size, x_head, other_head, lam = -1, None, 0, 0, 1, 1, 0.0
    if mix is not None:
        mix_run, other, size, x_head, other_head, lam = mix
        _rows("other", other, x.dtype)
        heads = -(-runs[mix_run][1] // x_head)
        if other.shape[0] != x.shape[0] or size > min(x_head, other_head) or (heads - 1) * other_head + size > other.shape[1]:
            raise KernelError("rows_prepare: the heads of the mixed run do not fit the other rows")
        ldo = other.stride(0)
    _check(library("norm").qf_rows_prepare(_I(_is_bf16(x.dtype)), _ptr(x), _I(x.stride(0)), _I(x.shape[0]), _I(n), col0, width, count,
                                           biases, weights, _I(mix_run), _ptr(other), _I(ldo), _I(size), _I(x_head), _I(other_head),
                                           _F(lam), _F(eps), _stream()), "rows_prepare")
