"""Interfaces of the parts a layer is put together from.

A part is built from a `PartSpec` alone: its sizes and constants are the spec's `params`,
the tensors it owns are named by the spec's `tensors`. No part knows which model it is in,
which layer it is, or what the other parts of its layer are.

Life of a part:
  1. `Part(spec)`           metadata only, no device memory
  2. `tensor_specs()`       what it wants from the weight files (name, shape, how to draw it at random)
  3. `kernel_libraries(dt)` which kernel libraries it will call for activation dtype `dt`
  4. `bind(tensors, dt, device)`  take its tensors (already on the device and in their kept dtype) and
                            arrange them as its kernels want them (fused, concatenated)
  5. `forward(...)`         per step

Interfaces by role (T = tokens of the step, W = model width):
  Norm           forward(hidden f32 [T, W] (updated in place), delta [T, W] | None) -> normed [T, W]
                 computes hidden += delta, then normalises.
  Mixer          cache_need() -> KvNeed | StateNeed | None
                 forward(x [T, W], ctx, site, writes_cache) -> delta [T, W]
                 `site` is the cache view of the schedule entry being run (or of the entry it
                 reads from when `writes_cache` is false).
  FeedForward    forward(x [T, W], ctx) -> delta [T, W]
  PositionEncoding
                 fused_rotary() -> (inv_freq f32 [R/2], R) | None   what a mixer's fused kernel may apply itself
                 apply(q [T, NH, D], k [T, KVH, D], ctx) -> None    in place, when there is no fused form
  Block          forward(hidden, delta, ctx, site, writes_cache) -> delta
                 arranges norms, mixer and feed-forward around the residual stream `hidden`.
Mixers and feed-forwards may also offer a form for steps of a few tokens that works on the stream in place
(`fused_takes`, `fused_forward`): it adds the pending delta of the part before, applies the preceding RMSNorm in its own
first kernel and adds its result to `hidden`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Mapping, Optional

import torch

from ..config.spec import PartSpec


@dataclass(frozen=True)
class TensorSpec:
    """One tensor of the weight files.

    init  how the random-weights mode draws it: "matrix" N(0, 0.02), "bias" N(0, 0.02), "norm" 1 + N(0, 0.1),
          "logit" N(0, 1), "conv" (1 + N(0, 0.5)) / sqrt(taps), "fraction" sigmoid(N(0, 1)), "rate" N(-1, 1),
          "low_rank" N(0, 0.5)
    shape an extent of -1 takes whatever size the file holds (the part reads it from the tensor it is bound to)
    keep  "compute": kept in the activation dtype (bfloat16, or float32 on the 32-bit path)
          "stored":  kept as the file stores it if that is a 32-bit float, else as "compute"
          "int32":   an integer table, kept as int32
          "float32": kept as float32 in both precisions
    fallback  another tensor name that stands in when the files do not hold `name` (a head that
              shares the embedding table in files that say nothing about tying)
    """
    name: str
    shape: tuple
    init: str = "matrix"
    keep: str = "compute"
    fallback: Optional[str] = None


class Part:
    kind = ""
    # False for a part whose forward needs the step's host-side lists (ctx.host_*): a model with such a part
    # decodes step by step instead of replaying captured graphs
    graph_safe = True

    def __init__(self, spec: PartSpec):
        self.spec = spec
        self.params = dict(spec.params)

    def file_name(self, logical: str) -> str:
        try:
            return self.spec.tensors[logical]
        except KeyError:
            raise KeyError(f"part {self.kind!r}: its spec names no tensor for {logical!r}") from None

    def tensor_specs(self) -> list[TensorSpec]:
        return []

    def kernel_libraries(self, dtype: torch.dtype) -> set[str]:
        return set()

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype: torch.dtype, device) -> None:
        pass

    def sub_parts(self) -> list["Part"]:
        return []

    def step_weights(self) -> list:
        """The bound tensors that every step reads in full (for the measurement's byte counts); tables that a step
        only gathers rows from are not among them."""
        return []


# ---- two chains of kernels side by side. A step of few rows is a chain of short dependent kernels; where a part has two
# chains that do not depend on each other (two mixers on one input, a shared expert beside the routed ones) the second runs on
# a stream of its own: `fork` makes it wait for the step's stream, `join` makes the step's stream wait for it. A capture of
# the step's stream takes both with it. Long steps fill the GPU with either chain and gain nothing.
SIDE_BY_SIDE_MAX_ROWS = 64
_side_streams: dict = {}


def runs_side_by_side(x: torch.Tensor) -> bool:
    """Whether a part with two independent chains should put the second on the side stream for this step's input."""
    return x.is_cuda and x.shape[0] <= SIDE_BY_SIDE_MAX_ROWS


def fork(x: torch.Tensor):
    """(the current stream, a side stream), the side stream waiting for what the current stream has issued so far. `x`, which
    the side stream will read, is marked as in use there. A part that already runs on a side stream gets the next one of the
    device's pool, so chains may fork inside chains."""
    index = x.device.index if x.device.index is not None else torch.cuda.current_device()
    pool = _side_streams.setdefault(index, [])
    main = torch.cuda.current_stream(x.device)
    depth = next((i + 1 for i, s in enumerate(pool) if s == main), 0)
    while len(pool) <= depth:
        pool.append(torch.cuda.Stream(device=index))
    side = pool[depth]
    event = torch.cuda.Event()
    event.record(main)
    side.wait_event(event)
    x.record_stream(side)
    return main, side


def join(main, side, *made_on_side) -> None:
    """The step's stream waits for the side stream; tensors made there and read from here on are marked as in use here."""
    event = torch.cuda.Event()
    event.record(side)
    main.wait_event(event)
    for t in made_on_side:
        if t is not None:
            t.record_stream(main)


class Pending:
    """What a block may leave in the place of a plain pending output: something that still has to reach the residual
    stream and knows how (`add_to`). A block that can fold it into its own first kernel names its class in
    `accepts_pending`; for every other block, and at the end of the schedule, the model calls `add_to` itself."""

    def add_to(self, hidden: torch.Tensor) -> None:
        raise NotImplementedError

    def value(self) -> torch.Tensor:
        """The float32 tensor that will be added (for diagnosis; not on the product path)."""
        raise NotImplementedError


class PendingPair(Pending):
    """The outputs of two sublayers that read the same input (a parallel layer): their sum goes into the stream, summed
    with each other first. Either may be None."""
    __slots__ = ("a", "b")

    def __init__(self, a, b=None):
        self.a, self.b = a, b

    def add_to(self, hidden: torch.Tensor) -> None:
        from .. import ops
        ops.residual_add_pair(hidden, self.a, self.b)

    def value(self) -> torch.Tensor:
        parts = [t.to(torch.float32) for t in (self.a, self.b) if t is not None]
        return parts[0] + parts[1] if len(parts) == 2 else parts[0]


class PendingScaled(Pending):
    """One or two sublayer outputs that enter the stream under a factor each: hidden += scale_a * a + scale_b * b (float32).
    What a block with a residual multiplier leaves pending, and what two mixers that run side by side hand to their block."""
    __slots__ = ("a", "scale_a", "b", "scale_b")

    def __init__(self, a, scale_a: float, b=None, scale_b: float = 0.0):
        self.a, self.scale_a, self.b, self.scale_b = a, float(scale_a), b, float(scale_b)

    @staticmethod
    def of(output, factor: float) -> "PendingScaled":
        """A mixer's or feed-forward's output (a tensor, or already a scaled pair) under one more factor."""
        if isinstance(output, PendingScaled):
            return PendingScaled(output.a, output.scale_a * factor, output.b, output.scale_b * factor)
        return PendingScaled(output, factor)

    def add_to(self, hidden: torch.Tensor) -> None:
        from .. import ops
        ops.residual_add_scaled(hidden, self.a, self.scale_a, self.b, self.scale_b)

    def value(self) -> torch.Tensor:
        out = self.a.to(torch.float32) * self.scale_a
        return out if self.b is None else out + self.b.to(torch.float32) * self.scale_b


class PendingNormed(Pending):
    """A sublayer's output that still has to be normalised (RMS, weight, eps) and added to the residual stream: what a
    block with norms after its sublayers hands to whoever runs next, so that the addition rides on that part's first norm
    kernel (`ops.sandwich_norm`). The model resolves it itself before anything that only knows plain deltas."""
    __slots__ = ("y", "weight", "eps", "rows")

    def __init__(self, y, weight: torch.Tensor, eps: float):
        """y: the sublayer's output [T, W], or a `RowSum` whose rows are still to be summed per token."""
        self.rows = y if isinstance(y, RowSum) else None
        self.y = y.rows if isinstance(y, RowSum) else y
        self.weight, self.eps = weight, eps

    def into(self, hidden: torch.Tensor, next_weight=None, next_eps: float = 0.0, out=None) -> None:
        """hidden += norm(y); and, with `next_weight`, out = the next norm of the stream, in the same kernel."""
        from .. import ops
        r = self.rows
        ops.sandwich_norm(hidden, self.y, self.weight, self.eps, next_weight, next_eps, out,
                          dest=None if r is None else r.dest, top=1 if r is None else r.top,
                          row_weight=None if r is None else r.row_weight)

    def add_to(self, hidden: torch.Tensor) -> None:
        self.into(hidden)

    def value(self) -> torch.Tensor:
        """The float32 tensor that will be added (for diagnosis; not on the product path)."""
        y = self.y.to(torch.float32)
        if self.rows is not None:
            r = self.rows
            if r.row_weight is not None:
                y = y * r.row_weight[:, None]
            y = y[r.dest.long()].view(-1, r.top, y.shape[1]).sum(1)
        return y * torch.rsqrt(y.square().mean(-1, keepdim=True) + self.eps) * self.weight.to(torch.float32)


class RowSum:
    """A sublayer's output that is not stored per token: token t's row is the sum of the `top` rows rows[dest[t * top + k]]
    (each times row_weight[that row], if given). A feed-forward with routed experts hands this to a block that can take it
    (`forward_rows`), so that the sum rides on the kernel that reads the output next."""
    __slots__ = ("rows", "dest", "top", "row_weight")

    def __init__(self, rows: torch.Tensor, dest: torch.Tensor, top: int, row_weight=None):
        self.rows, self.dest, self.top, self.row_weight = rows, dest, top, row_weight


class Embedding(Part):
    def forward(self, token_ids: torch.Tensor, ctx) -> torch.Tensor:
        """The float32 residual stream [T, width] of the step's token ids."""
        raise NotImplementedError

    def lookup_table(self):
        """The table [vocab, width] if this embedding is a plain row lookup (row id -> stream row, nothing added or
        scaled), which the kernel that advances a decode graph's state may then do for the next step; else None."""
        return None


class Norm(Part):
    def forward(self, hidden: torch.Tensor, delta: Optional[torch.Tensor]) -> torch.Tensor:
        raise NotImplementedError

    def fused_rms(self):
        """(weight, eps) if this norm is a plain RMSNorm that a following kernel may apply in its prologue, else None."""
        return None


class Mixer(Part):
    def cache_need(self):
        return None

    def forward(self, x: torch.Tensor, ctx, site, writes_cache: bool) -> torch.Tensor:
        raise NotImplementedError

    # Optional fast form for steps of a few tokens: the part adds the pending `delta` (if any) to the residual stream,
    # applies the preceding RMSNorm itself and adds its output to the stream in place
    # (hidden += delta; hidden += mixer(rmsnorm(hidden))). A block uses it when `fused_takes(ctx)` is true and its norm
    # has a `fused_rms()` form.
    def fused_takes(self, ctx) -> bool:
        return False

    def fused_forward(self, hidden: torch.Tensor, rms, ctx, site, writes_cache: bool, delta=None) -> None:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError

    def fused_takes(self, ctx) -> bool:
        return False

    def fused_forward(self, hidden: torch.Tensor, rms, ctx, delta=None) -> None:
        raise NotImplementedError


class PositionEncoding(Part):
    def fused_rotary(self):
        return None

    def apply(self, q: torch.Tensor, k: torch.Tensor, ctx) -> None:
        raise NotImplementedError
