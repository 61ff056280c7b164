"""Interfaces of the parts a layer is put together from.

A part is built from a `PartSpec` (its kind and all of its sizes and
constants), declares the tensors it wants by name, receives them in `bind()`
and then runs on the packed tokens of a step.  Parts never see the model
they are in: what they need of a step arrives in the `StepContext`.

Interfaces (all token tensors are packed `[tokens, width]`):
  Norm.forward(x float32, out_dtype, rows=None) -> normed rows
  Mixer.forward(x, ctx, residual)        adds its output into `residual`
  FeedForward.forward(x, ctx, residual)  adds its output into `residual`
  PositionEncoding.encode_and_store(...) turns projected q/k/v into encoded q
                                         and appends k/v to the cache
  Block.forward(h, ctx)                  runs its parts on the residual stream
`residual` is the float32 residual stream; adding into it lets the last
matrix product of a part do the residual sum in float32 in its epilogue.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

import torch

from ..cache import KVLayerView, KVRequest, StateRequest
from ..config import PartSpec


@dataclass(frozen=True)
class WeightSpec:
    """A tensor a part expects.  `role` picks the random-init rule and says
    how the tensor is used: 'matrix' and 'embedding' are operands of matrix
    products and keep their stored precision; 'bias' and 'norm_scale' are
    widened to float32 when bound."""
    name: str
    shape: tuple[int, ...]
    role: str


@dataclass
class Runtime:
    """What the engine tells every part: where it runs, the activation dtype
    (bfloat16 for serving, float32 for the all-32-bit path) and the longest
    sequence it will be asked to handle."""
    device: torch.device
    act_dtype: torch.dtype
    max_context: int
    sm_count: int = 0                 # streaming multiprocessors of the device (the engine fills it in)
    window_chunk: int = 64            # tokens a windowed layer accepts in one step that continues a sequence

    def __post_init__(self):
        if not self.sm_count and self.device.type == "cuda" and torch.cuda.is_available():
            self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count


@dataclass
class StepBatch:
    """The packed, ragged batch of one step, on the device (int32 tensors),
    with host copies of what the host needs for planning."""
    n_tokens: int
    n_seqs: int
    tokens: torch.Tensor          # [T] token ids
    tok_seq: torch.Tensor         # [T] row of the step each token belongs to
    tok_pos: torch.Tensor         # [T] absolute position of each token in its sequence
    cu_seqlens: torch.Tensor      # [B+1] first token of each row
    slots: torch.Tensor           # [B] cache slot of each row
    start_pos: torch.Tensor       # [B] tokens cached before this step
    new_lens: torch.Tensor        # [B] tokens cached after this step
    logit_rows: torch.Tensor      # [R] token indices whose logits are wanted
    n_logit_rows: int
    block_tables: list[tuple[torch.Tensor, int]]   # per cache group: (int32 [B, width], width)
    host_slots: list[int] = field(default_factory=list)
    host_start: list[int] = field(default_factory=list)
    host_lens: list[int] = field(default_factory=list)      # tokens each row brings
    packed_bytes: int = 0                                    # size of the one host-to-device copy
    plan_max_len: int = 0      # if > 0: the length to plan for instead of this step's own (replayed graphs)
    tok_src: Optional[torch.Tensor] = None    # [T] row of the sampler's last ids that holds the token, or -1
    any_source: bool = False                  # some token comes from the sampler's ids on the device

    @property
    def all_from_zero(self) -> bool:
        return all(s == 0 for s in self.host_start)

    @property
    def single_tokens(self) -> bool:
        return all(n == 1 for n in self.host_lens)

    @property
    def max_new_len(self) -> int:
        """Longest sequence after this step, for planning (grids, splits)."""
        if self.plan_max_len > 0:
            return self.plan_max_len
        return max(s + n for s, n in zip(self.host_start, self.host_lens))


@dataclass
class StepContext:
    batch: StepBatch
    runtime: Runtime
    entry: int                              # index of the running schedule entry
    kv: Optional[KVLayerView] = None        # cache of this entry (or of the entry it reads)
    state: Optional[torch.Tensor] = None    # [max_slots, *shape] state of this entry, indexed by slot


class Part:
    """Base of all parts."""

    # A part whose step needs the host (reads device data back, branches on
    # it) sets this to False; the engine then launches that model's decode
    # steps kernel by kernel instead of replaying a captured CUDA graph.
    graph_capturable = True
    # A step may carry rows beyond a sequence's real tokens (a prompt padded to the size of a captured graph; the
    # batch's new_lens holds the real length).  A part that says True treats rows independently, or — a mixer —
    # lets no real row see a padded one and writes nothing lasting for padded rows.  The engine pads only if
    # every part of the model says so.
    padded_rows_ok = False
    # A mixer or feed-forward that hands its input to `kernels.linear` and reads it nowhere else may set this:
    # the block then passes the norm before it as a `kernels.PendingNorm`, which the product can fold in.
    takes_pending_norm = False

    def __init__(self, spec: PartSpec):
        self.spec = spec
        self.prefix = spec.weights_prefix
        self.params: dict[str, Any] = spec.params

    def weight_specs(self) -> list[WeightSpec]:
        return []

    def ignored_weights(self) -> list[str]:
        """Tensor names that may be present in a checkpoint without being used."""
        return []

    def bind(self, tensors: dict[str, torch.Tensor], runtime: Runtime, shared: Optional[dict] = None) -> None:
        """Takes the loaded tensors (on the device) this part declared.
        `shared` is a dict that lives for one model build; parts may keep
        tables there that several layers use (position tables)."""


class Norm(Part):
    def forward(self, x: torch.Tensor, out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError


class Mixer(Part):
    def cache_request(self) -> Optional[KVRequest]:
        return None

    def state_request(self) -> Optional[StateRequest]:
        return None

    def check_step(self, start_pos: list[int], step_lens: list[int], owns_cache: bool) -> None:
        """Raises (before anything is launched) if the mixer cannot run the step."""

    def forward(self, x: torch.Tensor, ctx: StepContext, residual: torch.Tensor) -> None:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx: StepContext, residual: torch.Tensor) -> None:
        raise NotImplementedError


class PositionEncoding(Part):
    def prepare(self, runtime: Runtime) -> None:
        """Builds tables for positions 0 .. runtime.max_context - 1."""

    def encode_and_store(self, qkv: torch.Tensor, bias: Optional[torch.Tensor], ctx: StepContext, *, n_heads: int,
                         n_kv_heads: int, head_dim: int, q_out: torch.Tensor, k_out: Optional[torch.Tensor],
                         v_out: Optional[torch.Tensor]) -> None:
        raise NotImplementedError


def float32_vector(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.float32).contiguous()
