"""Interfaces of the building parts of a decoder, and the registries they live in.

A model is an assembly of parts, chosen by its configuration layer by layer:

* a **mixer** moves information between the tokens of a request (attention here);
  it may own a cache entry: pages of keys and values, or a slot of fixed-size state;
* a **feed-forward** works on each token alone (dense SwiGLU here);
* a **norm** adds a sub-layer's output to the residual stream and normalises it;
* a **position encoding** tells a mixer (or the embedding) where a token stands;
* a **block** arranges a mixer, a feed-forward and their norms around the residual.

No part knows which model it is in: every size and constant is a field of the
part's *spec* (a dataclass with a ``kind``), and the checkpoint tensor names a part
reads are given to it by the architecture's builder.  ``register_part`` adds a new
kind without touching this package; ``build_part`` turns a spec into a part.

The reference has the same pieces as ``nn.Module`` classes tied to one config
(``emberserve/model/qwen2.py:30-164``); the packed ``[num_tokens, hidden]`` layout
and "the model never touches the cache" rule are kept (``emberserve/attn/base.py:4-15``).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

import torch

# ---------------------------------------------------------------------------------------
# parameters and where they come from


@dataclass(frozen=True)
class Source:
    """One checkpoint tensor that fills (a row range of) a parameter."""

    name: str
    rows: tuple[int, int] | None = None  # destination rows [lo, hi) along dim 0; None = all


@dataclass
class ParamSpec:
    shape: tuple[int, ...]
    sources: list[Source]
    # "float": kept in the compute dtype, except that a tensor stored in 32 bits stays
    # 32-bit; "int": an integer table, held as int32.
    role: str = "float"
    # How the random-weights mode fills it: "normal" (matrices and embeddings),
    # "bias" (normal with the bias deviation), "ones" (norm gains), "zeros".
    init: str = "normal"


# ---------------------------------------------------------------------------------------
# what a mixer needs from the cache manager


@dataclass(frozen=True)
class PagedKV:
    """Keys and values of every token, in pages.  `window`: only the last `window`
    keys are ever read again (None = all), so older pages may be given back.  `chunk`: a query
    reads only keys of its own chunk of `chunk` positions (chunks counted from position 0), so
    pages that lie wholly before the chunk of the next position may be given back.  `keep_first`:
    the keys of positions below it are read by every later query whatever window or chunk say, so
    the pages that hold them are never given back.  `v_head_dim`: numbers per value head where
    they differ from the key heads' (None = head_dim)."""

    num_kv_heads: int
    head_dim: int
    window: int | None = None
    chunk: int | None = None
    keep_first: int = 0
    v_head_dim: int | None = None

    paged = True

    @property
    def value_dim(self) -> int:
        return self.head_dim if self.v_head_dim is None else self.v_head_dim

    def elements_per_token(self) -> int:
        return self.num_kv_heads * (self.head_dim + self.value_dim)


@dataclass(frozen=True)
class PagedLatent:
    """ONE vector of `dim` numbers per token, in pages: what a latent-attention mixer keeps (the
    compressed key/value latent and the rotated key part that all heads share, side by side).
    `window` as for PagedKV."""

    dim: int
    window: int | None = None

    paged = True

    def elements_per_token(self) -> int:
        return self.dim


@dataclass(frozen=True)
class FixedState:
    """State of fixed size per request (a recurrent or convolutional mixer)."""

    shape: tuple[int, ...]
    dtype: str = "float32"

    paged = False


CacheNeed = PagedKV | PagedLatent | FixedState


@dataclass
class PagedKVHandle:
    """One cache entry of kind PagedKV as a mixer sees it during a step."""

    k: torch.Tensor  # [num_pages, num_kv_heads, page_size, head_dim]
    v: torch.Tensor  # [num_pages, num_kv_heads, page_size, value_dim]
    block_tables: torch.Tensor  # [rows, max_pages] int32, page ids of this entry's group
    page_size: int
    window: int | None
    write: bool  # False: read what another layer call wrote in this step
    chunk: int | None = None
    keep_first: int = 0


@dataclass
class PagedLatentHandle:
    """One cache entry of kind PagedLatent as a mixer sees it during a step."""

    pages: torch.Tensor  # [num_pages, page_size, dim]
    block_tables: torch.Tensor  # [rows, max_pages] int32, page ids of this entry's group
    page_size: int
    window: int | None
    write: bool


@dataclass
class FixedStateHandle:
    state: torch.Tensor  # [num_slots, *shape]
    slots: torch.Tensor  # [rows] int32 slot of each row of the step
    write: bool


# ---------------------------------------------------------------------------------------
# the step as parts see it


@dataclass
class StepContext:
    """Everything about one step that a part may read.  Rows are requests; tokens are
    packed ``[num_tokens, ...]`` in row order (``emberserve/attn/base.py:4-15``)."""

    num_tokens: int
    num_rows: int
    dtype: torch.dtype  # activation dtype: float32 or bfloat16
    device: torch.device
    # device tensors, int32
    tokens: torch.Tensor  # [num_tokens] token ids
    positions: torch.Tensor  # [num_tokens] absolute position of each token
    row_of_token: torch.Tensor  # [num_tokens]
    cu_q: torch.Tensor  # [num_rows + 1] first packed token of each row
    starts: torch.Tensor  # [num_rows] tokens already cached before this step
    # host copies
    q_lens: list[int]
    start_list: list[int]
    max_q_len: int = 1
    max_ctx_len: int = 1
    # scratch buffers that live across steps: scratch(name, shape, dtype) -> tensor
    scratch: Callable[..., torch.Tensor] | None = None
    extra: dict[str, Any] = field(default_factory=dict)
    # int32 device tokens that earlier kernels of the stream have sampled; a token id -(k + 1)
    # in `tokens` stands for deferred[k] (the engine launches a step before it has read the
    # tokens of the step before)
    deferred: torch.Tensor | None = None

    @property
    def all_decode(self) -> bool:
        return self.max_q_len == 1


# ---------------------------------------------------------------------------------------
# a norm split between the products on either side of it


@dataclass
class NormRequest:
    """What a block asks of the LAST product of a sub-layer when the norm behind the sub-layer
    can be begun there (steps of few rows, where every kernel saved is microseconds): add the
    product into `residual` instead of returning it, and hand back `ScaledRows` for the norm
    with this `gain` and `eps`.  A sub-layer that does not know about this ignores it."""

    residual: torch.Tensor  # [num_tokens, width] float32, updated in place
    gain: torch.Tensor  # [width]
    eps: float


@dataclass
class NormedDelta:
    """A sub-layer's output that has to pass a norm of its OWN before it joins the residual stream
    (a block with a norm behind each sub-layer as well as before it).  The norm that receives it
    (`Norm.forward`) applies `norm` to `x`, adds the result into the 32-bit residual and goes on
    with its own work, in one kernel; nothing of the intermediate is rounded."""

    x: torch.Tensor  # [num_tokens, width], activation dtype
    norm: "Norm"

    @property
    def shape(self):
        return self.x.shape

    @property
    def dtype(self):
        return self.x.dtype


@dataclass
class ScaledSum:
    """What a block leaves to be added to the residual stream when it is a weighted sum of several
    sub-layer outputs: ``sum_i scale_i * x_i``.  The norm kernel that receives it adds every term into the
    32-bit residual itself, so the sum is never rounded to the activation type.  `terms` holds at most
    three (tensor, scale) pairs."""

    terms: "list[tuple[torch.Tensor, float]]"

    def scaled(self, factor: float) -> "ScaledSum":
        return ScaledSum([(x, s * factor) for x, s in self.terms])

    @property
    def shape(self):
        return self.terms[0][0].shape

    @property
    def dtype(self):
        return self.terms[0][0].dtype


@dataclass
class ScaledRows:
    """Activations of a norm that is not finished yet: `x` holds residual * gain (activation
    dtype); row n still has to be multiplied by rsqrt(sumsq[:parts, n].sum() / width + eps).
    That factor is one number per row, so it commutes with a product x W^T: the product that
    reads `x` applies it to its result (`parts.linear`), and the norm costs no kernel of its own.
    `materialize()` finishes the norm the plain way for a reader that cannot."""

    x: torch.Tensor  # [num_tokens, width]
    sumsq: torch.Tensor  # [parts, 16] float32: shares of each row's sum of squares
    parts: int
    eps: float

    @property
    def shape(self):
        return self.x.shape

    @property
    def dtype(self):
        return self.x.dtype

    @property
    def is_cuda(self) -> bool:
        return self.x.is_cuda

    def materialize(self) -> torch.Tensor:
        n, width = self.x.shape
        total = self.sumsq[:self.parts, :n].sum(0)
        rstd = torch.rsqrt(total / width + self.eps)
        return (self.x.float() * rstd[:, None]).to(self.x.dtype)


# ---------------------------------------------------------------------------------------
# parts


class SharedParts:
    """Parts that several layers share (one rotary table for all of them): built once
    per distinct spec while a model is assembled."""

    def __init__(self) -> None:
        self._memo: dict[tuple[str, Any], Part] = {}

    def get(self, category: str, spec: Any) -> "Part":
        key = (category, spec)
        if key not in self._memo:
            self._memo[key] = build_part(category, spec, f"shared.{category}.{len(self._memo)}", self)
        return self._memo[key]

    def all(self) -> list["Part"]:
        return list(self._memo.values())


class Part:
    """Base of all parts.  `prefix` is the path of the part inside the model, used only
    to name its parameters in error messages and in the loader's table."""

    def __init__(self, spec: Any, prefix: str, shared: SharedParts | None = None) -> None:
        self.spec = spec
        self.prefix = prefix
        self.shared = shared if shared is not None else SharedParts()

    def param_specs(self) -> dict[str, ParamSpec]:
        """Local parameter name -> shape and checkpoint sources."""
        return {}

    def bind(self, params: dict[str, torch.Tensor]) -> None:
        """Receive the loaded parameters (device tensors), keyed by local name."""
        for name, tensor in params.items():
            setattr(self, name, tensor)

    def children(self) -> dict[str, "Part"]:
        return {}

    def streamed_params(self) -> list[str]:
        """Local names of the weight matrices that `forward` hands to ``parts.linear`` in steps of few
        rows, where every weight is read once per step: the engine may keep a second, tiled copy of
        these for the weight-streaming kernels (``parts.linear.give_tiled_twin``).  Naming none is
        always right."""
        return []

    def scratch_elements_per_token(self) -> int:
        """Elements of the activation dtype that `forward` asks of ``ctx.scratch`` per token of a
        step, children not counted.  Only used to keep memory free for the steps when the
        cache is sized; a part that allocates by other means may leave it at 0 (small
        allocations are covered by a fixed workspace)."""
        return 0


class Norm(Part):
    def normalize_stream(self, residual: torch.Tensor, ctx: "StepContext") -> None:
        """Norm the 32-bit stream itself, in place (a norm that stands behind the embedding)."""
        raise NotImplementedError(f"{type(self).__name__} cannot norm the stream in place")

    def split_request(self, residual: torch.Tensor, ctx: StepContext) -> "NormRequest | None":
        """A `NormRequest` if, in this step, the norm can be begun by the product before it and
        finished by the product behind it (then `forward` will be handed the `ScaledRows` that
        came of it as `delta`, and passes them on); None (the default) if it is a kernel of its own."""
        return None

    def forward(self, delta: torch.Tensor | None, residual: torch.Tensor,
                ctx: StepContext, rows: torch.Tensor | None = None) -> torch.Tensor:
        """residual += delta (32-bit sum); return norm(residual) in the activation dtype.
        With `rows` (int32 packed token indices on the device; their count is ``rows.numel()``)
        only the rows ``residual[rows] + delta[rows]`` are normalised and returned, compactly,
        and the residual is left unchanged: that is how the decoder calls the final norm, on
        the rows whose logits are wanted."""
        raise NotImplementedError


class PositionEncoding(Part):
    """How positions reach the model.  A rotary kind returns its table; an absolute
    kind would add to the embedding in `on_embedding`."""

    def rotary(self, device: torch.device) -> tuple[torch.Tensor, int] | None:
        """(cos/sin table ``[max_pos, rotary_dim/2, 2]`` float32, rotary_dim) or None."""
        return None

    def on_embedding(self, hidden: torch.Tensor, ctx: StepContext) -> None:
        return None

    @property
    def max_positions(self) -> int | None:
        return None


class Mixer(Part):
    # True if `forward` takes `ScaledRows` for x (its first product finishes the norm) and looks
    # for a `NormRequest` in ctx.extra["norm_behind"] (its last product begins the next norm,
    # and `forward` then returns `ScaledRows`).  False: plain tensors in and out.
    splits_norms = False

    def cache_need(self) -> CacheNeed | None:
        return None

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: Any) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    splits_norms = False  # as for Mixer

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError


class StreamPart(Part):
    """Something that acts on the residual stream itself, behind a layer's sub-layers (a block lists
    such parts in its spec and runs them in order): an input of the layer's own that is added to the
    stream, a mix of the stream's states at several depths."""

    def on_entry(self, residual: torch.Tensor, ctx: StepContext) -> None:
        """Called before the block's first sub-layer, with the stream as the block receives it."""
        return None

    def forward(self, delta: Any, residual: torch.Tensor, ctx: StepContext) -> Any:
        """`delta` is what the block's last sub-layer (or the stream part before this one) left to be
        added to the stream: None, a tensor or a `NormedDelta`.  Returns what is still to be added
        (None once everything is in `residual`)."""
        raise NotImplementedError


class Block(Part):
    """Arrangement of a mixer, a feed-forward and their norms.  Works on the pair
    (delta, residual): `delta` is the previous sub-layer's output that has not been
    added to the 32-bit residual stream yet (None right after the embedding)."""

    def cache_need(self) -> "CacheNeed | tuple[CacheNeed, ...] | None":
        """What one call of the block keeps between steps: one need, or a tuple of needs (pages of
        a mixer beside the fixed-size state of a convolution, say); `forward` is then handed a
        tuple of handles in the same order, and the layer call names a tuple of cache entries."""
        raise NotImplementedError

    def entry_norm(self) -> "Norm | None":
        """The norm that receives what the block is given, if the sub-layer behind that norm takes
        `ScaledRows`: the block BEFORE this one may then let its last product begin that norm
        (the decoder tells it through ctx.extra["next_norm"]).  None: hand me a plain delta."""
        return None

    def forward(self, delta: torch.Tensor | None, residual: torch.Tensor, ctx: StepContext,
                cache: Any) -> torch.Tensor:
        """Returns the new delta; `residual` is updated in place."""
        raise NotImplementedError


# ---------------------------------------------------------------------------------------
# registries: spec kind -> part class

_CATEGORIES = ("mixer", "feed_forward", "norm", "position", "block", "conv", "stream")
_REGISTRY: dict[str, dict[str, type[Part]]] = {c: {} for c in _CATEGORIES}


def register_part(category: str, kind: str, cls: type[Part] | None = None):
    """Register `cls` as the part built for specs of `kind` in `category` (one of
    mixer, feed_forward, norm, position, block, conv, stream).  Usable as a decorator."""
    if category not in _REGISTRY:
        raise KeyError(f"unknown part category {category!r}; one of {_CATEGORIES}")

    def deco(c: type[Part]) -> type[Part]:
        _REGISTRY[category][kind] = c
        return c

    return deco if cls is None else deco(cls)


def build_part(category: str, spec: Any, prefix: str, shared: SharedParts | None = None) -> Part:
    kind = getattr(spec, "kind", None)
    try:
        cls = _REGISTRY[category][kind]
    except KeyError:
        known = sorted(_REGISTRY.get(category, {}))
        raise KeyError(f"no {category} part of kind {kind!r} is registered "
                       f"(known: {known})") from None
    return cls(spec, prefix, shared)


def registered_kinds(category: str) -> list[str]:
    return sorted(_REGISTRY[category])
