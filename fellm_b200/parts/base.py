"""Interfaces of the parts a layer is made of, and the registries that map a PartSpec.kind to
the class that builds it.

FeLLM marks the same seams with enums: `MixKind::{Attention, ShortConv, ...}`
(crates/fellm-model/src/probe.rs:36-56), the FFN kind next to it, and, for what a mixer keeps
between steps, `KvGroupKind::{FullAttention, SlidingWindow, Recurrent}`
(crates/fellm-runtime/src/kv_fabric/types.rs:101-111) plus `mutable_state_input_count`
(crates/fellm-runtime/src/compiled.rs:815-823).

No part knows which model it is in: a part gets its sizes and constants as constructor
arguments, its tensors by the local names it declares, and at run time a StepContext (who is in
the batch, at which positions) and a view of its own cache.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

# ----------------------------------------------------------------------------- parameters


@dataclass(frozen=True)
class ParamDecl:
    """A tensor a part owns.  role 'matrix': kept in the engine's dtype (bfloat16, or float32
    when the file stores 32-bit or the engine runs in 32-bit); 'vector': norm weights, conv taps
    and biases, always promoted to float32 (plugins/dspark/src/checkpoint.rs:154-169 promotes
    rank-1 tensors the same way); 'table': integer tables, int32.
    `init`: ('normal', std) | ('ones',) | ('const', value) | ('uniform', low, high) for the random-weights mode.
    `also`: other shapes of the same element count that a file may use.
    An extent of -1 in `shape` is read from the file (the rank of a low-rank projection, which no
    configuration key names); `fallback` is then the shape the random-weights mode makes."""
    shape: Tuple[int, ...]
    role: str = "matrix"
    init: Tuple = ("normal", 0.02)
    also: Tuple[Tuple[int, ...], ...] = ()
    fallback: Optional[Tuple[int, ...]] = None

    def fits(self, shape) -> bool:
        shape = tuple(shape)
        if shape in self.also:
            return True
        return len(shape) == len(self.shape) and all(w == -1 or w == h for w, h in zip(self.shape, shape))

    def made_shape(self) -> Tuple[int, ...]:
        """The shape the random-weights mode gives the tensor."""
        if -1 not in self.shape:
            return self.shape
        if self.fallback is None:
            raise ValueError(f"a tensor of shape {self.shape} needs a fallback shape to be made at random")
        return self.fallback


# ----------------------------------------------------------------------------- cache needs


@dataclass(frozen=True)
class PagedKV:
    """Keys and values per token: `kv_heads * head_dim` each.  `window` = how many of the
    latest positions a query reads (None: all of them).  `chunk`: a query reads only keys of its
    own block of `chunk` positions, counted from position 0 (None: no such blocks).  `v_dim`: the
    size of a value where it differs from a key's (None: head_dim); a page-layer record is then the
    keys [kv_heads][page_tokens][head_dim] followed by the values [kv_heads][page_tokens][v_dim].
    `values_are_keys`: the layer reads its keys as its values too; a record holds the keys alone."""
    kv_heads: int
    head_dim: int
    window: Optional[int] = None
    chunk: Optional[int] = None
    v_dim: Optional[int] = None
    values_are_keys: bool = False

    @property
    def value_dim(self) -> int:
        """What a record keeps of a value per head and token (0: nothing beside the key)."""
        if self.values_are_keys:
            return 0
        return self.head_dim if self.v_dim is None else self.v_dim


@dataclass(frozen=True)
class FixedState:
    """State of fixed size per request, float32, zero when a request starts."""
    shape: Tuple[int, ...]


# ----------------------------------------------------------------------------- parts


class Part:
    """Base of every part.  Subclasses fill `self.decls` in __init__, get `self.w[local]`
    tensors from bind(), and may repack them in prepare()."""

    def __init__(self):
        self.decls: Dict[str, ParamDecl] = {}
        self.w: Dict[str, torch.Tensor] = {}

    def param_decls(self) -> Dict[str, ParamDecl]:
        return self.decls

    def bind(self, tensors: Dict[str, torch.Tensor]):
        self.w = dict(tensors)
        self.prepare()

    def prepare(self):
        """Called once after bind(): repack or fuse weights for the kernels."""

    def weight_order(self):
        """The part's matrices in the order its forward() reads them (for the engine's chain of weights:
        each product asks the L2 for the matrix of the product after it)."""
        return []

    def reserve(self, device, max_rows: int, n_ctx: int):
        """Called once by the engine, after bind() and before the first step: allocate here what
        the part's kernels need besides inputs and outputs, sized for steps of up to max_rows rows
        and contexts of up to n_ctx (so that nothing grows under a captured CUDA graph)."""

    def kernel_modules(self, dtype: str):
        """[(module name, defines)] of the CUDA modules this part launches in `dtype`, so that
        they can be compiled before the first step."""
        return []

    def children(self):
        """Parts this part is made of that own tensors of their own (each built from a PartSpec): the
        model binds, reserves and compiles for them as for the parts of a block."""
        return []


class Norm(Part):
    def forward(self, x: torch.Tensor, out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None):
        """x: float32 [T, size] (the residual stream).  Returns [T or len(rows), size] in
        out_dtype; `rows` (int32, device) picks rows of x."""
        raise NotImplementedError

    def expect(self, x: torch.Tensor):
        """A block says, before a part adds into the residual rows x: this norm reads x next.  A norm
        whose work the adding product can do on the way (RMSNorm in a decode step) arranges that here;
        nothing has to happen."""


class PositionEncoding(Part):
    """What an attention mixer needs to place queries and keys: for rotary encodings the
    inverse-frequency table and the pairing; for none, nothing."""
    kind = "none"


class Mixer(Part):
    def cache_need(self):
        """What the mixer keeps between steps: PagedKV, FixedState, None, or a list of those when
        it keeps several things (pages and a state, or two states of different shapes); `cache` in
        forward() is then a list of views in the same order."""
        return None

    def private_need(self):
        """What the mixer keeps of its OWN even where its schedule entry reads another entry's cache (Run.cache_of): None,
        or needs as cache_need() gives them.  forward() then gets `cache` = (views of these, the other entry's views)."""
        return None

    def forward(self, xn: torch.Tensor, ctx, cache, out: torch.Tensor, reads_only: bool = False):
        """xn: [T, d] normed input in the engine's dtype; `out`: float32 [T, d] residual stream,
        to which the mixer ADDS its result in place.  `cache` is this run's view of its cache
        group (PagedView / StateView / None; a list of views when cache_need() returned a list).  `reads_only`: the cache belongs to an earlier run;
        read it, write nothing."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, hn: torch.Tensor, ctx, out: torch.Tensor):
        """hn: [T, d] normed input; ADDS its result to the float32 residual stream `out`."""
        raise NotImplementedError


class Connector(Part):
    """Rewrites the residual stream between two blocks (e.g. where a looped run of layers starts a
    pass): forward(x, x0, step) returns the new float32 [T, d] stream; x0 is the embedding's output,
    `step` the number of the pass.  needs_embedding = False: the connector never reads x0 (the model then keeps no
    copy of the embedding's output)."""
    needs_embedding = True

    def forward(self, x: torch.Tensor, x0: torch.Tensor, step: int, act_dtype: torch.dtype) -> torch.Tensor:
        raise NotImplementedError


class ResidualGate(Part):
    """Gates on what a block's sublayers add to the residual stream, computed from the sublayers' input."""

    def logits(self, h: torch.Tensor) -> torch.Tensor:
        """h [T, d], the sublayers' input -> float32 [T, n d], the gates' logits of the n sublayers side by side."""
        raise NotImplementedError

    def add(self, x: torch.Tensor, results, zg: torch.Tensor) -> torch.Tensor:
        """x float32 [T, d] += the sublayers' float32 results, each through its gate."""
        raise NotImplementedError


class SideInput(Part):
    """Something a token adds to the residual stream by itself after a block (read from the step's token ids, not from
    other tokens): forward(x, ctx) updates the float32 rows x in place.  `uses_shared`: the tensor name of a shared
    part of the model (ModelSpec.shared) that attach() is handed once, after every part is bound."""
    uses_shared = None
    takes_gated_add = False       # True: forward(x, ctx, pending=(results, logits)) first adds what ResidualGate.add would

    def attach(self, shared: "Shared"):
        pass

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError


class Shared(Part):
    """A part that owns tensors several other parts read (a table with a slice per layer)."""


class Embedding(Part):
    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        """tokens int32 [T] -> float32 [T, d]."""
        raise NotImplementedError


class Head(Part):
    def forward(self, xf: torch.Tensor) -> torch.Tensor:
        """xf [W, d] normed -> float32 logits [W, vocab]."""
        raise NotImplementedError

    def forward_greedy(self, xf, out_tokens: torch.Tensor) -> bool:
        """Greedy tokens of the rows without their logits: out_tokens[i] (int32, device) = argmax of row i's
        logits, ties to the lower id.  Returns False where the head has no such path for these sizes (the
        caller then takes forward() and the sampler)."""
        return False


# ----------------------------------------------------------------------------- registries

MIXERS: Dict[str, type] = {}
FEED_FORWARDS: Dict[str, type] = {}
NORMS: Dict[str, type] = {}
POSITION_ENCODINGS: Dict[str, type] = {}
EMBEDDINGS: Dict[str, type] = {}
HEADS: Dict[str, type] = {}
CONNECTORS: Dict[str, type] = {}
RESIDUAL_GATES: Dict[str, type] = {}
SIDE_INPUTS: Dict[str, type] = {}
SHARED: Dict[str, type] = {}

_TABLES = {"mixer": MIXERS, "feed_forward": FEED_FORWARDS, "norm": NORMS,
           "position": POSITION_ENCODINGS, "embedding": EMBEDDINGS, "head": HEADS, "connector": CONNECTORS,
           "gate": RESIDUAL_GATES, "side": SIDE_INPUTS, "shared": SHARED}


def register_part(category: str, kind: str):
    """Class decorator: `@register_part('mixer', 'attention')`."""
    table = _TABLES[category]

    def deco(cls):
        table[kind] = cls
        cls.kind = kind
        return cls
    return deco


def build_part(category: str, spec, dtype: str):
    from ..config.errors import ConfigError
    table = _TABLES[category]
    if spec.kind not in table:
        raise ConfigError(f"unknown {category} kind {spec.kind!r}; registered: {', '.join(sorted(table))}")
    part = table[spec.kind](dtype=dtype, **spec.kwargs())
    part.spec = spec
    return part
