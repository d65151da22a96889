"""A model assembled from a ModelSpec: embedding, blocks of (norm, mixer, norm, feed-forward),
final norm and head, run in the order the spec's schedule gives.

The forward pass here is the body of the step function: it runs exactly the rows of one
StepContext, reads and writes the caches through the views it is given, and computes the final
norm and the head only for the rows whose logits are wanted (FeLLM skips final_norm + lm_head for
mid-prompt tokens the same way, crates/fellm-runtime/src/compiled.rs:425-434).
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .. import ops
from ..config.errors import ConfigError
from ..parts.base import ParamDecl, build_part
from ..parts.linear import LazyNorm, linear
from ..parts.spec import ModelSpec


def _normed(x, norm, consumer, act_dtype):
    """The consumer's input: normed now, or left to the consumer's first product."""
    if getattr(consumer, "takes_lazy_norm", False):
        return LazyNorm(x, norm, act_dtype)
    return norm.forward(x, act_dtype)


ARRANGEMENTS = {}


def register_arrangement(name: str):
    """Decorator: `fn(block, x, ctx, cache, act_dtype, reads_only)` wires a block's parts for
    LayerSpec.arrangement == name.  x is the float32 residual stream [T, d] and is updated in
    place (mixers and feed-forwards ADD into the tensor they are given as `out`); `block` has
    .norm1, .mixer, .norm2, .ffn (None where the spec names none) and, during the call,
    .norm_after: the norm that reads x after this block (the next block's first, or the final one;
    None where that is not known).  An arrangement may tell a norm that it comes next
    (`norm.expect(x)`) right before the part whose last act is to add into x."""
    def deco(fn):
        ARRANGEMENTS[name] = fn
        return fn
    return deco


def normed(x, norm, consumer, act_dtype):
    """The consumer's input: normed now, or left to the consumer's first product."""
    return _normed(x, norm, consumer, act_dtype)


@register_arrangement("prenorm")
def _prenorm(block, x, ctx, cache, act_dtype, reads_only):
    """x += mixer(norm1(x)); x += ffn(norm2(x))   (crates/fellm-model/src/graph.rs:1650-1777)."""
    h = _normed(x, block.norm1, block.mixer, act_dtype)
    after_mixer = block.norm2 if block.ffn is not None else block.norm_after
    if after_mixer is not None:
        after_mixer.expect(x)
    block.mixer.forward(h, ctx, cache, x, reads_only=reads_only)
    if block.ffn is not None:
        h = _normed(x, block.norm2, block.ffn, act_dtype)
        if block.norm_after is not None:
            block.norm_after.expect(x)
        block.ffn.forward(h, ctx, x)


@register_arrangement("parallel")
def _parallel(block, x, ctx, cache, act_dtype, reads_only):
    """h = norm1(x); x += mixer(h) + ffn(h): one norm, both sublayers read its output (each adds into x, the mixer
    first)."""
    h = block.norm1.forward(x, act_dtype)
    block.mixer.forward(h, ctx, cache, x, reads_only=reads_only)
    if block.ffn is not None:
        block.ffn.forward(h, ctx, x)


@register_arrangement("parallel_gated")
def _parallel_gated(block, x, ctx, cache, act_dtype, reads_only):
    """h = norm1(x); x += mixer(h) * sigmoid(W_1 h + b_1) + ffn(h) * sigmoid(W_2 h + b_2): the sublayers add into rows of
    zeros of their own (or write rows of their own), and the block's gates take those into the stream."""
    if block.gate is None:
        raise ConfigError("the 'parallel_gated' arrangement needs the layer's gates")
    h = block.norm1.forward(x, act_dtype)
    pre = {}
    if block.joint is not None:
        # everything that reads h through float32 sums (the gates' logits, the mixer's down projections, a dense
        # feed-forward's up product) is ONE product; each part gets its columns
        w, bias, cols = block.joint
        z = linear(h, w, bias, out_dtype=torch.float32)
        pre = {key: {"pre": z[:, a:b]} for key, (a, b) in cols.items()}
    zg = pre["gate"]["pre"] if "gate" in pre else block.gate.logits(h)
    # (a sublayer that says `can_store` writes its result instead of adding it: no rows of zeros to make)
    if getattr(block.mixer, "can_store", False):
        results = [block.mixer.forward(h, ctx, cache, torch.empty_like(x), reads_only=reads_only, store=True, **pre.get("mixer", {}))]
    else:
        results = [block.mixer.forward(h, ctx, cache, torch.zeros_like(x), reads_only=reads_only, **pre.get("mixer", {}))]
    if block.ffn is not None:
        if getattr(block.ffn, "can_store", False):
            results.append(block.ffn.forward(h, ctx, torch.empty_like(x), store=True, **pre.get("ffn", {})))
        else:
            results.append(block.ffn.forward(h, ctx, torch.zeros_like(x), **pre.get("ffn", {})))
    if getattr(block.side, "takes_gated_add", False):
        return results, zg          # the side input's kernel reads the stream anyway: it adds the gated results on its way in
    block.gate.add(x, results, zg)


_parallel_gated.joins_inputs = True


@register_arrangement("outnorm")
def _outnorm(block, x, ctx, cache, act_dtype, reads_only):
    """x += norm1(mixer(x)); x += norm2(ffn(x)): the sublayers read the stream itself and the norms stand on their
    OUTPUTS.  A sublayer leaves float32 rows of its own (written where it says `can_store`, else added into zeros) and
    the norm's `add_normed` takes them into the stream; a mixer that says `reads_stream` gets the float32 rows
    themselves, any other part a copy in the activation dtype (which the first norm leaves behind for the feed-forward)."""
    for norm in (block.norm1, block.norm2 if block.ffn is not None else block.norm1):
        if norm is None or not hasattr(norm, "add_normed"):
            raise ConfigError("the 'outnorm' arrangement needs norms that offer add_normed (layernorm)")
    h = x if getattr(block.mixer, "reads_stream", False) else ops.cast_rows(x, act_dtype)
    if getattr(block.mixer, "can_store", False):
        y = block.mixer.forward(h, ctx, cache, torch.empty_like(x), reads_only=reads_only, store=True)
    else:
        y = block.mixer.forward(h, ctx, cache, torch.zeros_like(x), reads_only=reads_only)
    if block.ffn is None:
        block.norm1.add_normed(x, y)
        return
    h = x if act_dtype == torch.float32 else torch.empty(x.shape, dtype=act_dtype, device=x.device)
    block.norm1.add_normed(x, y, cast=None if h is x else h)
    if getattr(block.ffn, "can_store", False):
        y = block.ffn.forward(h, ctx, y, store=True)
    else:
        y = block.ffn.forward(h, ctx, y.zero_())
    block.norm2.add_normed(x, y)


def _with_children(part):
    return [part] + [q for c in part.children() for q in _with_children(c)]


class Block:
    """One layer's parts; how they are wired is looked up by the spec's arrangement name."""

    def __init__(self, spec, dtype: str):
        if spec.arrangement not in ARRANGEMENTS:
            raise ConfigError(f"unknown block arrangement {spec.arrangement!r}; registered: "
                              f"{', '.join(sorted(ARRANGEMENTS))}")
        self.spec = spec
        self.arrange = ARRANGEMENTS[spec.arrangement]
        self.norm1 = build_part("norm", spec.norm1, dtype) if spec.norm1 is not None else None
        self.mixer = build_part("mixer", spec.mixer, dtype)
        self.norm2 = build_part("norm", spec.norm2, dtype) if spec.norm2 is not None else None
        self.ffn = build_part("feed_forward", spec.ffn, dtype) if spec.ffn is not None else None
        self.gate = build_part("gate", spec.gate, dtype) if spec.gate is not None else None
        self.side = build_part("side", spec.side, dtype) if spec.side is not None else None
        self.norm_after = None
        self.joint = None           # (weight [N, d], bias float32 [N], {"gate" | "mixer" | "ffn": (first column, end)}) after join_inputs()

    def join_inputs(self):
        """After every part is bound: the rows of the parts that read the block's input through a product with
        float32 sums (a part names them `input_rows`) become ONE matrix, of which each part keeps a view; a part's bias
        (`input_bias`) lies at its rows of the joint bias, zeros elsewhere.  Only where the arrangement makes that
        product (`joins_inputs`), all rows have one dtype and at least two parts take part (a part whose rows are not a
        multiple of 8 stays out: the parts' columns start on 32 bytes)."""
        if not getattr(self.arrange, "joins_inputs", False):
            return
        users = [(key, p) for key, p in (("mixer", self.mixer), ("gate", self.gate), ("ffn", self.ffn))
                 if p is not None and getattr(p, "input_rows", None) and p.input_rows in p.w and p.w[p.input_rows].shape[0] % 8 == 0]
        mats = [p.w[p.input_rows] for _, p in users]
        if len(users) < 2 or any(m.dtype != mats[0].dtype or m.shape[1] != mats[0].shape[1] for m in mats):
            return
        joint = torch.cat(mats, 0).contiguous()
        bias = torch.zeros(joint.shape[0], dtype=torch.float32, device=joint.device)
        cols, at = {}, 0
        for (key, p), m in zip(users, mats):
            n = m.shape[0]
            p.w[p.input_rows] = joint[at:at + n]
            name = getattr(p, "input_bias", None)
            if name and name in p.w:
                bias[at:at + n] = p.w[name]
            cols[key] = (at, at + n)
            at += n
        self.joint = (joint, bias, cols)

    def parts(self):
        return [q for p in (self.norm1, self.mixer, self.norm2, self.ffn, self.gate, self.side) if p is not None
                for q in _with_children(p)]

    def forward(self, x, ctx, cache, act_dtype, reads_only=False, norm_after=None):
        """x: float32 residual stream [T, d], updated in place."""
        self.norm_after = norm_after
        pending = self.arrange(self, x, ctx, cache, act_dtype, reads_only)
        if pending is not None:
            self.side.forward(x, ctx, pending=pending)
        elif self.side is not None:
            self.side.forward(x, ctx)
        return x


class Model:
    def __init__(self, spec: ModelSpec, dtype: str):
        self.spec, self.dtype = spec, dtype
        self.act_dtype = torch.bfloat16 if dtype == "bfloat16" else torch.float32
        self.embedding = build_part("embedding", spec.embedding, dtype)
        self.blocks: List[Block] = [Block(ls, dtype) for ls in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, dtype)
        self.head = build_part("head", spec.head, dtype)
        self.connectors = [build_part("connector", cs, dtype) for cs in spec.connectors]
        self.shared = [build_part("shared", ss, dtype) for ss in spec.shared]
        self.schedule = list(spec.schedule)
        self.after_run = None          # a callable (schedule entry, x) that is shown the stream after every run (tests, debugging)

    # ---- parameters
    def all_parts(self):
        parts = [self.embedding]
        for b in self.blocks:
            parts += b.parts()
        return parts + self.connectors + self.shared + [self.final_norm, self.head]

    def param_table(self) -> Dict[str, tuple]:
        """{tensor name in the file: (part, local name, ParamDecl)} over all parts."""
        table = {}
        for part in self.all_parts():
            for local, decl in part.param_decls().items():
                name = part.spec.tensor_name(local)
                if name in table:
                    raise ConfigError(f"two parts claim the tensor {name}")
                table[name] = (part, local, decl)
        return table

    def tied_aliases(self) -> Dict[str, str]:
        """{name a file may also carry: name of the tensor it must equal}.  A tied head owns no
        tensor, but files written from a state dict often store the head all the same, as a copy of
        the embedding matrix (FeLLM reads `output.weight` when it is there and ties otherwise,
        crates/fellm-model/src/graph.rs:29-34); such a copy is accepted if it is one."""
        if getattr(self.head, "tied", False):
            return {self.head.spec.tensor_name("weight"): self.embedding.spec.tensor_name("weight")}
        return {}

    def bind(self, tensors: Dict[str, torch.Tensor]):
        """tensors: {file name: tensor already on the device, in its kept dtype}."""
        per_part: Dict[int, dict] = {}
        for name, (part, local, _) in self.param_table().items():
            per_part.setdefault(id(part), {})[local] = tensors[name]
        for part in self.all_parts():
            if part is self.head and getattr(part, "tied", False):
                continue
            part.bind(per_part.get(id(part), {}))
        if getattr(self.head, "tied", False):
            self.head.bind({"weight": self.embedding.w["weight"]})
        # parts that read a shared part's tensors are handed it by the name of its first tensor
        by_name = {sp.spec.tensor_name(next(iter(sp.param_decls()))): sp for sp in self.shared}
        for part in self.all_parts():
            want = getattr(part, "uses_shared", None)
            if want is not None:
                if want not in by_name:
                    raise ConfigError(f"a part asks for the shared tensor {want!r}, which the model does not have")
                part.attach(by_name[want])
        for block in self.blocks:
            block.join_inputs()

    def kernel_modules(self):
        mods = []
        for part in self.all_parts():
            mods += part.kernel_modules(self.dtype)
        return mods

    def weight_chain(self):
        """The matrices of one step in the order its products read them (the schedule's order)."""
        chain = []
        for run in self.schedule:
            b = self.blocks[run.layer]
            if run.before is not None:
                chain += self.connectors[run.before[0]].weight_order()
            chain += b.mixer.weight_order()
            if b.ffn is not None:
                chain += b.ffn.weight_order()
        return chain + self.head.weight_order()

    def cache_needs(self):
        """Per schedule entry: the mixer's cache need; when the entry reads another's, what it still keeps of its own
        (mostly None)."""
        return [self.blocks[run.layer].mixer.private_need() if run.cache_of is not None
                else self.blocks[run.layer].mixer.cache_need() for run in self.schedule]

    # ---- the step's body
    def forward(self, ctx, caches, greedy_tokens=None) -> torch.Tensor:
        """ctx: StepContext; caches[n]: the cache view of schedule entry n.  Returns float32
        logits [len(ctx.logit_rows), vocab] (an empty tensor when none are wanted).
        greedy_tokens (int32, device): the caller only wants the greedy token of every wanted row; where the
        head can give them without the logits it writes greedy_tokens[:wanted] and None is returned."""
        ops.forget_norm_handoff()
        x = self.embedding.forward(ctx.tokens, ctx.status)
        # a connector reads the embedding's output again later; the blocks update x in place
        x0 = x.clone() if any(c.needs_embedding for c in self.connectors) else None
        for n, run in enumerate(self.schedule):
            src = n if run.cache_of is None else run.cache_of
            if run.before is not None:
                x = self.connectors[run.before[0]].forward(x, x0, run.before[1], self.act_dtype)
            if n + 1 < len(self.schedule):
                norm_after = self.blocks[self.schedule[n + 1].layer].norm1
            else:
                norm_after = self.final_norm if (ctx.logits_all and ctx.n_logit_rows) else None
            cache = caches[src]
            if run.cache_of is not None and caches[n] is not None:
                cache = (caches[n], cache)          # what the entry keeps of its own, and the entry it reads
            self.blocks[run.layer].forward(x, ctx, cache, self.act_dtype,
                                           reads_only=run.cache_of is not None, norm_after=norm_after)
            if self.after_run is not None:
                self.after_run(n, x)
        if ctx.n_logit_rows == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=x.device)
        if ctx.logits_all and getattr(self.head, "takes_lazy_norm", False):
            xf = LazyNorm(x, self.final_norm, self.act_dtype)
        else:
            xf = self.final_norm.forward(x, self.act_dtype, rows=ctx.logit_rows)
        if greedy_tokens is not None and self.head.forward_greedy(xf, greedy_tokens):
            return None
        return self.head.forward(xf)


def build_model(spec: ModelSpec, dtype: str) -> Model:
    return Model(spec, dtype)
