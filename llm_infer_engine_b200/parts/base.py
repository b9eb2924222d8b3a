"""Interfaces and registries of the parts a layer is put together from.

Six kinds of part, each with a registry from a kind name to a class:

    mixer              x[T, d] -> [T, d], mixes information between positions; may own cache
    feed_forward       x[T, d] -> [T, d], position-wise
    norm               float32 residual rows -> normalised activations
    position_encoding  how positions enter a mixer (rotation of q and k here)
    pointwise          a float32 tensor -> the same tensor changed row by row; the model's two optional
                       slots outside the layers (after the embedding, after the head)
    block              the arrangement of a layer's parts around the residual stream; it declares the
                       roles it has (`ROLES`) and the part group of each

A part is constructed from `(params, runtime)`: `params` is the mapping of its `PartSpec`
(every size and constant it needs; nothing is read from a model-wide config), `runtime` says
where and in which precision it runs. It declares its checkpoint tensors with `param_specs()`
and receives them through `load()`. No part knows which model it is in.

Adding a part: subclass the interface, then `register_mixer("my_kind", MyMixer)` (or the
matching function); a `PartSpec("my_kind", {...})` in a `ModelSpec` now builds it.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Dict, List, Mapping, Optional, Tuple, Union

import torch


@dataclass(frozen=True)
class Runtime:
    device: torch.device
    dtype: torch.dtype            # activation dtype: torch.float32 (true 32-bit path) or torch.bfloat16
    max_positions: int            # longest sequence the engine will hold


@dataclass(frozen=True)
class ParamSpec:
    """A checkpoint tensor of a part. `role`: "matrix" (a GEMM operand), "vector" (norm weights,
    biases) or "table" (integers). `init` is how the random-weights mode fills it:
    ("normal",) uses the caller's std, ("ones",), ("zeros",) or ("uniform", lo, hi). The random-weights mode
    writes optional tensors too. A negative entry -n of `shape` is a size that the checkpoint decides (any size is
    accepted, the part reads it from the tensor it is given); the random-weights mode writes n there."""
    shape: Tuple[int, ...]
    role: str = "matrix"
    init: Tuple = ("normal",)
    optional: bool = False        # a tensor that a checkpoint may hold or not; `load` gets it only when it is there


@dataclass(frozen=True)
class AttentionOptions:
    """Everything about softmax(q k^T) v that is not a shape. A mixer fills one and hands it to
    `ctx.attention`; a further option (a score cap, a bias by distance) becomes a field here with a
    default that means "off", and `KernelPlan.attention` sends a call that sets it to a kernel that
    knows it (the plain kernel first), so the call sites of the existing options do not change."""
    scale: float
    window: int = 0              # 0 = every earlier key; n = the last n keys, the token's own included
    keep_first: int = 0          # with a window: the first n keys of the sequence stay visible behind it
    sink: bool = False           # one more term exp(0) in the softmax's denominator (a key of score 0, no value)
    sink_values: Optional[torch.Tensor] = None   # float32 [query heads]: the sink's score per head instead of 0
    softcap: float = 0.0         # c > 0: a scaled score s becomes c * tanh(s / c)
    # float32 [query heads, L]: a number per head and distance (query position - key position) added to the score
    # after the cap, unscaled; distances of L - 1 and more share the last column
    distance_bias: Optional[torch.Tensor] = None
    # float32 [query heads]: no softmax at all; a visible key's weight is sigmoid(score + this number of its head), and
    # the weights are not normalised over the keys (so there is no denominator for a sink to enter)
    sigmoid_bias: Optional[torch.Tensor] = None

    @property
    def plain(self) -> bool:
        """Only the options every attention kernel knows (scale, window)."""
        return self.keep_first == 0 and not self.sink and not self.scored and self.sigmoid_bias is None

    @property
    def scored(self) -> bool:
        """Whether an option changes single scores (a cap, a bias by distance, a learned sink)."""
        return self.softcap > 0 or self.distance_bias is not None or self.sink_values is not None


class Part:
    def __init__(self, params: Mapping, runtime: Runtime):
        self.params = dict(params)
        self.runtime = runtime

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Receives the tensors named by param_specs(), already on the device."""

    def weight_bytes(self) -> int:
        """Bytes of weights that one step reads (for roofline accounting)."""
        return 0


class Norm(Part):
    def forward(self, h: torch.Tensor, delta, out: Optional[torch.Tensor] = None,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """h (float32 [T, d]) += delta in place when rows is None; returns norm(h) in the
        activation dtype. With `rows`, only those rows are produced and h is untouched. `delta` is a tensor, None,
        or a tuple of two branch outputs that are both added (a block whose branches run side by side); a norm whose
        kernel adds one tensor calls `single_delta` first."""
        raise NotImplementedError

    def add_normed(self, h: torch.Tensor, y: torch.Tensor, bias: Optional[torch.Tensor] = None,
                   act: Optional[torch.Tensor] = None) -> torch.Tensor:
        """For blocks whose norm sits on a branch's OUTPUT: h (float32 [T, d]) += norm(y + bias) in place. `act`,
        if given, receives the new h rounded to its dtype (the next product's input)."""
        raise NotImplementedError

    def norm_sum(self, h: torch.Tensor, y: torch.Tensor, vector: Optional[torch.Tensor] = None,
                 act: Optional[torch.Tensor] = None) -> torch.Tensor:
        """For blocks whose norm comes AFTER the residual sum: h (float32 [T, d]) = norm(alpha * h + vector (.) y) in
        place, alpha a constant of the norm and `vector` a float32 [d] scale per channel on the branch (None = ones).
        `act`, if given, receives the new h rounded to its dtype (the next product's input)."""
        raise NotImplementedError

    def defer(self, h: torch.Tensor) -> Optional["DeferredNorm"]:
        """A promise of norm(h) for a consumer that can fold the norm into its own first kernel,
        or None when this norm (or this shape) cannot be folded."""
        return None


class ScaledDelta:
    """Branch output that is scaled on its way into the stream: vector (.) (c1 t1 + c2 t2), with `terms` a list of
    one or two (tensor, constant) pairs and `vector` a float32 [d] scale per channel or None. A mixer made of two
    mixers returns one without a vector; a block with a learned scale per channel puts its vector on whatever its
    branch returned. A norm whose kernel knows the form adds it while it reads the stream; `materialize()` gives the
    plain float32 tensor to everything else."""

    def __init__(self, terms, vector: Optional[torch.Tensor] = None):
        terms = [(t, float(c)) for t, c in terms]
        if not 1 <= len(terms) <= 2:
            raise ValueError("a ScaledDelta has one or two terms")
        self.terms, self.vector = terms, vector

    @staticmethod
    def of(y, vector: Optional[torch.Tensor]) -> "ScaledDelta":
        """`y` (a tensor or a ScaledDelta without a vector) times `vector`, channel by channel."""
        if isinstance(y, ScaledDelta):
            if y.vector is not None:
                raise ValueError("this branch output already carries a vector")
            return ScaledDelta(y.terms, vector)
        return ScaledDelta([(y, 1.0)], vector)

    def materialize(self) -> torch.Tensor:
        from ..kernels import ops
        (t1, c1), (t2, c2) = self.terms[0], (self.terms[1] if len(self.terms) > 1 else (None, 0.0))
        out = torch.zeros(t1.shape, dtype=torch.float32, device=t1.device)
        ops.scaled_add_rmsnorm(out, t1, c1, t2, c2, self.vector, None, 0.0, None)
        return out


def single_delta(delta):
    """One tensor for norms whose kernel adds one: the members of a tuple are summed into a float32 member (or a
    float32 copy of the first) by the residual-add kernel; a ScaledDelta is worked out."""
    if isinstance(delta, ScaledDelta):
        return delta.materialize()
    if not isinstance(delta, (tuple, list)):
        return delta
    parts = [d for d in delta if d is not None]
    if not parts:
        return None
    if len(parts) == 1:
        return parts[0]
    from ..kernels import ops
    parts.sort(key=lambda t: t.dtype != torch.float32)
    total = parts[0] if parts[0].dtype == torch.float32 else parts[0].to(torch.float32)
    for d in parts[1:]:
        ops.residual_add(total, d)
    return total


class DeferredNorm:
    """norm(h) that has not been computed. A part that declares `accepts_deferred_norm = True`
    may receive one instead of a tensor; it either folds the norm into its first kernel (using
    `kind`, `weight`, `eps`) or calls `apply()` and goes on with the tensor."""

    def __init__(self, norm: Norm, h: torch.Tensor, kind: str, weight: torch.Tensor, eps: float):
        self.norm, self.h, self.kind, self.weight, self.eps = norm, h, kind, weight, eps

    @property
    def shape(self):
        return self.h.shape

    def apply(self) -> torch.Tensor:
        return self.norm.forward(self.h, None)


class DeferredBranchAdd:
    """h += norm(y + bias) that has not been done: what a block whose norm sits on the branch's OUTPUT hands on instead
    of doing it, so that the product that opens the next branch can do it while it stages its input. Whoever receives
    one (a part that declares `accepts_deferred_branch_add`, the next block, or the model after the last layer)
    either folds it into its first kernel and sets `resolved` to the new stream, or calls `apply()`."""

    def __init__(self, norm: Norm, h: torch.Tensor, y: torch.Tensor, bias: Optional[torch.Tensor]):
        self.norm, self.h, self.y, self.bias = norm, h, y, bias
        self.resolved: Optional[torch.Tensor] = None       # the stream after the add, once someone has done it

    @property
    def shape(self):
        return self.h.shape

    def foldable(self, weight: torch.Tensor) -> bool:
        """Whether a product with this bfloat16 weight should do the add itself: one-token steps of as few rows as
        the fold was measured to pay for (`ops.BRANCH_FOLD_BEST_ROWS`; the kernel takes up to 8)."""
        from ..kernels import ops
        return (getattr(self.norm, "kind", None) == "rmsnorm" and weight.dtype == torch.bfloat16
                and self.y.dtype == torch.float32 and weight.shape[0] % 16 == 0
                and self.h.shape[0] <= ops.BRANCH_FOLD_BEST_ROWS
                and ops.norm_gemm_supported(self.h.shape[0], self.h.shape[1]))

    def apply(self, act: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Does the add in a kernel of its own; `act` receives the new stream rounded to its dtype."""
        if self.resolved is None:
            self.resolved = self.norm.add_normed(self.h, self.y, self.bias, act)
        return self.resolved


class PositionEncoding(Part):
    def encode_and_store(self, qkv: torch.Tensor, ctx, kv, n_q: int, n_kv: int, head_dim: int,
                         write_kv: bool) -> torch.Tensor:
        """Takes the packed projections [T, (n_q + 2 n_kv) head_dim], returns position-encoded
        queries [T, n_q head_dim] and, if write_kv, writes encoded keys and the values into
        the cache unit `kv` at each token's position."""
        raise NotImplementedError


class Mixer(Part):
    """Two class flags widen what a block hands to `forward`; both default to False, and a part that
    leaves them so is called with exactly `(x, ctx, unit, owns_cache)`:

    accepts_deferred_norm  x may be a `DeferredNorm` instead of a tensor: the part folds the norm into
                           its first kernel, or calls `x.apply()` and goes on with the tensor.
    adds_to_residual       the block also passes `residual=h` (the float32 residual stream [T, d]); the
                           part may add its output into it inside its last kernel and then returns None
                           instead of a branch output, or ignores it and returns the output as usual.
    """
    accepts_deferred_norm = False
    adds_to_residual = False
    accepts_deferred_branch_add = False     # x may be a DeferredBranchAdd: the part folds it or calls x.apply(act)

    def cache_requests(self) -> List[object]:
        """KVRequest / StateRequest objects: what one run of this mixer needs per sequence."""
        return []

    def forward(self, x: Union[torch.Tensor, "DeferredNorm"], ctx, unit, owns_cache: bool,
                residual: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """x: normalised activations [T, d] (or a DeferredNorm, see the class flags). `unit` is the
        CacheUnit to use; when `owns_cache` is False it belongs to an earlier schedule entry and must
        only be read. Returns the branch output [T, d], or None after adding it into `residual`."""
        raise NotImplementedError


class FeedForward(Part):
    """The class flags of `Mixer` hold here too, with the call `(x, ctx)` as the plain form."""
    accepts_deferred_norm = False
    adds_to_residual = False

    def forward(self, x: Union[torch.Tensor, "DeferredNorm"], ctx,
                residual: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        raise NotImplementedError


class Pointwise(Part):
    """A change of a float32 tensor row by row, for the model's two slots outside the layers."""

    def forward(self, x: torch.Tensor, ctx, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x: float32 [n, width], changed in place or replaced by the returned tensor. After the embedding
        row i is token i of the step (`ctx.tok_pos[i]` is its position) and `rows` is None; after the head
        row i is the logits of packed token `rows[i]`."""
        raise NotImplementedError


def call_branch(part, x, ctx, *cache_args, residual: Optional[torch.Tensor] = None):
    """Calls a mixer or feed-forward the way its class flags ask for: `residual` is passed only to a part
    that declared `adds_to_residual`, and a DeferredNorm is applied first unless the part accepts one."""
    if isinstance(x, DeferredNorm) and not part.accepts_deferred_norm:
        x = x.apply()
    if part.adds_to_residual and residual is not None:
        return part.forward(x, ctx, *cache_args, residual=residual)
    return part.forward(x, ctx, *cache_args)


class Block:
    """Arrangement of one layer's parts around the float32 residual stream.

    A subclass declares `ROLES`: role name -> part group ("mixer", "feed_forward", "norm", ...). The model
    builder builds one part per role from the layer's `LayerSpec.parts` and hands them over as a dict;
    each is then an attribute of the block under its role name.

    forward(h, pending, ctx, unit, owns_cache) -> (h, pending): `pending` is a branch output
    not yet added to h (None at the first layer), so that each residual add can be fused with
    the norm that follows it."""
    ROLES: Dict[str, str] = {}

    def __init__(self, parts: Dict[str, Part], runtime: Runtime):
        missing = [r for r in self.ROLES if r not in parts]
        unknown = [r for r in parts if r not in self.ROLES]
        if missing or unknown:
            raise ValueError(f"{type(self).__name__} has the roles {sorted(self.ROLES)}; missing {missing}, "
                             f"unknown {unknown}")
        clash = [r for r in self.ROLES if hasattr(Block, r) or r in ("runtime", "_parts")]
        if clash:
            raise ValueError(f"{type(self).__name__}: role name(s) {clash} collide with the block's own attributes")
        self._parts = {role: parts[role] for role in self.ROLES}
        self.runtime = runtime
        for role, part in self._parts.items():
            setattr(self, role, part)

    def parts(self) -> Dict[str, Part]:
        return dict(self._parts)

    def mixer_roles(self) -> List[str]:
        return [role for role, group in self.ROLES.items() if group == "mixer"]

    def cache_requests(self) -> List[object]:
        """What one run of this layer needs per sequence: the requests of its mixers. With one mixer they
        are the mixer's own; with several, each request's name is prefixed with the mixer's role
        ("role.name") and `unit.scoped(role)` gives that mixer its own view."""
        roles = self.mixer_roles()
        if len(roles) == 1:
            return list(self._parts[roles[0]].cache_requests())
        out = []
        for role in roles:
            for r in self._parts[role].cache_requests():
                out.append(dataclasses.replace(r, name=f"{role}.{r.name}"))
        return out

    def forward(self, h, pending, ctx, unit, owns_cache):
        raise NotImplementedError


_REGISTRIES: Dict[str, Dict[str, type]] = {"mixer": {}, "feed_forward": {}, "norm": {}, "position_encoding": {},
                                           "pointwise": {}, "block": {}}


def _register(group: str, kind: str, cls: type) -> None:
    _REGISTRIES[group][kind] = cls


def register_mixer(kind: str, cls: type) -> None:
    _register("mixer", kind, cls)


def register_feed_forward(kind: str, cls: type) -> None:
    _register("feed_forward", kind, cls)


def register_norm(kind: str, cls: type) -> None:
    _register("norm", kind, cls)


def register_position_encoding(kind: str, cls: type) -> None:
    _register("position_encoding", kind, cls)


def register_pointwise(kind: str, cls: type) -> None:
    _register("pointwise", kind, cls)


def register_block(kind: str, cls: type) -> None:
    _register("block", kind, cls)


def lookup(group: str, kind: str) -> type:
    reg = _REGISTRIES[group]
    if kind not in reg:
        raise KeyError(f"no {group} of kind {kind!r} is registered (known: {sorted(reg)})")
    return reg[kind]


def undefer(x):
    """The tensor behind x, applying a deferred norm if x is one."""
    return x.apply() if isinstance(x, DeferredNorm) else x


def build_part(group: str, spec, runtime: Runtime):
    """spec: a PartSpec (or anything with .kind and .params)."""
    return lookup(group, spec.kind)(spec.params, runtime)
