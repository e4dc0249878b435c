"""The decoder assembled from a ``ModelSpec``: builds the parts, plans the cache groups the
mixers need, receives the weights and runs the schedule on a ``StepContext``.

Nothing here is specific to an architecture."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from dispec_b200.cache.manager import CacheGroupSpec
from dispec_b200.models.spec import LayerCall, ModelSpec
from dispec_b200.parts.base import CacheNeed, Part, PartSpec, StateNeed
from dispec_b200.registry import part_class


@dataclass(frozen=True)
class CachePlacement:
    group: int
    slot: int


def build_part(spec: PartSpec, built: dict, bindings: list, prefix: str = "") -> Part:
    """Instantiates a part; nested ``PartSpec`` values among the parameters are built first
    (the same spec object is built once and shared)."""
    if id(spec) in built:
        return built[id(spec)]
    params = {}
    for k, v in spec.params.items():
        params[k] = build_part(v, built, bindings) if isinstance(v, PartSpec) else v
    part = part_class(spec.role, spec.kind)(**params)
    built[id(spec)] = part
    local = part.tensor_specs()
    missing = sorted(set(local) - set(spec.tensors))
    extra = sorted(set(spec.tensors) - set(local))
    if missing or extra:
        raise ValueError(f"{spec.role} {spec.kind!r}: tensor name map does not match the part "
                         f"(unmapped: {missing}, unknown: {extra})")
    bindings.append((part, {name: (spec.tensors[name], local[name]) for name in local}))
    return part


class DecoderModel:
    def __init__(self, spec: ModelSpec, config=None):
        self.spec = spec
        self.config = config
        self.dtype = None
        self.device = None
        built: dict = {}
        self._bindings: list = []  # (part, {local: (checkpoint name, TensorSpec)})
        self.embedding = build_part(spec.embedding, built, self._bindings)
        self.layers = [build_part(s, built, self._bindings) for s in spec.layers]
        self.final_norm = build_part(spec.final_norm, built, self._bindings)
        self.head = build_part(spec.head, built, self._bindings)
        self._parts = list(built.values())
        self.schedule: list[LayerCall] = list(spec.schedule)
        self._plan_caches()

    # ------------------------------------------------------------------ cache planning
    def _plan_caches(self) -> None:
        """One layer cache per distinct cache label; caches with equal needs share a group."""
        needs: dict[int, CacheNeed] = {}
        writers: dict[int, int] = {}
        self.state_needs: list[StateNeed] = []
        self.call_state: list[int | None] = []
        self.call_cache: list[int | None] = []
        for idx, call in enumerate(self.schedule):
            mixer = self.layers[call.layer].mixer
            need = mixer.cache_need()
            label = None
            if need is not None:
                label = idx if call.cache is None else call.cache
                if label in needs and needs[label] != need:
                    raise ValueError(f"schedule entry {idx}: cache {label} is shared by mixers with "
                                     f"different needs ({needs[label]} vs {need})")
                needs.setdefault(label, need)
                if call.write:
                    if label in writers:
                        raise ValueError(f"schedule entry {idx}: cache {label} already has a writer "
                                         f"(entry {writers[label]})")
                    writers[label] = idx
                elif label not in writers:
                    raise ValueError(f"schedule entry {idx} reads cache {label} before any entry wrote it")
            self.call_cache.append(label)
            sneed = mixer.state_need()
            if sneed is not None:
                self.call_state.append(len(self.state_needs))
                self.state_needs.append(sneed)
            else:
                self.call_state.append(None)
        group_keys: list[CacheNeed] = []
        members: list[list[int]] = []
        self.placement: dict[int, CachePlacement] = {}
        for label in sorted(needs):
            need = needs[label]
            if need not in group_keys:
                group_keys.append(need)
                members.append([])
            g = group_keys.index(need)
            self.placement[label] = CachePlacement(g, len(members[g]))
            members[g].append(label)
        self.cache_groups = [CacheGroupSpec(tuple(k.tensors), k.window, len(m))
                             for k, m in zip(group_keys, members)]
        tiles: set = set()
        for c in self.schedule:
            want = self.layers[c.layer].mixer.tokens_per_attention_tile()
            if want:
                tiles.update(want if isinstance(want, (tuple, list)) else (want,))
        self.attention_tile_tokens = sorted(t for t in tiles if t)

    # ----------------------------------------------------------------------- weights
    def tensor_requirements(self) -> dict:
        """checkpoint name -> TensorSpec, over all parts (a name used twice must agree)."""
        req: dict = {}
        for part, names in self._bindings:
            for local, (ckpt, tspec) in names.items():
                if ckpt in req and (req[ckpt].shape != tspec.shape or req[ckpt].dtype != tspec.dtype):
                    raise ValueError(f"tensor {ckpt!r} is wanted with two shapes: "
                                     f"{req[ckpt].shape} and {tspec.shape}")
                req.setdefault(ckpt, tspec)
        return req

    def load(self, tensors: dict, dtype: torch.dtype, device) -> None:
        """``tensors``: checkpoint name -> device tensor, already checked and converted."""
        self.dtype, self.device = dtype, device
        for part, names in self._bindings:
            part.load({local: tensors[ckpt] for local, (ckpt, _) in names.items()})
        for part in self._parts:
            if hasattr(part, "prepare"):
                part.prepare(device)

    # ----------------------------------------------------------------------- forward
    def forward(self, ctx):
        """Runs the schedule.  Returns (x, pending): the residual stream and the last block's
        output not yet added to it."""
        x = self.embedding.forward(ctx)
        pending = None
        for idx, call in enumerate(self.schedule):
            label = self.call_cache[idx]
            cache = ctx.cache_view(self.placement[label], call.write) if label is not None else None
            sidx = self.call_state[idx]
            state = ctx.state_view(sidx) if sidx is not None else None
            # a block may take its first norm from the product that wrote x (see PreNormBlock)
            nxt = self.layers[self.schedule[idx + 1].layer] if idx + 1 < len(self.schedule) else None
            offer = getattr(nxt, "first_norm_after_product", None)
            then_norm = offer() if offer is not None else None
            if then_norm is not None and hasattr(self.layers[call.layer], "first_norm_after_product"):
                x, pending = self.layers[call.layer].forward(ctx, x, pending, cache, state, then_norm=then_norm)
            else:
                x, pending = self.layers[call.layer].forward(ctx, x, pending, cache, state)
        return x, pending

    def logits(self, ctx, x, pending, rows: torch.Tensor) -> torch.Tensor:
        """32-bit logits at the given flat token rows (int32 device tensor)."""
        if pending is None:
            h = self.final_norm.forward(ctx, x, rows=rows)
        else:
            h = self.final_norm.forward_add(ctx, x, pending, rows=rows)
        return self.head.forward(ctx, h)
