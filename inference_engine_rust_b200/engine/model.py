"""A model assembled from a `ModelSpec`: embedding table, one block per layer, final norm,
output head; and its forward pass over the tokens of one step.

Reference: the layer loop and the last-row logits of src/engine/runtime.rs:14-33,76-116,
embedding of src/engine/embed.rs:104-138.  Differences on purpose: the loop follows the
spec's schedule (a list of layer executions), and logits are produced for any wanted rows.
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional

import torch

from ..cache import CacheRequest
from ..config.specs import ModelSpec
from ..csrc import bindings as B
from ..parts.base import Runtime, StepContext, first_norm_request_of, part_class
from ..weights.loader import (RandomSource, TensorSpec, WeightError, check_source, fetch_many)


class Model:
    def __init__(self, spec: ModelSpec, rt: Runtime):
        spec.validate()
        self.spec = spec
        self.rt = rt
        self.blocks = []
        self._layer_parts = []       # (norm1, mixer, norm2, ffn) per layer
        self._cut_askers = None
        h = spec.hidden_size
        self._extra_norms = []       # {role: norm} per layer (arrangements with more than two norms)
        for ls in spec.layers:
            norm_cls = part_class("norm", ls.norm.kind)
            norm1 = norm_cls(ls.norm, h, rt)
            norm2 = norm_cls(ls.norm, h, rt) if ls.ffn is not None else None
            mixer = part_class("mixer", ls.mixer.kind)(ls.mixer, rt)
            ffn = part_class("ffn", ls.ffn.kind)(ls.ffn, rt) if ls.ffn is not None else None
            extra = {role: part_class("norm", ns.kind)(ns, h, rt) for role, (ns, _) in ls.extra_norms.items()}
            kw = {"extra_norms": extra} if extra else {}
            block = part_class("block", ls.block.kind)(ls, norm1, mixer, norm2, ffn, rt, **kw)
            self._layer_parts.append((norm1, mixer, norm2, ffn))
            self._extra_norms.append(extra)
            self.blocks.append(block)
        self.final_norm = part_class("norm", spec.final_norm.kind)(spec.final_norm, h, rt)
        self.embedding: Optional[torch.Tensor] = None
        self.lm_head = part_class("head", spec.head.kind)(spec.head, h, spec.vocab_size, rt)
        self.inputs = [(part_class("input", ps.kind)(ps, h, spec.vocab_size, rt), prefix) for ps, prefix in spec.inputs]
        self.loaded = False
        self.ignored_tensors: List[str] = []
        self.notes: List[str] = []       # what loading decided on its own (tied head, ignored tensors)

    # ---- weights ------------------------------------------------------------------------
    def expected_tensors(self) -> Dict[str, TensorSpec]:
        """Every tensor name the model reads from a folder, with its shape."""
        spec = self.spec
        out: Dict[str, TensorSpec] = {
            spec.embedding_name: TensorSpec((spec.vocab_size, spec.hidden_size)),
            spec.final_norm_name: self.final_norm.tensor_specs()["weight"],
        }
        if spec.lm_head_name is not None:
            out[spec.lm_head_name] = self.lm_head.tensor_specs()["weight"]
        for part, prefix in self.inputs:
            for local, ts in part.tensor_specs().items():
                out[prefix + local] = ts
        for ls, (norm1, mixer, norm2, ffn), extra in zip(spec.layers, self._layer_parts, self._extra_norms):
            out[ls.mixer_norm_name] = norm1.tensor_specs()["weight"]
            for local, ts in mixer.tensor_specs().items():
                out[ls.mixer_prefix + local] = ts
            if ffn is not None:
                out[ls.ffn_norm_name] = norm2.tensor_specs()["weight"]
                for local, ts in ffn.tensor_specs().items():
                    out[ls.ffn_prefix + local] = ts
            for role, norm in extra.items():
                out[ls.extra_norms[role][1]] = norm.tensor_specs()["weight"]
        return out

    def load(self, source, where: str = "weights", strict: bool = True) -> None:
        """Check `source` against the expected tensors (one error for everything that is
        wrong), then hand each part its tensors.

        A source without the output head's tensor ties the head to the embedding table, as
        the reference does whenever `output.weight` is absent
        (src/model_weights/names.rs:300-310), whatever the configuration's flag says.
        `strict=False` accepts tensors the model does not know (a checkpoint that carries
        extras) and lists them in `self.ignored_tensors`."""
        expected = self.expected_tensors()
        rt, spec = self.rt, self.spec
        head_name = spec.lm_head_name
        if head_name is not None and head_name not in set(source.names()):
            expected.pop(head_name)
            head_name = None
            self.notes.append(f"{where}: no {spec.lm_head_name!r}; the output head is tied to "
                              f"{spec.embedding_name!r}")
        self.ignored_tensors = check_source(expected, source, where, strict=strict)
        if self.ignored_tensors:
            self.notes.append(f"{where}: {len(self.ignored_tensors)} tensor(s) the model does not use were "
                              f"ignored: " + ", ".join(self.ignored_tensors[:8])
                              + (" ..." if len(self.ignored_tensors) > 8 else ""))

        # every tensor to the device first (files: one pass of the native reader per file), then
        # each part takes its own; a part that fuses matrices lets go of the separate ones
        tensors = fetch_many(source, list(expected), rt.dtype, rt.device)

        def get(name):
            return tensors.pop(name)

        self.embedding = get(spec.embedding_name)
        self.final_norm.load({"weight": get(spec.final_norm_name)})
        self.lm_head.load({"weight": self.embedding if head_name is None else get(head_name)})
        tied = getattr(self.lm_head, "weight", None)
        if head_name is None and tied is not None and tied.dtype == self.embedding.dtype \
                and tied.shape == self.embedding.shape:
            self.embedding = tied                          # tied: one copy
        for part, prefix in self.inputs:
            part.load({local: get(prefix + local) for local in part.tensor_specs()})
        for ls, (norm1, mixer, norm2, ffn), extra in zip(spec.layers, self._layer_parts, self._extra_norms):
            norm1.load({"weight": get(ls.mixer_norm_name)})
            mixer.load({local: get(ls.mixer_prefix + local) for local in mixer.tensor_specs()})
            if ffn is not None:
                norm2.load({"weight": get(ls.ffn_norm_name)})
                ffn.load({local: get(ls.ffn_prefix + local) for local in ffn.tensor_specs()})
            for role, norm in extra.items():
                norm.load({"weight": get(ls.extra_norms[role][1])})
        self.loaded = True

    def load_random(self, seed: int, std: float = 0.02, on_device: bool = False) -> None:
        """Seeded random weights without a folder (`on_device` draws them on the GPU, for
        models too large to make on the host in reasonable time)."""
        src = RandomSource(self.expected_tensors(), seed, std, dtype=self.rt.dtype,
                           device=self.rt.device if on_device else "cpu")
        self.load(src, where="random weights")

    # ---- cache ----------------------------------------------------------------------------
    def cache_requests(self) -> Dict[int, CacheRequest]:
        """What each cache-writing schedule entry asks of the cache, keyed by its position."""
        out = {}
        for pos, e in enumerate(self.spec.schedule):
            if e.writes_cache:
                out[pos] = self._layer_parts[e.layer][1].cache_request()
        return out

    def graph_safe(self) -> bool:
        """True when every part declares `graph_safe`: its forward reads the step's sequences
        from device memory only, so a captured launch sequence stays right for later steps."""
        parts = [self.final_norm, self.lm_head] + [part for part, _ in self.inputs]
        for e in self.spec.schedule:
            parts.extend(p for p in self._layer_parts[e.layer] if p is not None)
            parts.extend(self._extra_norms[e.layer].values())
            parts.append(self.blocks[e.layer])
        return all(getattr(p, "graph_safe", False) for p in parts)

    def weight_bytes_per_step(self) -> int:
        """Bytes of weights a one-token step reads: every matrix each scheduled layer uses,
        the norm scales, the output head (the embedding rows it gathers are negligible)."""
        total = self.lm_head.nbytes() + sum(part.weight_bytes() for part, _ in self.inputs if hasattr(part, "weight_bytes"))
        for e in self.spec.schedule:
            norm1, mixer, norm2, ffn = self._layer_parts[e.layer]
            for part in (mixer, ffn):
                if part is not None and hasattr(part, "weight_bytes"):
                    total += part.weight_bytes()
            for n in (norm1, norm2, *self._extra_norms[e.layer].values()):
                if getattr(n, "weight", None) is not None:
                    total += n.weight.numel() * n.weight.element_size()
        return total

    # ---- forward --------------------------------------------------------------------------
    def cut_by_length(self, pos0, cache) -> bool:
        """Does any mixer want this one-token step (positions of the live sequences) cut by length?
        Each is asked with the view of the cache that its layer reads."""
        if self._cut_askers is None:
            # every mixer that has the (optional) method, one per `cut_by_length_key()` where mixers
            # say that their answers are the same (layers of equal shape): asked every step
            seen, self._cut_askers = set(), []
            for pos, e in enumerate(self.spec.schedule):
                mixer = self._layer_parts[e.layer][1]
                ask = getattr(mixer, "cut_by_length", None)
                if ask is None:
                    continue
                key = getattr(mixer, "cut_by_length_key", lambda m=mixer: id(m))()
                if key not in seen:
                    seen.add(key)
                    self._cut_askers.append((ask, self.spec.cache_entry(pos)))
        return any(ask(pos0, cache.layer_view(entry)) for ask, entry in self._cut_askers)

    def forward(self, ctx: StepContext, tokens: torch.Tensor, cache, logit_rows: Optional[torch.Tensor],
                n_logit_rows: int, logits_out: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Run the step's tokens through the scheduled layers.

        tokens      int32 [n_tokens] on the device
        logit_rows  int32 [n_logit_rows] on the device: packed-token rows whose logits are wanted
        Returns float32 [n_logit_rows, vocab] (None when no row is wanted)."""
        rt, spec, ws = self.rt, self.spec, self.rt.workspace
        T, H = ctx.n_tokens, spec.hidden_size
        x = ws.take("model.residual", (T, H), torch.float32)
        sched = spec.schedule
        # the first block's first norm may ask the embedding kernel for its element-wise half
        # (not when step inputs may still change the embedded rows)
        request = first_norm_request_of(self.blocks[sched[0].layer], ctx) if sched and not self.inputs else None
        ahead = finish = None
        if request is not None:
            from ..parts.norm import honour
            ahead, finish = honour(request, x, ctx, "embed", 1)
        B.embed_gather(self.embedding, tokens, x, spec.embedding_scale, rt.err, ctx.stream, ahead=ahead)
        ctx.rows_ahead = finish() if finish is not None else None
        for part, _ in self.inputs:
            part.prepare(tokens, x, ctx)
        for pos, e in enumerate(sched):
            view = cache.layer_view(spec.cache_entry(pos))
            ctx.next_block = self.blocks[sched[pos + 1].layer] if pos + 1 < len(sched) else None
            self.blocks[e.layer].forward(x, ctx, view, e.writes_cache)
        ctx.rows_ahead = None
        if n_logit_rows == 0:
            return None
        hn = ws.take("model.head_in", (n_logit_rows, H), rt.dtype)
        self.final_norm.forward(x, hn, ctx, rows_idx=logit_rows, rows=n_logit_rows)
        if logits_out is None:
            logits_out = torch.empty((n_logit_rows, spec.vocab_size), dtype=torch.float32, device=rt.device)
        self.lm_head.forward(hn, logits_out, n_logit_rows, ctx)
        return logits_out
