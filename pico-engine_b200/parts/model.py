"""The decoder assembled from a plan: embedding, the schedule of layer executions, final norm
and the head that gives logits at the wanted rows."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..cache import CacheNeeds
from ..config.specs import ModelPlan
from ..ops import kernels, linear
from ..weights.loader import ParamSpec
from .base import NORMS, STREAM_POSITIONS, StepContext, build_part
from .block import Layer


class DecoderModel:
    """pico-engine's forward (src/pico_engine/model.py:146-165) for a batch of packed tokens:
    embed, run the schedule, norm the wanted rows, project them to the vocabulary."""

    def __init__(self, plan: ModelPlan, dtype: torch.dtype, device):
        plan.validate()
        self.plan, self.dtype, self.device = plan, dtype, torch.device(device) if device != "meta" else device
        self.layers: List[Layer] = [Layer(s, dtype, self.device) for s in plan.layers]
        self.final_norm = build_part(NORMS, "norm", plan.final_norm, dtype, self.device)
        self.embedding_position = None if plan.embedding_position is None else \
            build_part(STREAM_POSITIONS, "stream position", plan.embedding_position, dtype, self.device)
        self.stream_vectors: Dict[str, torch.Tensor] = {}      # [rows, hidden] tensors whose rows schedule entries add to the stream
        self._keeps_embedding = any(e.add_embedding for e in plan.schedule)
        self.embedding: Optional[torch.Tensor] = None
        self.pair_table: Optional[torch.Tensor] = None         # rows added to the embedding by (previous token, token)
        self.head: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------ weights
    def _parts(self):
        for layer in self.layers:
            yield from layer.parts()
        yield self.final_norm
        if self.embedding_position is not None:
            yield self.embedding_position

    def expected_tensors(self) -> Dict[str, ParamSpec]:
        p = self.plan
        out = {p.embedding: ParamSpec((p.vocab_size, p.hidden_size))}
        for part in self._parts():
            out.update(part.expected_tensors())
        if p.head is not None:
            out[p.head] = ParamSpec((p.vocab_size, p.hidden_size))
        for name, rows in p.stream_vectors:
            out[name] = ParamSpec((rows, p.hidden_size))
        if p.embedding_pairs is not None:
            out[p.embedding_pairs.table] = ParamSpec((p.embedding_pairs.buckets + 1, p.hidden_size))
        return out

    def take_tensors(self, get) -> None:
        self.embedding = get(self.plan.embedding)
        for part in self._parts():
            part.take_tensors(get)
        self.head = self.embedding if self.plan.head is None else get(self.plan.head)
        self.stream_vectors = {name: get(name) for name, _ in self.plan.stream_vectors}
        if self.plan.embedding_pairs is not None:
            self.pair_table = get(self.plan.embedding_pairs.table).to(self.embedding.dtype).contiguous()

    def prepare(self, max_positions: int) -> None:
        for part in self._parts():
            part.prepare(max_positions)

    # ------------------------------------------------------------------ cache
    def cache_needs(self) -> List[Optional[CacheNeeds]]:
        """Per schedule entry; None for an entry that reads another entry's cache.  Behind the schedule's entries comes what
        the model itself keeps per sequence: the token before the next one (int32), where the embedding reads pairs."""
        needs = [None if e.cache_of is not None else self.layers[e.layer].cache_needs() for e in self.plan.schedule]
        if self.plan.embedding_pairs is not None:
            needs.append(CacheNeeds(state_elems=1, state_dtype="int32"))
        return needs

    # ------------------------------------------------------------------ a step
    def hidden(self, token_ids: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        """The residual stream [T, hidden] float32 after the last layer."""
        pairs = self.plan.embedding_pairs
        if pairs is None:
            x = kernels.embed(self.embedding, token_ids, scale=self.plan.embedding_scale)
        else:
            x = kernels.embed_pairs(self.embedding, self.pair_table, token_ids, ctx.tok_pos, ctx.tok_row, ctx.row_first, ctx.slots,
                                    ctx.state(len(self.plan.schedule)), pairs.buckets, pairs.mul_prev, pairs.mul_cur)
        if self.embedding_position is not None:
            self.embedding_position.add_to(x, ctx)
        x0 = x.clone() if self._keeps_embedding else None
        for e, entry in enumerate(self.plan.schedule):
            cache_entry = e if entry.cache_of is None else entry.cache_of
            if entry.add_embedding or entry.add_vector is not None:
                ctx.settle(x)
                vec = None if entry.add_vector is None else self.stream_vectors[entry.add_vector[0]][entry.add_vector[1]]
                kernels.add_rows(x, x0 if entry.add_embedding else None, vec)
            self.layers[entry.layer].run(x, ctx, e, cache_entry, entry.cache_of is None)
        ctx.settle(x)
        return x

    def logits(self, x: torch.Tensor, rows_index: torch.Tensor) -> torch.Tensor:
        """float32 logits [len(rows_index), vocab] of the rows ``rows_index`` of ``x``."""
        h = self.final_norm.forward(x, self.dtype, rows_index)
        logits = linear(h, self.head, out_dtype=torch.float32)
        if self.plan.logit_softcap:
            kernels.softcap(logits, self.plan.logit_softcap)
        return logits

    def forward(self, token_ids: torch.Tensor, ctx: StepContext, rows_index: torch.Tensor) -> torch.Tensor:
        return self.logits(self.hidden(token_ids, ctx), rows_index)

    def step_weight_bytes(self) -> int:
        """Bytes of weights a step reads in full: every matrix and vector of every executed layer
        and the head; the embedding table only where it is the head too (a lookup reads a row a token)."""
        seen, total = set(), 0
        tensors = [self.head] + list(self.final_norm.weights())      # (the pair table, like the embedding, is read a row a token)
        for entry in self.plan.schedule:
            for part in self.layers[entry.layer].parts():
                tensors.extend(part.weights())
        for t in tensors:
            if t is not None and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        return total
