"""A model at run time: the parts of a ``ModelSpec`` with their weights on the device,
run over the tokens of one step in the order the schedule gives.

Embedding -> scheduled layers -> rows whose logits are wanted -> final norm ->
head (crates/bitnet-core/src/llama/model.rs:230-232, :236-307, :309-315).  Only
the wanted rows go through the final norm and the head.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..parts import ModelSpec, build_block, build_part
from ..weights import check_tensors


#: the key of the state area that holds every sequence's last token (for an embedding of token pairs)
PREVIOUS_TOKEN = ("model", "previous_token")


class Model:
    def __init__(self, spec: ModelSpec, tensors: Dict[str, torch.Tensor], ops):
        for n in check_tensors(spec.expected_shapes(), tensors, ignorable=spec.ignorable):
            tensors = {k: v for k, v in tensors.items() if k != n}
        self.spec, self.ops = spec, ops
        self.width, self.vocab_size = spec.width, spec.vocab_size
        dev = ops.device
        self.blocks = []
        for blk in spec.layers:
            block = build_block(blk)
            for name, part in block.parts().items():
                weights = {key: tensors[blk.names[f"{name}.{key}"]].to(dev)
                           for key in part.weight_shapes()}
                part.bind(weights, ops)
            self.blocks.append(block)
        self.embedding_scale, self.logit_scale = float(spec.embedding_scale), float(spec.logit_scale)
        self.residual_streams = int(getattr(spec, "residual_streams", 1) or 1)
        for i, block in enumerate(self.blocks):
            if int(getattr(block, "streams", 1)) != self.residual_streams:
                raise ValueError(f"layer {i} works on {getattr(block, 'streams', 1)} residual streams, the model has "
                                 f"{self.residual_streams}")
        self.final_norm = build_part("norm", spec.final_norm)
        self.final_norm.bind({k: tensors[n].to(dev) for k, n in spec.final_norm_names.items()}, ops)
        self.embedding_norm = None
        if getattr(spec, "embedding_norm", None) is not None:
            self.embedding_norm = build_part("norm", spec.embedding_norm)
            self.embedding_norm.bind({k: tensors[n].to(dev) for k, n in spec.embedding_norm_names.items()}, ops)
        self.logit_softcap = float(getattr(spec, "logit_softcap", 0.0) or 0.0)
        self.embedding = ops.prepare_embedding(tensors[spec.embedding_name])
        self.embedding_pairs = self.pair_hash = None
        pairs = getattr(spec, "embedding_pairs", None)
        if pairs is not None:
            self.embedding_pairs = ops.prepare_embedding(tensors[pairs["name"]])
            self.pair_hash = (int(pairs["buckets"]), int(pairs["mul_prev"]), int(pairs["mul_cur"]))
        if spec.head_name is None:
            self.head = ops.prepare_linear([self.embedding])     # tied: the table itself
        else:
            self.head = ops.prepare_linear([tensors[spec.head_name].to(dev)])
        for e, entry in enumerate(spec.schedule):
            if not 0 <= entry.layer < len(self.blocks):
                raise ValueError(f"schedule entry {e} names layer {entry.layer}, which does not exist")
            if entry.reads_cache_of is not None and not 0 <= entry.reads_cache_of < e:
                raise ValueError(f"schedule entry {e} may only read the cache of an earlier entry")

    @staticmethod
    def _mixer_of(block, layer: int):
        """The part of a block that may need cache or state: its one mixer (None if it has none)."""
        from ..parts.base import Mixer
        mixers = [p for p in block.parts().values() if isinstance(p, Mixer)]
        if len(mixers) > 1:
            raise ValueError(f"layer {layer} has {len(mixers)} mixers; a cache entry belongs to one run of one "
                             "mixer, so give each mixer a layer of its own")
        return mixers[0] if mixers else None

    # what the cache has to provide
    def cache_plan(self):
        from ..parts.base import Mixer
        cache_needs, reads, state_needs = {}, {}, {}
        for e, entry in enumerate(self.spec.schedule):
            mixer = self._mixer_of(self.blocks[entry.layer], entry.layer)
            if mixer is None:
                continue
            need = mixer.cache_need()
            if need is not None:
                if entry.reads_cache_of is None:
                    cache_needs[e] = need
                else:
                    reads[e] = entry.reads_cache_of
                    src = self._mixer_of(self.blocks[self.spec.schedule[entry.reads_cache_of].layer], -1)
                    theirs = src.cache_need() if src is not None else None
                    if theirs is not None and theirs.window and (not need.window or need.window > theirs.window):
                        raise ValueError(f"schedule entry {e} sees {need.window or 'all'} keys but reads the cache of "
                                         f"entry {entry.reads_cache_of}, which keeps only the last {theirs.window}")
            st = mixer.state_need()
            if st:
                state_needs[e] = st            # one StateNeed, or several by name
        # parts of a block other than its mixer that keep state per sequence (an input filter): per run of the layer
        for e, entry in enumerate(self.spec.schedule):
            for name, part in self.blocks[entry.layer].parts().items():
                if isinstance(part, Mixer):
                    continue
                need = getattr(part, "state_need", None)
                st = need() if need is not None else None
                if st:
                    state_needs[("part", e, name)] = st
        if self.embedding_pairs is not None:
            from ..parts.base import StateNeed
            state_needs[PREVIOUS_TOKEN] = StateNeed((1,), torch.int32)
        return cache_needs, reads, state_needs

    def weight_bytes(self) -> int:
        """Bytes of every matrix a step multiplies by (prepared weights of all parts, parts inside parts
        included, and float32 matrices a part keeps for itself; vectors and the embedding table are left out)."""
        from ..parts.base import Part
        seen, total, visited = set(), 0, set()

        def add(t):
            nonlocal total
            if isinstance(t, torch.Tensor) and t.dim() >= 2 and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()

        def walk(obj, depth=0):
            if id(obj) in visited or depth > 4:
                return
            visited.add(id(obj))
            if isinstance(obj, torch.Tensor):
                add(obj)
            elif isinstance(obj, dict):
                for v in obj.values():
                    walk(v, depth + 1)
            elif isinstance(obj, Part):
                for v in vars(obj).values():
                    walk(v, depth + 1)
            else:
                w = getattr(obj, "w", None)
                if isinstance(w, torch.Tensor):
                    add(w)
        add(self.head.w)
        for b in self.blocks:
            walk(b.parts())
        return total

    def forward(self, ctx) -> Optional[torch.Tensor]:
        """Runs the step's tokens; returns float32 logits [wanted rows, vocab] or None."""
        ops, meta = ctx.ops, ctx.meta
        # what parts share within ONE pass over the layers (the values a first layer leaves for later ones, say); a
        # step's meta may serve several passes (the trial run and the capture of a decode step), this dict serves one
        ctx.pass_state = {}
        if self.embedding_pairs is None:
            x = ops.embed(meta.token_ids, self.embedding, self.embedding_scale)   # float32 residual stream [T, E]
        else:
            # plus a row chosen by the pair (previous token, token); the previous token belongs to the sequence
            x = ops.embed_pairs(meta, self.embedding, self.embedding_scale, self.embedding_pairs, self.pair_hash,
                                ctx.cache.state(PREVIOUS_TOKEN))
        if self.embedding_norm is not None:
            x = self.embedding_norm.forward(ctx, x, out_dtype=torch.float32)
        s = self.residual_streams
        if s > 1:
            x = ops.streams_expand(x, s)                                      # [T, s * E]: every stream starts as the embedding
        schedule, pending = self.spec.schedule, None
        taps = getattr(ctx, "layer_outputs", None)                            # a list: the residual sum after every run of a layer
        # a schedule that adds the embedded rows again later keeps them (the blocks change x in place)
        x0 = x.clone() if any(en.adds_embedding for en in schedule) else None
        for e, entry in enumerate(schedule):
            block = self.blocks[entry.layer]
            if entry.adds_embedding:
                if pending is not None:
                    raise ValueError(f"schedule entry {e} adds the embedded rows, but the block before left its norm pending")
                ops.add_rows(x, x0)
            if getattr(block, "chains_reads", False):
                # a block that can hand the normed read of the next block's first sublayer on (see parts/block.py)
                after = self.blocks[schedule[e + 1].layer] if e + 1 < len(schedule) else None
                next_read = after.first_read() if getattr(after, "chains_reads", False) and taps is None else None
                pending = block.run(ctx, x, e, pending=pending, next_read=next_read)
                if taps is not None:
                    taps.append(ops.streams_sum(x, s) if s > 1 else x.clone())
                continue
            if getattr(block, "chains_rows", False):
                # a block whose last addition also leaves the rows in the compute dtype, which the block after reads
                # (see parts/block.py); the last block of the schedule leaves none
                after = self.blocks[schedule[e + 1].layer] if e + 1 < len(schedule) else None
                hand_on = getattr(after, "chains_rows", False) and not schedule[e + 1].adds_embedding
                pending = block.run(ctx, x, e, rows=pending, want_rows=hand_on)
                if taps is not None:
                    taps.append(x.clone())
                continue
            if not getattr(block, "chains_norms", False):
                block.run(ctx, x, e)
                pending = None
                if taps is not None:
                    taps.append(x.clone())
                continue
            # a block that can hand the rows of the next block's first norm on (see parts/block.py); not to a run
            # that adds the embedded rows first, whose norm sees another residual stream
            after = self.blocks[schedule[e + 1].layer] if e + 1 < len(schedule) else None
            hand_on = getattr(after, "chains_norms", False) and not schedule[e + 1].adds_embedding
            next_norm = after.first_norm() if hand_on else None
            pending = block.run(ctx, x, e, pending=pending, next_norm=next_norm)
            if taps is not None:
                taps.append(ops.streams_sum(x, s) if s > 1 else x.clone())
        if meta.n_want == 0:
            return None
        rows = x if meta.want_every_row else ops.gather_rows(x, meta.want_rows)
        if s > 1:
            rows = ops.streams_sum(rows, s)
        h = self.final_norm.forward(ctx, rows)
        logits = ops.linear(h, self.head, out_dtype=torch.float32, scale=self.logit_scale)
        if self.logit_softcap > 0.0:
            logits = ops.softcap(logits, self.logit_softcap)          # cap * tanh(logits / cap), float32
        return logits
