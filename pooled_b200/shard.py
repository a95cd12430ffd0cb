"""KV-sequence-sharded decode across the GPUs of one box (one process per GPU, torch.distributed).

Each rank keeps a contiguous chunk of every sequence's K/V rows in its own layer caches: rank r of P holds global
rows [r * chunk, (r + 1) * chunk).  A decode step runs the ordinary split-K kernel on the rank's rows, which leaves
one (o, m, l) record per (sequence, head); the ranks all-gather their record blocks (NCCL over NVLink; about
head_dim + 2 floats per row, so the exchange is latency-, not bandwidth-bound) and every rank merges them with the
same LSE combine the single-GPU path uses, gate included.  The new token's K/V row is appended by the rank that owns
its position.  pooled itself never shards attention (it is pipeline-parallel over layers); the merge is the
arithmetic of its attn_dec_combine (engine/wgsl/attn_dec.js:215-287) applied across GPUs instead of across splits.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class ShardPlan:
    """Contiguous chunks of `chunk` rows per rank."""
    world: int
    chunk: int

    def owner(self, pos: int) -> int:
        r = pos // self.chunk
        if r >= self.world:
            raise ValueError(f"position {pos} is past the {self.world} x {self.chunk} rows the ranks hold")
        return r

    def local_rows(self, rank: int, n_rows: int) -> int:
        """How many of the global rows [0, n_rows) rank holds."""
        return max(0, min(self.chunk, n_rows - rank * self.chunk))

    def local_pos(self, rank: int, pos: int) -> int:
        return pos - rank * self.chunk

    def block_columns(self, rank: int, pos: int, n_cols: int) -> tuple[int, int]:
        """Columns [c_lo, c_hi) of a k-token block at pos .. pos + n_cols - 1 whose rows rank holds (empty when
        c_lo >= c_hi).  A block that straddles a chunk boundary is appended in two parts, each by its owner; this is
        the rule pa_attn_layer_sharded applies."""
        lo, hi = rank * self.chunk, (rank + 1) * self.chunk
        c_lo = 0 if pos >= lo else min(lo - pos, n_cols)
        c_hi = n_cols if pos + n_cols <= hi else (0 if pos >= hi else hi - pos)
        return c_lo, c_hi


class ShardedDecoder:
    """One decode step of a sharded layer.  `engine` needs set_origin(), rope(), rope_append(), decode_partial() and
    merge() with AttnEngine's signatures (rope_append_items() is used when it is there); `dist` is torch.distributed (or a stand-in with all_gather_into_tensor).
    Every position stays global: the engine's layers are told which global row their cache starts at."""

    def __init__(self, engine, plan: ShardPlan, rank: int, dist, group=None, exchange: str = "nccl"):
        """exchange: "nccl" (all-gather of the record blocks, then pa_merge) or "peer" (pa_decode_exchange: the combine
        kernel itself stores the records into every rank's buffer over NVLink and merges; needs engine.exchange_setup)."""
        self.eng, self.plan, self.rank, self.dist, self.group, self.exchange = engine, plan, rank, dist, group, exchange
        # a layer's extent is its max_seq: a longer cache would make this rank attend (and append) rows of the next
        # rank's chunk as well, and the merge would count those positions twice
        if engine.cfg.max_seq != plan.chunk:
            raise ValueError(f"sharded decode needs layer caches of exactly one chunk: max_seq {engine.cfg.max_seq} != chunk {plan.chunk}")
        for li in range(engine.cfg.n_layers):
            engine.set_origin(li, rank * plan.chunk)

    def step(self, li: int, seqs_pos, q, k, v, gate, out=None, gather_buf=None):
        """seqs_pos: [(seq, global position of the new token)], one token per sequence; q/k/v/gate: [n_seqs, ...]
        on every rank (the projections are replicated).  Returns out [n_seqs, q_dim] on every rank."""
        eng, plan = self.eng, self.plan
        n = len(seqs_pos)
        if self.exchange == "peer" and n == 1:      # one sequence: the whole layer step is one library call
            return eng.encode_layer_sharded(li, seqs_pos[0][1], q, k, v, gate, out, seq=seqs_pos[0][0])
        if self.exchange == "peer" and hasattr(eng, "encode_items"):   # ... and so is a batch of sequences
            return eng.encode_items(li, seqs_pos, q, k, v, gate, out, sharded=True)
        if n > 1 and hasattr(eng, "rope_append_items"):
            # every sequence's token in one launch; rows of other shards get their q rotated only
            q_rot = eng.rope_append_items(li, seqs_pos, q, k, v)
        else:
            q_rot = []
            for i, (seq, pos) in enumerate(seqs_pos):
                if plan.owner(pos) == self.rank:   # this rank owns the new row: rotate q and k, append k and v
                    q_rot.append(eng.rope_append(li, seq, pos, q[i:i + 1], k[i:i + 1], v[i:i + 1]))
                else:
                    q_rot.append(eng.rope(q[i:i + 1], eng.cfg.n_heads, pos))
            q_rot = q_rot[0] if n == 1 else _cat(q_rot)
        if self.exchange == "peer":
            return eng.decode_exchange(li, [(seq, pos, 1) for seq, pos in seqs_pos], q_rot, gate, out)
        part = eng.decode_partial(li, [(seq, pos, 1) for seq, pos in seqs_pos], q_rot)
        if plan.world == 1:
            return eng.merge(part[None], n, gate, out)
        if gather_buf is None:
            gather_buf = part.new_empty((plan.world, part.numel()))
        self.dist.all_gather_into_tensor(gather_buf.view(-1), part, group=self.group)
        return eng.merge(gather_buf, n, gate, out)


def _cat(parts):
    import torch
    return torch.cat(parts, dim=0)
