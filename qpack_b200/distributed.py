"""Multi-GPU host logic (one process per GPU, torch.distributed for the plumbing).

Two ways of cutting the work over the GPUs of a node, neither of which exists in the single-device reference:

* rows: rows are independent samplers, GPU g takes a contiguous block of them; NO collective on the data path.
* vocabulary shards (a tensor-parallel LM head): GPU g holds the columns [g * V / G, (g + 1) * V / G) of every
  row.  Each GPU finds the exact local winners of its columns, ONE all-gather moves the (key, global id) entries
  (8 bytes each, `slots` per row and GPU), then every rank merges, filters and draws; the ids equal those of the
  reference sampler on the concatenated row.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist


def row_partition(n_rows: int, world: int, rank: int) -> Tuple[int, int]:
    """Rows [begin, end) of rank `rank`: contiguous blocks, sizes differing by at most one."""
    base, extra = divmod(n_rows, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def vocab_shard(vocab: int, world: int, rank: int, align: int = 4) -> Tuple[int, int]:
    """Columns [begin, end) of rank `rank`: contiguous, begin a multiple of `align` (16-byte aligned f32 slices)."""
    per = -(-vocab // world)
    per = -(-per // align) * align
    begin = min(vocab, rank * per)
    return begin, min(vocab, begin + per)


def gather_candidates(local: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """All-gather of the per-rank candidate entries: local [rows, slots] int64 -> [world, rows, slots]."""
    world = dist.get_world_size(group)
    out = torch.empty((world,) + tuple(local.shape), dtype=local.dtype, device=local.device)
    dist.all_gather(list(out.unbind(0)), local.contiguous(), group=group)  # works on NCCL and gloo alike
    return out


def sample_vocab_sharded(sampler, logits_shard: torch.Tensor, vocab_total: int, id_offset: int, history=None,
                         hist_len=None, max_out: int = 0, group: Optional[dist.ProcessGroup] = None):
    """One sampling step over vocabulary shards.  `sampler` provides cand_slots / local_candidates /
    merge_sample (qpack_b200.sampler.BatchSampler on a GPU).  Every rank returns the same ids."""
    world = dist.get_world_size(group)
    per_max = max(vocab_shard(vocab_total, world, r)[1] - vocab_shard(vocab_total, world, r)[0] for r in range(world))
    slots = sampler.cand_slots(vocab_total, per_max)
    local = sampler.local_candidates(logits_shard, vocab_total, id_offset, slots, history, hist_len)
    allc = gather_candidates(local, group)
    return sampler.merge_sample(allc, vocab_total, history, hist_len, max_out=max_out)
