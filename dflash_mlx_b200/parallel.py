"""Tensor-parallel sharding of the verify step across the GPUs of one node (one process per GPU, NCCL).

The reference has no parallel strategy of its own beyond mirroring mlx-lm's sharded layer (one ``all_sum`` after
the GatedDeltaNet ``out_proj``, dflash_mlx/runtime.py:360-366, 449-450).  Here every mixer and MLP is
column-parallel on its input projections (query / KV / GDN heads, MLP intermediate, vocabulary are split over
ranks, no collective) and row-parallel on its output projection, followed by one all-reduce of the
``[16, hidden]`` partial sums.  KV heads are replicated when there are more ranks than KV heads.
"""
from __future__ import annotations

import copy

import torch


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


def shard_config(cfg, world: int):
    """The per-rank shape of a tensor-parallel shard.  Row-parallel input widths are rounded up to a multiple of
    8 quantisation groups (the streaming matmul's K granularity); the pad columns carry zero activations."""
    if world == 1:
        return cfg
    c = copy.copy(cfg)
    for name in ("q_heads", "gdn_k_heads", "gdn_v_heads"):
        v = getattr(cfg, name)
        if v % world != 0:
            raise ValueError(f"{name}={v} is not divisible by {world} ranks")
        setattr(c, name, v // world)
    c.kv_heads = max(1, cfg.kv_heads // world)
    if c.q_heads % c.kv_heads != 0:
        raise ValueError("query heads per rank must be a multiple of KV heads per rank")
    c.intermediate = _round_up(-(-cfg.intermediate // world), 8 * cfg.group_size)
    c.vocab = -(-cfg.vocab // world)
    c.embed_rows = cfg.vocab            # the embedding table is replicated
    c.vocab_offset_stride = c.vocab
    c.tp_world = world
    return c


def make_collectives(world: int):
    """(all_reduce, all_gather) callables over NCCL, or (None, None) for a single rank."""
    if world == 1:
        return None, None
    import torch.distributed as dist

    def all_reduce(t: torch.Tensor) -> None:
        dist.all_reduce(t)

    def all_gather(out: torch.Tensor, t: torch.Tensor) -> None:
        dist.all_gather_into_tensor(out, t)

    return all_reduce, all_gather


def shard_ranges(n: int, world: int):
    """[start, end) of each rank's slice of ``n`` items, remainder to the first ranks (used by the CPU tests)."""
    base, rem = divmod(n, world)
    out, s = [], 0
    for r in range(world):
        e = s + base + (1 if r < rem else 0)
        out.append((s, e))
        s = e
    return out
