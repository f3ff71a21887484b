"""Tensor-parallel partitioning on CPU ranks (gloo, world size 2): each rank cuts its shard out of the full
weights and caches (dflash_mlx_b200.parallel), runs the CPU oracle of the verify step with an all-reduce after every
row-parallel projection and a vocabulary-parallel greedy token, and rank 0 compares with the unsharded run."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from dflash_mlx_b200 import parallel
from oracle import model as om
from tests.test_verify_step import small_case, small_moe_case


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, moe=False):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    try:
        cfg, W, caches, ids, ctx = small_moe_case() if moe else small_case()
        lc, lw = parallel.shard_weights(cfg, W, rank, world)
        lcaches = parallel.shard_caches(cfg, caches, rank, world)
        assert lc.q_heads == cfg.q_heads // world
        if moe:   # expert parallel: half of the routed experts each, the shared expert on rank 0
            per = cfg.moe_experts // world
            assert lc.moe_local == (rank * per, (rank + 1) * per) and lc.moe_shared_here == (rank == 0)
            assert lw["layers"][0]["experts_down"]["w"].shape[0] == (per + (1 if rank == 0 else 0)) * cfg.hidden
        else:
            assert lc.intermediate == cfg.intermediate // world
        assert lw["layers"][0]["proj"]["w"].shape[0] == lc.gdn_proj_n
        assert lw["layers"][3]["proj"]["w"].shape[0] == lc.attn_proj_n

        def reduce(t):
            f = t.float()
            dist.all_reduce(f)
            return f.to(torch.bfloat16)

        def gather_tokens(vals, idx):
            pair = torch.stack([vals, (idx + rank * lc.vocab).float()], dim=1)
            allp = [torch.empty_like(pair) for _ in range(world)]
            dist.all_gather(allp, pair)
            allp = torch.stack(allp)
            best = allp[..., 0].max(dim=0).values
            pick = torch.where(allp[..., 0] == best[None], allp[..., 1], torch.full_like(allp[..., 1], 3e8)).min(dim=0).values
            return pick.to(torch.int32)

        logits, toks, new, tapes = om.verify_step_ref(lc, lw, ids, lcaches, ctx, reduce=reduce, gather_tokens=gather_tokens)
        alll = [torch.empty_like(logits) for _ in range(world)]
        dist.all_gather(alll, logits)
        if rank == 0:
            clone = {k: [t.clone() for t in v] for k, v in caches.items()}
            ref_logits, ref_toks, ref_new, ref_tapes = om.verify_step_ref(cfg, W, ids, clone, ctx)
            full = torch.cat(alll, dim=1).float()
            rel = float((full - ref_logits.float()).abs().max() / ref_logits.float().abs().max())
            assert rel <= 3e-2, rel
            rl = ref_logits.float()
            top2 = rl.topk(2, dim=-1).values
            sure = (top2[:, 0] - top2[:, 1]) > 3e-2 * rl.abs().max()
            assert torch.equal(toks[sure], ref_toks[sure])
            # the shard's GDN state / tape are exactly the head slice of the full ones for the first layer
            gv = lc.gdn_v_heads
            torch.testing.assert_close(new["state"][0], ref_new["state"][0][:gv], rtol=1e-4, atol=1e-5)
            torch.testing.assert_close(tapes[0]["tape"], ref_tapes[0]["tape"][:, :gv], rtol=1e-4, atol=1e-5)
    finally:
        dist.destroy_process_group()


def test_two_rank_tensor_parallel_matches_single_rank():
    mp.spawn(_worker, args=(2, _free_port()), nprocs=2, join=True)


def test_two_rank_expert_parallel_matches_single_rank():
    mp.spawn(_worker, args=(2, _free_port(), True), nprocs=2, join=True)


def test_shard_config_rules():
    from dflash_mlx_b200.verify_step import HybridConfig
    full = HybridConfig()
    for world in (2, 4, 8):
        c = parallel.shard_config(full, world)
        assert c.q_heads * world == full.q_heads and c.gdn_v_heads * world == full.gdn_v_heads
        assert c.kv_heads == max(1, full.kv_heads // world) and c.q_heads % c.kv_heads == 0
        assert c.intermediate % 512 == 0 and c.intermediate * world >= full.intermediate
        assert c.vocab * world >= full.vocab
    assert parallel.shard_ranges(10, 4) == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert parallel.shard_config(full, 1) is full
