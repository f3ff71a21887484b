"""Host-side checks of the tensor-parallel sharder: configurations it cannot shard correctly are refused, and the
vocabulary shards it does make tile the vocabulary exactly (the global token id of a rank's local winner is
``local + rank * vocab_offset_stride``)."""
import pytest
import torch

from dflash_mlx_b200 import parallel
from dflash_mlx_b200.verify_step import HybridConfig


def _cfg(**kw):
    base = dict(layers=4, hidden=512, intermediate=2048, q_heads=8, kv_heads=4, head_dim=128, gdn_k_heads=4,
                gdn_v_heads=8, vocab=1024, max_context=256)
    base.update(kw)
    return HybridConfig(**base)


def test_vocab_must_split_evenly():
    with pytest.raises(ValueError, match="vocab"):
        parallel.shard_config(_cfg(vocab=1001), 2)
    lc = parallel.shard_config(_cfg(vocab=1024), 4)
    assert lc.vocab == 256 and lc.vocab_offset_stride == 256


@pytest.mark.parametrize("kv,world,ok", [(4, 2, True), (4, 4, True), (4, 8, True), (2, 8, True), (4, 3, False),
                                         (6, 4, False), (3, 2, False)])
def test_kv_heads_against_ranks(kv, world, ok):
    cfg = _cfg(kv_heads=kv, q_heads=24, gdn_k_heads=24, gdn_v_heads=24, vocab=24 * 64)
    if ok:
        lc = parallel.shard_config(cfg, world)
        assert lc.kv_heads == max(1, kv // world)
        assert lc.q_heads * world == cfg.q_heads
    else:
        with pytest.raises(ValueError):
            parallel.shard_config(cfg, world)


def test_heads_must_divide():
    with pytest.raises(ValueError):
        parallel.shard_config(_cfg(q_heads=6), 4)


def test_vocab_shards_tile_the_vocabulary_and_kv_pairing():
    """Every lm_head row lands on exactly one rank at local index = global - rank * stride, and with more ranks than KV
    heads each rank's query heads keep the KV head the unsharded model pairs them with."""
    from dflash_mlx_b200.verify_step import init_weights
    cfg = _cfg(kv_heads=2, q_heads=8, vocab=512)
    W = init_weights(cfg, 3, "cpu")
    world = 4
    rows = []
    for r in range(world):
        lc, lw = parallel.shard_weights(cfg, W, r, world)
        assert lw["lm_head"]["w"].shape[0] == lc.vocab == lc.vocab_offset_stride
        rows.append(lw["lm_head"]["w"])
        g0 = r * lc.vocab_offset_stride
        assert torch.equal(lw["lm_head"]["w"], W["lm_head"]["w"][g0:g0 + lc.vocab])
        # attention layer 3: rank r holds query heads [2r, 2r+2) -> KV head (2r) // (8 // 2) = r // 2
        D, Hq, Hkv = cfg.head_dim, cfg.q_heads, cfg.kv_heads
        proj = lw["layers"][3]["proj"]["w"]
        kv = (r * lc.q_heads) // (Hq // Hkv)
        k_rows = W["layers"][3]["proj"]["w"][2 * Hq * D + kv * D: 2 * Hq * D + (kv + 1) * D]
        assert torch.equal(proj[2 * lc.q_heads * D: 2 * lc.q_heads * D + D], k_rows)
    assert torch.equal(torch.cat(rows), W["lm_head"]["w"])
