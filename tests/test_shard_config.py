"""Host-side checks of the tensor-parallel sharder: configurations it cannot shard correctly are refused, and the
vocabulary shards it does make tile the vocabulary exactly (the global token id of a rank's local winner is
``local + rank * vocab_offset_stride``)."""
import pytest
import torch

from dflash_mlx_b200 import parallel
from dflash_mlx_b200.verify_step import HybridConfig, init_weights


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


def test_mlp_share_is_padded_with_exact_zeros():
    """intermediate / ranks need not be a multiple of 8 groups: gate|up gets zero rows, down zero columns, so the padded
    shard computes exactly what the unpadded one would (the dense model's 17408 over 4 or 8 ranks)."""
    from oracle import qmm as oq
    cfg = _cfg(intermediate=1280, layers=1, attn_every=4)      # 1280 / 2 = 640 = 10 groups -> padded to 1024
    W = init_weights(cfg, 3, "cpu")
    world = 2
    x = torch.randn(4, cfg.hidden, generator=torch.Generator().manual_seed(1)).bfloat16()
    full_gu = oq.qmm_ref(x, W["layers"][0]["gate_up"]["w"], W["layers"][0]["gate_up"]["s"], W["layers"][0]["gate_up"]["b"],
                         64, out_dtype=torch.float32)
    I = cfg.intermediate
    act = (torch.nn.functional.silu(full_gu[:, :I]) * full_gu[:, I:]).bfloat16()
    D = W["layers"][0]["down"]
    want = oq.qmm_ref(act, D["w"], D["s"], D["b"], 64, out_dtype=torch.float32)
    total = torch.zeros_like(want)
    for r in range(world):
        lc, lw = parallel.shard_weights(cfg, W, r, world)
        assert lc.intermediate == 1024
        gu, dn = lw["layers"][0]["gate_up"], lw["layers"][0]["down"]
        assert gu["w"].shape[0] == 2 * 1024 and dn["w"].shape[1] * 8 == 1024
        assert not gu["w"][640:1024].any() and not gu["s"][640:1024].any() and not gu["w"][1024 + 640:].any()
        y = oq.qmm_ref(x, gu["w"], gu["s"], gu["b"], 64, out_dtype=torch.float32)
        a = (torch.nn.functional.silu(y[:, :1024]) * y[:, 1024:]).bfloat16()
        assert not a[:, 640:].any()
        total += oq.qmm_ref(a, dn["w"], dn["s"], dn["b"], 64, out_dtype=torch.float32)
    assert torch.allclose(total, want, rtol=1e-4, atol=1e-4)
