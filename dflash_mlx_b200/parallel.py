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
    # KV heads are split while there are at least as many as ranks, else each is replicated on world / kv_heads
    # ranks; any other ratio would pair a rank's query heads with a wrong (or missing) KV head.
    if cfg.kv_heads % world != 0 and world % cfg.kv_heads != 0:
        raise ValueError(f"kv_heads={cfg.kv_heads} and {world} ranks: one must divide the other")
    c.kv_heads = max(1, cfg.kv_heads // world)
    if c.q_heads % c.kv_heads != 0:
        raise ValueError("query heads per rank must be a multiple of KV heads per rank")
    c.intermediate = _round_up(-(-cfg.intermediate // world), 8 * cfg.group_size)
    # equal vocabulary shards: a rank's global token id is its local index + rank * vocab_offset_stride
    if cfg.vocab % world != 0:
        raise ValueError(f"vocab={cfg.vocab} is not divisible by {world} ranks (pad lm_head to equal shards)")
    c.vocab = cfg.vocab // world
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


def _rows(Wq, idx):
    """Column-parallel slice of a quantised linear: output rows ``idx``."""
    return {"w": Wq["w"][idx].contiguous(), "s": Wq["s"][idx].contiguous(), "b": Wq["b"][idx].contiguous()}


def _rows_padded(Wq, idx, n_rows):
    """Rows ``idx`` followed by zero rows (zero codes, scales and biases: they produce exact zeros) up to ``n_rows``."""
    out = {}
    for k in ("w", "s", "b"):
        t = Wq[k][idx]
        if n_rows > t.shape[0]:
            t = torch.cat([t, torch.zeros(n_rows - t.shape[0], t.shape[1], dtype=t.dtype, device=t.device)], dim=0)
        out[k] = t
    return out


def _cols(Wq, k0, k1, group_size, pad_to=None):
    """Row-parallel slice of a quantised linear: input columns [k0, k1) (multiples of the group size), optionally
    zero-padded on the right to ``pad_to`` columns (zero codes, zero scale and bias)."""
    assert k0 % group_size == 0 and k1 % group_size == 0
    w = Wq["w"][:, k0 // 8:k1 // 8]
    s = Wq["s"][:, k0 // group_size:k1 // group_size]
    b = Wq["b"][:, k0 // group_size:k1 // group_size]
    if pad_to is not None and pad_to > k1 - k0:
        extra = pad_to - (k1 - k0)
        w = torch.cat([w, torch.zeros(w.shape[0], extra // 8, dtype=w.dtype, device=w.device)], dim=1)
        s = torch.cat([s, torch.zeros(s.shape[0], extra // group_size, dtype=s.dtype, device=s.device)], dim=1)
        b = torch.cat([b, torch.zeros(b.shape[0], extra // group_size, dtype=b.dtype, device=b.device)], dim=1)
    return {"w": w.contiguous(), "s": s.contiguous(), "b": b.contiguous()}


def _arange(a, b, device):
    return torch.arange(a, b, device=device)


def shard_weights(cfg, W, rank: int, world: int):
    """Cuts rank ``rank``'s tensor-parallel shard out of a full set of weights (the dict ``init_weights`` makes).
    Returns ``(local_cfg, local_weights)``.  Requires head counts divisible by ``world`` and an MLP intermediate
    whose per-rank share is a whole number of quantisation groups; the share is padded with zero rows (gate|up) and
    zero columns (down) up to the multiple of 8 groups that ``shard_config`` gives the local shape."""
    lc = shard_config(cfg, world)
    if world == 1:
        return lc, W
    G, dev = cfg.group_size, W["norm"].device
    moe = getattr(cfg, "moe_experts", 0) > 0
    if not moe and (cfg.intermediate % world != 0 or (cfg.intermediate // world) % G != 0):
        raise ValueError("shard_weights needs intermediate/world to be a whole number of quantisation groups")
    I, Il = cfg.intermediate, cfg.intermediate // world
    Ilp = lc.intermediate                      # padded local width (a multiple of 8 groups)
    if moe:
        # expert parallel: a contiguous range of routed experts per rank, the shared expert on rank 0, router replicated
        if cfg.moe_experts % world != 0:
            raise ValueError("shard_weights needs the number of experts to be divisible by the ranks")
        per = cfg.moe_experts // world
        lc.moe_e_lo, lc.moe_e_hi, lc.moe_shared_here = rank * per, (rank + 1) * per, rank == 0
    D, Hq, Hkv = cfg.head_dim, cfg.q_heads, cfg.kv_heads
    hq0, hq1 = rank * lc.q_heads, (rank + 1) * lc.q_heads
    kv0 = (rank * Hkv) // world if Hkv >= world else hq0 // (Hq // Hkv)
    kv1 = kv0 + lc.kv_heads
    Hk, Hv, Dk, Dv = cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_dk, cfg.gdn_dv
    gk0, gk1 = rank * lc.gdn_k_heads, (rank + 1) * lc.gdn_k_heads
    gv0, gv1 = rank * lc.gdn_v_heads, (rank + 1) * lc.gdn_v_heads
    layers = []
    for i, L in enumerate(W["layers"]):
        o = {"in_norm": L["in_norm"], "post_norm": L["post_norm"]}
        if moe:
            from .moe import slice_experts
            gu_l, dn_l = slice_experts(L["experts_gate_up"], L["experts_down"], cfg.moe_experts, cfg.moe_inter, cfg.hidden,
                                       lc.moe_e_lo, lc.moe_e_hi, lc.moe_shared_here)
            o.update(router=L["router"], experts_gate_up=gu_l, experts_down=dn_l)
        else:
            gate = _rows_padded(L["gate_up"], _arange(rank * Il, (rank + 1) * Il, dev), Ilp)
            up = _rows_padded(L["gate_up"], _arange(I + rank * Il, I + (rank + 1) * Il, dev), Ilp)
            o.update(gate_up={k: torch.cat([gate[k], up[k]], dim=0).contiguous() for k in ("w", "s", "b")},
                     down=_cols(L["down"], rank * Il, (rank + 1) * Il, G, pad_to=Ilp))
        if cfg.is_attention(i):
            idx = torch.cat([_arange(hq0 * 2 * D, hq1 * 2 * D, dev),
                             _arange(2 * Hq * D + kv0 * D, 2 * Hq * D + kv1 * D, dev),
                             _arange(2 * Hq * D + Hkv * D + kv0 * D, 2 * Hq * D + Hkv * D + kv1 * D, dev)])
            ko = lc.q_heads * D
            o.update(proj=_rows(L["proj"], idx), q_norm=L["q_norm"], k_norm=L["k_norm"],
                     o_proj=_cols(L["o_proj"], hq0 * D, hq1 * D, G, pad_to=_round_up(ko, 8 * G)))
        else:
            kd = Hk * Dk
            cd = cfg.conv_dim
            zo = cd
            bo = zo + Hv * Dv
            ao = bo + Hv
            ch = torch.cat([_arange(gk0 * Dk, gk1 * Dk, dev), _arange(kd + gk0 * Dk, kd + gk1 * Dk, dev),
                            _arange(2 * kd + gv0 * Dv, 2 * kd + gv1 * Dv, dev)])
            idx = torch.cat([ch, _arange(zo + gv0 * Dv, zo + gv1 * Dv, dev), _arange(bo + gv0, bo + gv1, dev),
                             _arange(ao + gv0, ao + gv1, dev)])
            o.update(proj=_rows(L["proj"], idx), conv_w=L["conv_w"][ch].contiguous(), A_log=L["A_log"][gv0:gv1].contiguous(),
                     dt_bias=L["dt_bias"][gv0:gv1].contiguous(), g_norm=L["g_norm"],
                     out_proj=_cols(L["out_proj"], gv0 * Dv, gv1 * Dv, G))
        layers.append(o)
    v0 = rank * lc.vocab
    v1 = min(cfg.vocab, v0 + lc.vocab)
    lm = _rows(W["lm_head"], _arange(v0, v1, dev))
    return lc, {"layers": layers, "embed": W["embed"], "norm": W["norm"], "lm_head": lm}


def shard_caches(cfg, caches, rank: int, world: int):
    """The matching slice of the recurrent / KV caches (oracle-style dict of per-layer tensors)."""
    if world == 1:
        return caches
    lc = shard_config(cfg, world)
    Hk, Hv, Dk, Dv = cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_dk, cfg.gdn_dv
    gk0, gk1 = rank * lc.gdn_k_heads, (rank + 1) * lc.gdn_k_heads
    gv0, gv1 = rank * lc.gdn_v_heads, (rank + 1) * lc.gdn_v_heads
    kd = Hk * Dk
    dev = caches["conv"][0].device if caches["conv"] else None
    kv0 = (rank * cfg.kv_heads) // world if cfg.kv_heads >= world else (rank * lc.q_heads) // (cfg.q_heads // cfg.kv_heads)
    out = {"conv": [], "state": [], "k": [], "v": []}
    for c in caches["conv"]:
        ch = torch.cat([_arange(gk0 * Dk, gk1 * Dk, dev), _arange(kd + gk0 * Dk, kd + gk1 * Dk, dev),
                        _arange(2 * kd + gv0 * Dv, 2 * kd + gv1 * Dv, dev)])
        out["conv"].append(c[:, ch].contiguous())
    for s in caches["state"]:
        out["state"].append(s[gv0:gv1].contiguous())
    for k in caches["k"]:
        out["k"].append(k[kv0:kv0 + lc.kv_heads].contiguous())
    for v in caches["v"]:
        out["v"].append(v[kv0:kv0 + lc.kv_heads].contiguous())
    return out


class PeerReducer:
    """Row-parallel sum + residual add + RMSNorm in ONE kernel over peer-mapped memory (NVLink), in place of an NCCL
    all-reduce followed by the add/norm kernel.  Every rank owns an inbox and a flag array allocated by the library
    (``cudaMalloc``), exports them through CUDA IPC and maps the other ranks' copies; the kernel pushes this rank's
    partial block into every inbox, publishes per-row flags, waits (bounded) for the other ranks' rows and finishes
    the residual add and the norm.  ``group`` is only used at set-up, to exchange the 64-byte IPC handles.

    world == 1 works without any process group (the kernel pushes to its own inbox): that is what a single-GPU
    test exercises."""

    def __init__(self, rank: int, world: int, rows: int, hidden: int, device, group=None, _wire=None):
        import ctypes

        from . import _lib
        self.lib = _lib.lib()
        self._ct = ctypes
        c = ctypes
        vp, i32, sz = c.c_void_p, c.c_int, c.c_size_t
        _lib.declare("dflash_peer_inbox_bytes", sz, [i32, i32, i32])
        _lib.declare("dflash_peer_flags_bytes", sz, [i32, i32])
        _lib.declare("dflash_peer_alloc", i32, [sz, c.POINTER(vp)])
        _lib.declare("dflash_peer_free", i32, [vp])
        _lib.declare("dflash_peer_export", i32, [vp, c.c_char_p])
        _lib.declare("dflash_peer_open", i32, [c.c_char_p, c.POINTER(vp)])
        _lib.declare("dflash_peer_close", i32, [vp])
        _lib.declare("dflash_peer_set_wait_polls", None, [c.c_uint])
        _lib.declare("dflash_peer_set_protocol", None, [i32])
        _lib.declare("dflash_peer_reduce_add_rmsnorm", i32,
                     [vp, c.POINTER(vp), c.POINTER(vp), i32, i32, vp, vp, vp, vp, i32, i32, c.c_float, i32, vp])
        self._check = _lib.check
        import os
        if os.environ.get("DFLASH_PEER_PROTOCOL", "") in ("0", "1", "2"):      # hand-over protocol, see set_protocol
            self.lib.dflash_peer_set_protocol(int(os.environ["DFLASH_PEER_PROTOCOL"]))
        self.rank, self.world, self.rows, self.hidden = rank, world, rows, hidden
        self.dev = torch.device(device)
        self._own, self._opened = [], []
        with torch.cuda.device(self.dev):
            nb_in = self.lib.dflash_peer_inbox_bytes(world, rows, hidden)
            nb_fl = self.lib.dflash_peer_flags_bytes(world, rows)
            if nb_in == 0 or nb_fl == 0:
                raise ValueError("PeerReducer: world 1..8, hidden a multiple of 8")
            if _wire is not None:        # buffers of every rank live in this process (see local_group)
                self._inbox = (vp * world)(*_wire[0])
                self._flags = (vp * world)(*_wire[1])
                return
            inbox, flags = vp(), vp()
            self._check(self.lib.dflash_peer_alloc(nb_in, c.byref(inbox)), "dflash_peer_alloc")
            self._own.append(inbox.value)
            self._check(self.lib.dflash_peer_alloc(nb_fl, c.byref(flags)), "dflash_peer_alloc")
            self._own.append(flags.value)
            inbox_ptrs, flag_ptrs = [None] * world, [None] * world
            inbox_ptrs[rank], flag_ptrs[rank] = inbox.value, flags.value
            if world > 1:
                import torch.distributed as dist
                h_in, h_fl = c.create_string_buffer(64), c.create_string_buffer(64)
                self._check(self.lib.dflash_peer_export(inbox, h_in), "dflash_peer_export")
                self._check(self.lib.dflash_peer_export(flags, h_fl), "dflash_peer_export")
                gathered = [None] * world
                dist.all_gather_object(gathered, (rank, h_in.raw, h_fl.raw), group=group)
                for (r, hi, hf) in gathered:
                    if r == rank:
                        continue
                    pi, pf = vp(), vp()
                    self._check(self.lib.dflash_peer_open(hi, c.byref(pi)), "dflash_peer_open")
                    self._opened.append(pi.value)
                    self._check(self.lib.dflash_peer_open(hf, c.byref(pf)), "dflash_peer_open")
                    self._opened.append(pf.value)
                    inbox_ptrs[r], flag_ptrs[r] = pi.value, pf.value
                dist.barrier(group=group)        # every rank has mapped every buffer before the first push
            self._inbox = (vp * world)(*inbox_ptrs)
            self._flags = (vp * world)(*flag_ptrs)

    @classmethod
    def local_group(cls, world: int, rows: int, hidden: int, device):
        """``world`` reducers whose inboxes all live on ONE device of this process, wired to each other by plain device
        pointers.  Their kernels must not be launched so that one waits for another (launches of one GPU are not
        guaranteed to run at the same time): use it with a short wait limit, for tests of the data path and of the
        give-up path."""
        first = cls(0, world, rows, hidden, device, _wire=([None] * world, [None] * world))
        c, lib = first._ct, first.lib
        inboxes, flags = [], []
        with torch.cuda.device(first.dev):
            for _ in range(world):
                a, b = c.c_void_p(), c.c_void_p()
                first._check(lib.dflash_peer_alloc(lib.dflash_peer_inbox_bytes(world, rows, hidden), c.byref(a)), "dflash_peer_alloc")
                first._check(lib.dflash_peer_alloc(lib.dflash_peer_flags_bytes(world, rows), c.byref(b)), "dflash_peer_alloc")
                inboxes.append(a.value)
                flags.append(b.value)
        group = [cls(r, world, rows, hidden, device, _wire=(inboxes, flags)) for r in range(world)]
        group[0]._own = inboxes + flags
        return group

    def set_protocol(self, protocol: int) -> None:
        """0 = by rank count (default), 1 = 8-byte {data, sequence} entries, 2 = vector pushes + fence + flags.  Process-wide;
        every rank must choose the same."""
        self.lib.dflash_peer_set_protocol(int(protocol))

    def set_wait_polls(self, polls: int) -> None:
        """Bound of the device-side wait for the other ranks' rows (a poll is roughly half a microsecond)."""
        self.lib.dflash_peer_set_wait_polls(int(polls))

    def reduce_add_rmsnorm(self, delta: torch.Tensor, h: torch.Tensor, w: torch.Tensor, x: torch.Tensor, eps: float,
                           dtype_code: int) -> None:
        """h += sum over ranks of delta;  x = rmsnorm(h) * w  (h is updated in place)."""
        st = torch.cuda.current_stream(self.dev).cuda_stream
        rc = self.lib.dflash_peer_reduce_add_rmsnorm(delta.data_ptr(), self._inbox, self._flags, self.rank, self.world,
                                                     h.data_ptr(), w.data_ptr(), h.data_ptr(), x.data_ptr(), self.rows,
                                                     self.hidden, eps, dtype_code, st)
        self._check(rc, "dflash_peer_reduce_add_rmsnorm")

    def close(self) -> None:
        """Unmaps the peers' buffers and frees this rank's (call after a barrier: no rank may still push)."""
        with torch.cuda.device(self.dev):
            torch.cuda.synchronize(self.dev)
            for p in self._opened:
                self.lib.dflash_peer_close(p)
            for p in self._own:
                self.lib.dflash_peer_free(p)
        self._opened, self._own = [], []
