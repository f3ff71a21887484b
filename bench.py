#!/usr/bin/env python
"""Benchmark of the dflash target-verify hot path on B200.

    python bench.py --gpus N --steps K --warmup W [--workload qmm_cfg1|replay|sdpa] [--impl reference]

Prints ONE JSON line (rank 0): the metric, its roofline (dominant kernel timed alone), the end-to-end figure through
the public API with host buffers, sampled clocks, a CPU baseline and, on one GPU, the single-op lines `extra`.
Workloads (synthetic, seeded; shapes of BASELINE.json's configs):
  qmm_cfg1  x bf16 [16,4096] . int4-g64 W [12288,4096]^T.  A step = one pass over a pool of weight
            matrices larger than L2 (so every launch streams its weights from HBM).
  replay    GatedDeltaNet tape replay of all 48 layers of the dense model in one launch.
  sdpa      16-row verify attention at one KV length.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

L2_BYTES = 126 * 1024 * 1024
# DRAM bytes (read + write) per algorithmic byte of the tcgen05 matmul, from an ncu capture of single launches
# (summary under profiles/: qmm_tc_kernel, configuration 1); None = not captured for this build
QMM_TC_TRAFFIC_RATIO = 0.989
QMM_TC_TRAFFIC_SOURCE = ("ncu capture of two configuration-1 launches (dram read 28.53 MB + write 0 - the 0.4 MB of output stay "
                         "in L2 - against 28.84 MB algorithmic; an earlier capture of gate|up launches gave 1.023), scaled by "
                         "algorithmic bytes; not measured at this launch mix")


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return float(d["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks / throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.gpu), "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [t.strip() for t in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx = float(f[2])
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def qmm_bytes(M, K, N, G=64):
    """Algorithmic bytes of one verify matmul: packed weights + scales + biases + x + y."""
    return N * K // 2 + 2 * (N * (K // G)) * 2 + M * K * 2 + M * N * 2


class QmmWorkload:
    """Configuration 1 of BASELINE.json.  With R ranks the output columns are split R ways (column-parallel
    linear: no collective on the data path), so the job's work is fixed: strong scaling."""
    name = "qmm_cfg1"
    metric, unit, higher_is_better, scaling, dtype = "m16_int4_verify_qmm_latency", "us", False, "strong", "bf16"
    M, K, N, G = 16, 4096, 12288, 64

    def __init__(self, rank, world, device):
        import torch
        from oracle import qmm as oq
        self.torch, self.device, self.world = torch, device, world
        self.n_local = self.N // world
        per = qmm_bytes(self.M, self.K, self.n_local, self.G)
        self.pool = max(2, (3 * L2_BYTES) // per + 1)          # pool > 3 x L2: every launch reads HBM
        self.per_launch_bytes = per
        self.ws = []
        for i in range(self.pool):
            wq, s, b = oq.random_quantized(self.n_local, self.K, seed=0xDF1A + 131 * i + rank, group_size=self.G)
            self.ws.append((wq.to(device), s.to(device), b.to(device)))
        gen = torch.Generator().manual_seed(0xDF1A)
        self.x_host = torch.randn(self.M, self.K, generator=gen).bfloat16().pin_memory()
        self.x = self.x_host.to(device)
        self.y_host = torch.empty(self.M, self.n_local, dtype=torch.bfloat16).pin_memory()
        self.launches_per_step = self.pool
        self.units_per_step = self.pool
        self.config = {"workload": self.name, "M": self.M, "K": self.K, "N": self.N, "group_size": self.G,
                       "columns_per_rank": self.n_local, "weight_pool": self.pool,
                       "l2": "inputs larger than L2: a step walks a pool of %d weight matrices (%.0f MB)" %
                             (self.pool, self.pool * per / 1e6), "parallelism": f"column-parallel x{world}"}

    def step(self):
        from dflash_mlx_b200.verify_qmm import verify_matmul
        out = None
        for w in self.ws:
            out = verify_matmul(self.x, *w, group_size=self.G, bits=4)
        return out

    def e2e_step(self):
        """One call through the public API with host buffers: x from pinned host memory, y back to the host."""
        from dflash_mlx_b200.verify_qmm import verify_matmul
        self._i = (getattr(self, "_i", -1) + 1) % self.pool
        x = self.x_host.to(self.device, non_blocking=True)
        y = verify_matmul(x, *self.ws[self._i], group_size=self.G, bits=4)
        self.y_host.copy_(y, non_blocking=True)
        self.torch.cuda.current_stream().synchronize()
        return 1

    h2d_bytes = property(lambda self: self.M * self.K * 2)
    d2h_bytes = property(lambda self: self.M * self.n_local * 2)

    def value_from_ms(self, ms_per_step):
        return ms_per_step * 1e3 / self.units_per_step      # us per matmul

    def e2e_value(self, seconds, calls):
        return seconds * 1e6 / calls

    def roofline(self, ms_per_step, aux_ms, peak, peak_src):
        us_per_launch = ms_per_step * 1e3 / self.launches_per_step
        achieved = self.per_launch_bytes / us_per_launch / 1e3
        return {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": QMM_TC_TRAFFIC_RATIO * self.per_launch_bytes if (self.world == 1 and QMM_TC_TRAFFIC_RATIO) else None,
                "traffic_source": QMM_TC_TRAFFIC_SOURCE, "peak_source": peak_src, "kernel": "qmm_tc_kernel (tcgen05)",
                "algorithmic_bytes_per_launch": self.per_launch_bytes, "us_per_launch": us_per_launch}

    def cpu_sample(self):
        """The C restatement of the stock CPU path (oracle/qmm_ref.c) on all host cores, same shape: one evaluation =
        one full-size call."""
        import torch
        from oracle import qmm as oq
        lib, kind_note = load_oracle_lib()
        wq, s, b = oq.random_quantized(self.N, self.K, seed=1, group_size=self.G)
        x = self.x_host.clone()
        y = torch.empty(self.M, self.N, dtype=torch.float32)
        args = (x.data_ptr(), wq.data_ptr(), s.data_ptr(), b.data_ptr(), y.data_ptr(), self.M, self.K, self.N, self.G)
        keep = (wq, s, b, x, y)

        def evaluate():
            t0 = time.perf_counter()
            lib.qmm_ref(*args)
            return (time.perf_counter() - t0) * 1e6, None, keep

        return evaluate, {"unit": "us", "cores": int(lib.qmm_ref_threads()), "kind": "port",
                          "sample": f"full-size calls (M=16,K=4096,N=12288); {kind_note}; MLX unavailable on this box: CPU "
                                    "baseline = C restatement of the stock qmm"}


class DenseStepWorkload:
    """Configuration 4 of BASELINE.json: one 16-token verify step of the dense hybrid model (64 layers, 3 GDN : 1
    attention, hidden 5120, SwiGLU 17408, 24 q / 4 KV heads of 256, int4 g64 linears, vocab 151936) at context
    4096, random-init weights.  GDN dimensions come from configuration 2 (16 key / 32 value heads of 128).
    With R ranks the step is tensor-parallel (heads, MLP intermediate and vocabulary split R ways, one
    all-reduce after each row-parallel matmul): strong scaling."""
    name = "dense_step_cfg4"
    metric, unit, higher_is_better, scaling, dtype = "m16_int4_verify_step_latency", "us", False, "strong", "bf16"
    CONTEXT = 4096
    MOE = False

    def __init__(self, rank, world, device, layers=None):
        import torch
        from dflash_mlx_b200.verify_step import HybridConfig, HybridVerifyModel, init_weights
        from dflash_mlx_b200.parallel import shard_config, make_collectives, PeerReducer
        self.torch, self.device, self.world, self.rank = torch, device, world, rank
        full = HybridConfig.moe_cfg5(max_context=self.CONTEXT + 64) if self.MOE else HybridConfig(max_context=self.CONTEXT + 64)
        if layers:
            full.layers = layers
        self.full_cfg = full
        cfg = shard_config(full, world)
        if self.MOE and world > 1:      # expert parallel: a contiguous range of experts per rank, shared expert on rank 0
            per = full.moe_experts // world
            cfg.moe_e_lo, cfg.moe_e_hi, cfg.moe_shared_here = rank * per, (rank + 1) * per, rank == 0
        self.cfg = cfg
        with torch.cuda.device(device):
            if world > 1:
                # ONE seeded model, the same on every rank, cut into this rank's shard (heads, MLP columns, vocabulary,
                # experts): the ranks together compute the single-GPU model
                from dflash_mlx_b200.parallel import shard_weights
                full_w = init_weights(full, 0xDF1D, device)
                cfg, weights = shard_weights(full, full_w, rank, world)
                self.cfg = cfg
                del full_w
                torch.cuda.empty_cache()
            else:
                weights = init_weights(cfg, 0xDF1D, device)
        self.weights = weights
        ar, ag = make_collectives(world)
        # row-parallel sums: the fused peer-memory kernel (default) or NCCL all-reduce + add/norm (DFLASH_TP_REDUCE=nccl)
        peer, self.reduce_mode = None, "none"
        if world > 1:
            self.reduce_mode = os.environ.get("DFLASH_TP_REDUCE", "peer")
            if self.reduce_mode == "peer":
                try:
                    peer = PeerReducer(rank, world, cfg.block, cfg.hidden, device)
                except Exception as exc:  # CUDA IPC refused in this container: say so and use the NCCL path
                    self.reduce_mode = "nccl (peer set-up failed: %s)" % str(exc)[:80]
                import torch.distributed as dist
                ok = torch.tensor([1 if peer is not None else 0], device=device)
                dist.all_reduce(ok, op=dist.ReduceOp.MIN)
                if int(ok) == 0 and peer is not None:
                    peer = None
                    self.reduce_mode = "nccl (peer set-up failed on another rank)"
        self.model = HybridVerifyModel(cfg, weights, device, all_reduce=ar, all_gather=ag, peer=peer)
        self.model.prefill_synthetic(self.CONTEXT, 0xDF1D)
        gen = torch.Generator().manual_seed(0xDF1D)
        self.ids_host = torch.randint(0, full.vocab, (cfg.block,), generator=gen, dtype=torch.int32).pin_memory()
        self.ids = self.ids_host.to(device)
        self.tok_host = torch.empty(cfg.block, dtype=torch.int32).pin_memory()
        self.model.verify(self.ids)
        self.launches_per_step = self.model.launches_per_step
        self.units_per_step = 1
        self.bytes = self.model.algorithmic_bytes()
        self.n_qmm = len(self.model.qmm_launch_list())
        self.config = {"workload": self.name, "layers": cfg.layers, "hidden": cfg.hidden, "context": self.CONTEXT,
                       "block": cfg.block, "vocab": full.vocab, "gdn_dims": "Hk16/Hv32/128x128 (from config 2)",
                       "experts": ("%d top-%d + shared, inter %d, experts %d..%d on this rank" % (
                           full.moe_experts, full.moe_top_k, full.moe_inter, *cfg.moe_local)) if self.MOE else "none",
                       "algorithmic_bytes_per_step_per_rank": self.bytes,
                       "l2": "inputs larger than L2: one step streams %.1f GB of weights" % (self.bytes["qmm"] / 1e9),
                       "parallelism": f"tp{world}", "row_parallel_reduce": self.reduce_mode}
        if self.MOE and world > 1:
            # "none": every rank holds all tokens, partial expert outputs are summed like any row-parallel output;
            # "a2a": dispatch + combine all-to-all collectives (DFLASH_MOE_EXCHANGE=a2a)
            self.config["expert_exchange"] = self.model.moe_exchange

    def step(self):
        self.model.verify(self.ids)

    def aux_step(self):
        self.model.run_qmm_only()

    def self_check(self):
        """Greedy tokens of the timed step against a second formulation of the same step on the same weights and caches:
        N > 1: row-parallel sums by NCCL all-reduce + separate add/norm kernels instead of the fused peer-memory kernel;
        N = 1: separate norm / residual / SwiGLU kernels instead of the matmul epilogues.  Both keep the residual stream
        in bf16 and round at different places, and the difference grows with depth like a random walk (measured on the
        random-init model: 2 % of the largest logit after 4 layers, 5 % after 16, 9 % after 64), so the bound is 3e-2 (the
        4-layer bound the tests hold against the oracle) x sqrt(layers / 4): the logits must agree within it, and the
        greedy tokens on every row whose top-2 margin exceeds it.  Every rank calls it."""
        import torch
        from dflash_mlx_b200.verify_step import HybridVerifyModel
        from dflash_mlx_b200.parallel import make_collectives
        world, dev = self.world, self.device
        if world > 1:
            ar, ag = make_collectives(world)
            other = HybridVerifyModel(self.cfg, self.weights, dev, all_reduce=ar, all_gather=ag, peer=None)
            what = "peer-memory reduce vs NCCL all-reduce"
        else:
            if not self.model.fused:
                return {"match": True, "compared": "the unfused step is the timed one"}
            other = HybridVerifyModel(self.cfg, self.weights, dev, fused=False)
            what = "fused matmul epilogues vs separate kernels"
        other.prefill_synthetic(self.CONTEXT, 0xDF1D)
        la = self.model.verify(self.ids).float()
        ta = self.model.tokens.clone()
        if self.MOE:
            # both passes route by the first one's router logits: with the random-init router the top-k weights are
            # nearly equal, so rounding noise that flips the k-th expert changes a row by ~1/k of its expert output
            other.routing_from = self.model.router_logits
            what += " (same routing)"
        lb = other.verify(self.ids).float()
        tb = other.tokens.clone()
        torch.cuda.synchronize()
        top2 = lb.topk(2, dim=-1).values                       # this rank's vocabulary shard
        amax = lb.abs().max().reshape(1)
        if world > 1:
            import torch.distributed as dist
            allt = [torch.empty_like(top2) for _ in range(world)]
            dist.all_gather(allt, top2.contiguous())
            top2 = torch.cat(allt, dim=1).topk(2, dim=-1).values
            dist.all_reduce(amax, op=dist.ReduceOp.MAX)
        # (mixture-of-experts layers: measured 0.07 - 0.10 over 2 / 4 / 8 ranks at 40 layers, a third above the dense walk)
        bound = (4e-2 if self.MOE else 3e-2) * max(1.0, (self.cfg.layers / 4.0) ** 0.5)
        dev_max = (la - lb).abs().max().reshape(1)
        if world > 1:
            dist.all_reduce(dev_max, op=dist.ReduceOp.MAX)
        rel = float(dev_max / amax)
        clear = (top2[:, 0] - top2[:, 1]) > bound * amax
        same = ta == tb
        del other
        return {"match": bool(torch.all(same | ~clear)) and rel <= bound, "equal_rows": int(same.sum()),
                "clear_rows": int(clear.sum()), "rows": int(same.numel()), "logits_rel_err": rel, "bound": bound,
                "compared": what}

    def e2e_step(self):
        self.model.verify_captured(self.ids_host)        # pinned host ids -> device inside the call
        self.tok_host.copy_(self.model.tokens, non_blocking=True)
        self.torch.cuda.current_stream().synchronize()
        return 1

    h2d_bytes = property(lambda self: self.cfg.block * 4)
    d2h_bytes = property(lambda self: self.cfg.block * 4)

    def value_from_ms(self, ms_per_step):
        return ms_per_step * 1e3

    def e2e_value(self, seconds, calls):
        return seconds * 1e6 / calls

    def roofline(self, ms_per_step, aux_ms, peak, peak_src):
        """Dominant kernel = the int4 matmul: its launches alone are replayed as a second CUDA graph."""
        us_per_launch = aux_ms * 1e3 / self.n_qmm
        per_launch = self.bytes["qmm"] / self.n_qmm
        achieved = per_launch / us_per_launch / 1e3
        return {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                # DRAM bytes per launch, scaled from the ncu captures of both kernels (read + write = 0.99 x the
                # algorithmic bytes for the mma.sync kernel on configuration 1, 1.03 x for the tcgen05 kernel on gate|up)
                "traffic": QMM_TC_TRAFFIC_RATIO * per_launch if (self.world == 1 and QMM_TC_TRAFFIC_RATIO) else None,
                "traffic_source": QMM_TC_TRAFFIC_SOURCE,
                "peak_source": peak_src,
                "kernel": "qmm_tc_kernel (tcgen05 int4 matmul: every matmul of the step, with its norm / residual / SwiGLU "
                          "epilogue when the step is fused)",
                "fused_epilogues": bool(getattr(self.model, "fused", False)),
                "launches_per_step": self.n_qmm, "algorithmic_bytes_per_launch": per_launch,
                "us_per_launch": us_per_launch, "matmul_share_of_step": aux_ms / ms_per_step,
                "whole_step_gbps": self.bytes["total"] / (ms_per_step * 1e-3) / 1e9}

    def cpu_sample(self):
        return dense_step_cpu_sample(self.full_cfg, self.CONTEXT)


class MoeStepWorkload(DenseStepWorkload):
    """Configuration 5 of BASELINE.json: one verify step of the 40-layer mixture-of-experts hybrid model (256 experts,
    top-8, one shared expert of intermediate 512, hidden 2048; attention 16 q / 2 KV heads of 256 and GatedDeltaNet
    16 / 32 heads of 128 from configurations 3 and 2) at context 8192.  N > 1: attention / GatedDeltaNet heads tensor
    parallel, experts expert-parallel (256 / N per rank, shared expert on rank 0); every rank holds all 16 tokens, so
    there is no dispatch - the ranks' partial block outputs are summed by the same fused peer-memory reduction."""
    name = "moe_step_cfg5"
    CONTEXT = 8192
    MOE = True

    def aux_step(self):
        self.model.run_experts_only()

    def roofline(self, ms_per_step, aux_ms, peak, peak_src):
        """Dominant kernels = the two expert-gathered matmuls of every layer (replayed alone, with the routing kernels,
        as a second CUDA graph); algorithmic bytes = matrices of the experts some token chose."""
        n = 2 * self.cfg.layers
        per_launch = self.bytes["experts"] / n
        us_per_launch = aux_ms * 1e3 / n
        achieved = per_launch / us_per_launch / 1e3
        return {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": None, "peak_source": peak_src,
                "kernel": "expert-gathered qmm_tc_kernel (tcgen05; rows gathered: gate|up; K chunks gathered: down), timed with "
                          "their routing and SwiGLU kernels",
                "launches_per_step": n, "algorithmic_bytes_per_launch": per_launch, "us_per_launch": us_per_launch,
                "matmul_share_of_step": aux_ms / ms_per_step,
                "whole_step_gbps": self.bytes["total"] / (ms_per_step * 1e-3) / 1e9}

    def cpu_sample(self):
        slots = int(round(self.bytes.get("active_expert_slots_per_layer", 0) * self.cfg.layers))
        return dense_step_cpu_sample(self.full_cfg, self.CONTEXT, expert_slots=slots)


class ReplayWorkload:
    """Configuration 2 of BASELINE.json, per speculative cycle: tape replay of ALL 48 GatedDeltaNet layers of the dense
    model (stacked along the batch axis) in one launch; 32 value / 16 key heads, 128x128 fp32 state, 16-step tape.
    A step walks a pool of independent state sets larger than L2.  Ranks shard the value heads."""
    name = "gdn_replay_cfg2"
    metric, unit, higher_is_better, scaling, dtype = "gdn_tape_replay_latency_per_cycle", "us", False, "strong", "f32"
    LAYERS, T, STEPS = 48, 16, 16

    def __init__(self, rank, world, device):
        import torch
        self.torch, self.device, self.world = torch, device, world
        Hk, Hv, D = 16 // world, 32 // world, 128
        self.shape = (Hk, Hv, D)
        L = self.LAYERS
        per = L * (2 * Hv * D * D * 4 + self.STEPS * (Hv * D * 4 + Hk * D * 2 + Hv * 4))
        self.per_launch_bytes = per
        self.pool = max(2, (3 * L2_BYTES) // per + 1)
        g = torch.Generator(device=device).manual_seed(0xDF1B + rank)
        rn = lambda *s: torch.randn(*s, generator=g, device=device)  # noqa: E731
        self.sets = []
        for _ in range(self.pool):
            k = rn(L, self.T, Hk, D)
            k = (k / k.norm(dim=-1, keepdim=True)).bfloat16()
            self.sets.append(dict(tape=rn(L, self.T, Hv, D), k=k,
                                  g=torch.exp(-torch.nn.functional.softplus(rn(L, self.T, Hv))),
                                  state=0.1 * rn(L, Hv, D, D), out=torch.empty(L, Hv, D, D, device=device)))
        self.steps_host = torch.tensor([self.STEPS], dtype=torch.int32).pin_memory()
        self.steps_dev = self.steps_host.to(device)
        self.flag_host = torch.empty(1, dtype=torch.float32).pin_memory()
        self.launches_per_step = self.pool
        self.units_per_step = self.pool
        self.config = {"workload": self.name, "layers": L, "tape_steps": self.T, "replayed_steps": self.STEPS,
                       "value_heads_per_rank": Hv, "state": "fp32 [48,Hv,128,128]", "pool": self.pool,
                       "l2": "inputs larger than L2: a step walks %d independent state sets (%.0f MB)" % (self.pool, self.pool * per / 1e6),
                       "parallelism": f"value heads x{world}"}

    def _one(self, s, steps):
        from dflash_mlx_b200.kernels import tape_replay_kernel
        return tape_replay_kernel(s["tape"], s["k"], s["g"], s["state"], steps=steps, out=s["out"])

    def step(self):
        for s in self.sets:
            self._one(s, self.steps_dev)

    def e2e_step(self):
        self._i = (getattr(self, "_i", -1) + 1) % self.pool
        self.steps_dev.copy_(self.steps_host, non_blocking=True)       # the accepted length arrives from the host
        out = self._one(self.sets[self._i], self.steps_dev)
        self.flag_host.copy_(out.view(-1)[:1], non_blocking=True)
        self.torch.cuda.current_stream().synchronize()
        return 1

    h2d_bytes = property(lambda self: 4)
    d2h_bytes = property(lambda self: 4)

    def value_from_ms(self, ms):
        return ms * 1e3 / self.units_per_step

    def e2e_value(self, seconds, calls):
        return seconds * 1e6 / calls

    def roofline(self, ms_per_step, aux_ms, peak, peak_src):
        us = ms_per_step * 1e3 / self.launches_per_step
        ach = self.per_launch_bytes / us / 1e3
        return {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak, "traffic": None,
                "peak_source": peak_src, "kernel": "tape_replay_pipe_kernel (persistent blocks, bulk-copy pipeline, packed fp32 pair arithmetic)", "algorithmic_bytes_per_launch": self.per_launch_bytes,
                "us_per_launch": us}

    def cpu_sample(self):
        import torch
        from oracle import gdn as og
        torch.set_num_threads(os.cpu_count() or 1)
        c = og.make_gdn_case(seed=1)
        tape = torch.randn(1, 16, 32, 128)

        def evaluate():
            t0 = time.perf_counter()
            og.tape_replay_ref(tape, c["k"], c["g"], c["state"], steps=self.STEPS)
            return (time.perf_counter() - t0) * self.LAYERS * 1e6, None, None

        return evaluate, {"unit": "us", "cores": torch.get_num_threads(), "kind": "port",
                          "sample": "one layer with the torch restatement of _tape_replay_ops x 48 layers; MLX unavailable "
                                    "on this box"}


class SdpaWorkload:
    """Configuration 3 of BASELINE.json: 16 query heads / 2 KV heads of 256, 16 query rows, KV length 8192 (bf16).
    A step walks a pool of KV caches larger than L2.  Ranks shard the KV heads (with their query heads)."""
    name = "verify_sdpa_cfg3"
    metric, unit, higher_is_better, scaling, dtype = "verify_sdpa_latency", "us", False, "strong", "bf16"
    N = 8192

    def __init__(self, rank, world, device, kv_len=0):
        import torch
        self.torch, self.device, self.world = torch, device, world
        if kv_len:
            self.N = int(kv_len)       # profiling aid (--kv-len): the metric's configuration is N = 8192
        Hk = max(1, 2 // world)
        Hq = 16 // world
        self.Hq, self.Hk, D = Hq, Hk, 256
        per = 2 * Hk * self.N * D * 2 + 2 * Hq * 16 * D * 2
        self.per_launch_bytes = per
        self.pool = max(2, (3 * L2_BYTES) // per + 1)
        g = torch.Generator(device=device).manual_seed(0xDF1C + rank)
        self.kv = [(torch.randn(1, Hk, self.N, D, generator=g, device=device).bfloat16(),
                    torch.randn(1, Hk, self.N, D, generator=g, device=device).bfloat16()) for _ in range(self.pool)]
        self.q_host = torch.randn(1, Hq, 16, D).bfloat16().pin_memory()
        self.q = self.q_host.to(device)
        self.o_host = torch.empty(1, Hq, 16, D, dtype=torch.bfloat16).pin_memory()
        self.launches_per_step = 2 * self.pool
        self.units_per_step = self.pool
        self.config = {"workload": self.name, "q_heads": Hq, "kv_heads": Hk, "head_dim": D, "kv_len": self.N, "pool": self.pool,
                       "l2": "inputs larger than L2: a step walks %d KV caches (%.0f MB)" % (self.pool, self.pool * per / 1e6),
                       "parallelism": f"kv heads x{world}"}

    def step(self):
        from dflash_mlx_b200.kernels import batched_sdpa_2pass_exact
        for k, v in self.kv:
            batched_sdpa_2pass_exact(self.q, k, v, 1.0 / 16.0)

    def e2e_step(self):
        from dflash_mlx_b200.kernels import batched_sdpa_2pass_exact
        self._i = (getattr(self, "_i", -1) + 1) % self.pool
        q = self.q_host.to(self.device, non_blocking=True)
        o = batched_sdpa_2pass_exact(q, *self.kv[self._i], 1.0 / 16.0)
        self.o_host.copy_(o, non_blocking=True)
        self.torch.cuda.current_stream().synchronize()
        return 1

    h2d_bytes = property(lambda self: self.Hq * 16 * 256 * 2)
    d2h_bytes = property(lambda self: self.Hq * 16 * 256 * 2)

    def value_from_ms(self, ms):
        return ms * 1e3 / self.units_per_step

    def e2e_value(self, seconds, calls):
        return seconds * 1e6 / calls

    def roofline(self, ms_per_step, aux_ms, peak, peak_src):
        us = ms_per_step * 1e3 / self.units_per_step
        ach = self.per_launch_bytes / us / 1e3
        return {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak, "traffic": None,
                "peak_source": peak_src, "kernel": "sdpa_tc_kernel (tcgen05: S / P / O in tensor memory, K / V by TMA) + combine_kernel",
                "algorithmic_bytes_per_launch": self.per_launch_bytes, "us_per_launch": us}

    def cpu_sample(self):
        import torch
        from oracle import sdpa as osd
        torch.set_num_threads(os.cpu_count() or 1)
        q, k, v, sc = osd.make_sdpa_case(self.N, seed=1)

        def evaluate():
            t0 = time.perf_counter()
            osd.sdpa_ref(q, k, v, sc)
            return (time.perf_counter() - t0) * 1e6, None, None

        return evaluate, {"unit": "us", "cores": torch.get_num_threads(), "kind": "port",
                          "sample": "dense-softmax torch restatement; MLX unavailable on this box"}


def load_oracle_lib():
    from oracle.build_ref import load
    out_dir = Path(os.environ.get("DFLASH_ORACLE_BUILD", str(ROOT / "oracle" / "_build" / "native")))
    try:
        return load(native=True, out_dir=out_dir), "gcc -O3 -march=native -fopenmp"
    except Exception:
        return load(native=False), "gcc -O3 -fopenmp"


def run_cpu_sample(sample, warmup, steps, budget_s):
    """`warmup` untimed evaluations, then up to `steps` timed ones (fewer if `budget_s` runs out; at least one): the
    median is the value.  Says how many ran."""
    evaluate, meta = sample
    for _ in range(max(1, warmup)):
        evaluate()
    vals, parts, t_end = [], None, time.perf_counter() + budget_s
    while len(vals) < steps and (not vals or time.perf_counter() < t_end):
        v, p, _ = evaluate()
        vals.append(v)
        parts = p if p is not None else parts
    order = sorted(vals)
    out = dict(meta)
    out["value"] = order[len(order) // 2]
    out["evaluations"] = len(vals)
    out["warmup_evaluations"] = max(1, warmup)
    out["spread"] = [order[0], order[-1]]
    out["sample"] = "median of %d timed evaluations after %d untimed; one evaluation = %s" % (len(vals), max(1, warmup), meta["sample"])
    if parts:
        out["parts_ms_last"] = parts
    return out


def dense_step_cpu_sample(cfg, context, expert_slots=0):
    """CPU path of one verify step on all host cores as a bounded sample: one evaluation runs every distinct linear
    shape once with the C restatement of the stock qmm (oracle/qmm_ref.c) and one GDN recurrence and one attention with
    the torch oracle; its value is sum(count x time) over the step.  Element-wise glue is left out (it favours the CPU
    number).  Operands are made once."""
    import torch
    from oracle import gdn as og
    from oracle import qmm as oq
    from oracle import sdpa as osd
    torch.set_num_threads(os.cpu_count() or 1)
    lib, note = load_oracle_lib()
    n_attn = sum(cfg.is_attention(i) for i in range(cfg.layers))
    n_gdn = cfg.layers - n_attn
    H, I, G, T = cfg.hidden, cfg.intermediate, cfg.group_size, cfg.block
    shapes = [("gdn_proj", cfg.gdn_proj_n, H, n_gdn, T), ("gdn_out", H, cfg.gdn_v_heads * cfg.gdn_dv, n_gdn, T),
              ("attn_proj", cfg.attn_proj_n, H, n_attn, T), ("attn_o", H, cfg.q_heads * cfg.head_dim, n_attn, T),
              ("lm_head", cfg.vocab, H, 1, T)]
    if cfg.moe_experts > 0:
        # routed experts see only the tokens that chose them (top_k * T / distinct experts, about 1.25 rows): timed with
        # 2 rows; expert_slots = active (expert, layer) pairs of the measured step, shared expert included
        slots = expert_slots if expert_slots else cfg.layers * min(T * cfg.moe_top_k, cfg.moe_experts)
        shapes += [("router", cfg.moe_experts + 1, H, cfg.layers, T), ("expert_gate_up", 2 * cfg.moe_inter, H, slots, 2),
                   ("expert_down", H, cfg.moe_inter, slots, 2)]
    else:
        shapes += [("gate_up", 2 * I, H, cfg.layers, T), ("down", H, I, cfg.layers, T)]
    ops = []
    for name, n, k, count, rows in shapes:
        if count == 0:
            continue
        wq, s, b = oq.random_quantized(n, k, seed=7, group_size=G)
        x = torch.randn(rows, k).bfloat16()
        y = torch.empty(rows, n, dtype=torch.float32)
        ops.append((name, count, (x.data_ptr(), wq.data_ptr(), s.data_ptr(), b.data_ptr(), y.data_ptr(), rows, k, n, G),
                    (wq, s, b, x, y)))
    c = og.make_gdn_case(seed=1, T=T, Hk=cfg.gdn_k_heads, Hv=cfg.gdn_v_heads, Dk=cfg.gdn_dk, Dv=cfg.gdn_dv)
    q, k_, v, sc = osd.make_sdpa_case(context + T, seed=2, Hq=cfg.q_heads, Hk=cfg.kv_heads, D=cfg.head_dim)

    def evaluate():
        total, parts = 0.0, {}
        for name, count, args, _keep in ops:
            t0 = time.perf_counter()
            lib.qmm_ref(*args)
            parts[name] = time.perf_counter() - t0
            total += count * parts[name]
        t0 = time.perf_counter()
        og.gated_delta_with_tape_ref(c["q"], c["k"], c["v"], c["g"], c["beta"], c["state"])
        parts["gdn_recurrence"] = time.perf_counter() - t0
        total += n_gdn * parts["gdn_recurrence"]
        t0 = time.perf_counter()
        osd.sdpa_ref(q, k_, v, sc)
        parts["attention"] = time.perf_counter() - t0
        total += n_attn * parts["attention"]
        return total * 1e6, {k2: round(v2 * 1e3, 3) for k2, v2 in parts.items()}, None

    return evaluate, {"unit": "us", "cores": int(lib.qmm_ref_threads()), "kind": "port",
                      "sample": "sum over the step of count x time of each distinct op (every linear shape once with the C "
                                f"qmm; one GDN recurrence and one attention with the torch oracle); {note}; MLX unavailable "
                                "on this box: CPU baseline = restatement of the stock path"}


WORKLOADS = {"qmm_cfg1": QmmWorkload, "dense_step_cfg4": DenseStepWorkload, "moe_step_cfg5": MoeStepWorkload,
             "gdn_replay_cfg2": ReplayWorkload,
             "verify_sdpa_cfg3": SdpaWorkload}
DEFAULT_WORKLOAD = "dense_step_cfg4"
EXTRA_WORKLOADS = ("qmm_cfg1", "gdn_replay_cfg2")      # reported under "extra" by the default one-GPU run
wl_extra_holder = []


def run_reference_arm(args, rank, world):
    """The reference's CPU implementation of the path on this box's host cores (rank 0 only; MLX is not installable
    here, so it is the oracle port).  --warmup untimed evaluations of the bounded sample, then --steps timed ones (fewer
    if 150 s run out): `steps` in the line is the number that ran, the value their median."""
    if rank != 0:
        return
    cls = WORKLOADS[args.workload]
    if cls is QmmWorkload:
        import torch
        w = cls.__new__(cls)
        w.torch = torch
        w.x_host = torch.randn(cls.M, cls.K, generator=torch.Generator().manual_seed(0xDF1A)).bfloat16()
        w.world, w.n_local = 1, cls.N
        sample = w.cpu_sample()
        config = {"workload": cls.name, "M": cls.M, "K": cls.K, "N": cls.N, "group_size": cls.G}
    elif cls in (ReplayWorkload, SdpaWorkload):
        sample = cls.__new__(cls).cpu_sample()
        config = {"workload": cls.name}
    else:
        from dflash_mlx_b200.verify_step import HybridConfig
        moe = getattr(cls, "MOE", False)
        cfg = HybridConfig.moe_cfg5(max_context=cls.CONTEXT + 64) if moe else HybridConfig(max_context=cls.CONTEXT + 64)
        # MoE: the expected number of distinct routed experts for 16 tokens x top-k uniform routing, + the shared one
        slots = 0
        if moe:
            E, picks = cfg.moe_experts, cfg.block * cfg.moe_top_k
            slots = int(round(cfg.layers * (E * (1.0 - (1.0 - 1.0 / E) ** picks) + 1)))
        sample = dense_step_cpu_sample(cfg, cls.CONTEXT, expert_slots=slots)
        config = {"workload": cls.name, "layers": cfg.layers, "hidden": cfg.hidden, "context": cls.CONTEXT,
                  "block": cfg.block, "vocab": cfg.vocab}
        if moe:
            config["experts"] = "%d top-%d + shared, inter %d; %d active (expert, layer) pairs assumed" % (
                cfg.moe_experts, cfg.moe_top_k, cfg.moe_inter, slots)
    cb = run_cpu_sample(sample, args.warmup, args.steps, budget_s=150.0)
    line = {"impl": "reference", "metric": cls.metric, "value": cb["value"], "unit": cls.unit, "n_gpus": args.gpus,
            "steps": cb["evaluations"], "steps_requested": args.steps, "warmup": cb["warmup_evaluations"],
            "ms_per_step": cb["value"] / 1e3,
            "higher_is_better": cls.higher_is_better, "scaling": cls.scaling, "vs_baseline": None, "dtype": cls.dtype,
            "data": "synthetic", "config": config, "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": cls.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the single-op lines that ride along on one GPU")
    ap.add_argument("--profiler-range", action="store_true",
                    help="bracket the timed steps with cudaProfilerStart/Stop (for `ncu --profile-from-start off`)")
    ap.add_argument("--layers", type=int, default=0, help="profiling aid: run the dense / MoE step with fewer layers")
    ap.add_argument("--kv-len", type=int, default=0, help="profiling aid: KV length of verify_sdpa_cfg3 (default 8192)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path); use --impl reference for the CPU arm")
    os.environ["DFLASH_VERIFY_QMM"] = "1"
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if args.layers and args.workload in ("dense_step_cfg4", "moe_step_cfg5"):
        wl = WORKLOADS[args.workload](rank, world, device, layers=args.layers)
    elif args.kv_len and args.workload == "verify_sdpa_cfg3":
        wl = WORKLOADS[args.workload](rank, world, device, kv_len=args.kv_len)
    else:
        wl = WORKLOADS[args.workload](rank, world, device)

    # ---- device-resident loop: one CUDA graph = one step ----
    def time_graph(fn, steps, warmup, sample=False):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()                      # untimed: creates workspaces, tensor maps, kernel attributes
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                fn()
        torch.cuda.current_stream().wait_stream(side)
        for _ in range(warmup):
            graph.replay()
        barrier()
        if sample and rank == 0:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        if sample and args.profiler_range:
            torch.cuda.profiler.start()
        e0.record()
        for _ in range(steps):
            graph.replay()
        e1.record()
        barrier()
        if sample and args.profiler_range:
            torch.cuda.profiler.stop()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / steps

    sampler = ClockSampler(local_rank)
    ms_per_step = time_graph(wl.step, args.steps, args.warmup, sample=True)
    aux_ms = time_graph(wl.aux_step, args.steps, args.warmup) if hasattr(wl, "aux_step") else None

    # ---- end to end through the public API with host buffers ----
    for _ in range(3):
        wl.e2e_step()
    barrier()
    calls, t0 = 0, time.perf_counter()
    e2e_iters = max(50, args.steps * 4)
    for _ in range(e2e_iters):
        calls += wl.e2e_step()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    clocks = sampler.stop() if rank == 0 else None

    check = wl.self_check() if hasattr(wl, "self_check") else None

    # ---- on one GPU: the single-op lines of the other configurations ride along (short runs) ----
    extra = {}
    if world == 1 and not args.no_extra and args.workload == DEFAULT_WORKLOAD:
        peak, peak_src = measured_peaks()
        for name in EXTRA_WORKLOADS:
            del wl_extra_holder[:]
            torch.cuda.empty_cache()
            w2 = WORKLOADS[name](rank, world, device)
            wl_extra_holder.append(w2)
            k2 = max(5, args.steps // 2)
            ms2 = time_graph(w2.step, k2, 3)
            extra[name] = {"metric": w2.metric, "value": w2.value_from_ms(ms2), "unit": w2.unit, "steps": k2, "warmup": 3,
                           "dtype": w2.dtype, "config": w2.config, "roofline": w2.roofline(ms2, None, peak, peak_src),
                           "gpu_launches": w2.launches_per_step * k2}
        del wl_extra_holder[:]

    from dflash_mlx_b200 import _lib
    dev_err = _lib.lib().dflash_device_error(local_rank)

    if rank == 0:
        peak, peak_src = measured_peaks()
        line = {"metric": wl.metric, "value": wl.value_from_ms(ms_per_step), "unit": wl.unit, "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
                "higher_is_better": wl.higher_is_better, "scaling": wl.scaling, "vs_baseline": None,
                "dtype": wl.dtype, "data": "synthetic", "config": wl.config,
                "roofline": wl.roofline(ms_per_step, aux_ms, peak, peak_src),
                "e2e": {"value": wl.e2e_value(e2e_s, calls), "unit": wl.unit, "h2d_bytes_per_step": wl.h2d_bytes,
                        "d2h_bytes_per_step": wl.d2h_bytes, "calls": calls},
                "gpu_launches": wl.launches_per_step * args.steps,
                "clocks": clocks, "device_error": dev_err}
        if check is not None:
            line["tp_tokens_match" if world > 1 else "fused_tokens_match"] = check["match"]
            line["self_check"] = check
        if extra:
            line["extra"] = extra
        if not args.no_cpu_baseline and world == 1:
            line["cpu_baseline"] = run_cpu_sample(wl.cpu_sample(), 1, 5, budget_s=20.0)
        print(json.dumps(line), flush=True)
    if world > 1:
        # CUDA graphs that captured NCCL kernels are still alive here; tearing the process group down under them can
        # block.  All ranks have finished their work: synchronise, then leave without the teardown.
        sys.stdout.flush()
        barrier()
        os._exit(0)


if __name__ == "__main__":
    main()
