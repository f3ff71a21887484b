"""Where the time of one verify matmul launch goes: per-block time stamps of the tcgen05 kernel.

    python -m dflash_mlx_b200.qmm_stamps [K N] ...        (default: 4096 12288  5120 151936  2048 256)

Launches `dflash_verify_qmm` once per shape on weights that were never touched before (cold in L2 and HBM row buffers),
with the stamp buffer of `dflash_verify_qmm_set_stamps` attached, and prints for every shape the average / maximum over
the blocks of: set-up done, first activation tile landed, first pipeline stage complete, first MMA issued, last MMA
issued, last accumulators read, last output written, exit (microseconds from the block's entry), and the kernel's
span from the first entry to the last exit.  A measurement aid, not part of the verify path.
"""
from __future__ import annotations

import ctypes
import sys

import torch

from . import _lib

NAMES = ["set-up", "x tile 0", "stage 0", "first MMA", "last MMA", "acc read", "last out", "exit"]


def stamps_for(K: int, N: int, M: int = 16, G: int = 64):
    lib = _lib.lib()
    c = ctypes
    lib.dflash_verify_qmm_set_stamps.restype = None
    lib.dflash_verify_qmm_set_stamps.argtypes = [c.c_void_p]
    dev = torch.device("cuda")
    gen = torch.Generator(device=dev).manual_seed(K * 31 + N)
    wq = torch.randint(-2 ** 31, 2 ** 31 - 1, (N, K // 8), generator=gen, device=dev, dtype=torch.int64).to(torch.int32)
    s = (0.008 * (1.0 + 0.1 * torch.randn(N, K // G, generator=gen, device=dev))).bfloat16()
    b = (-7.5 * s.float()).bfloat16()
    x = (torch.randn(M, K, generator=gen, device=dev) * (8.0 / K ** 0.5)).bfloat16()
    y = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    ws = torch.zeros(lib.dflash_verify_qmm_workspace_bytes(M, K, N, G) + 256, dtype=torch.uint8, device=dev)
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    stamps = torch.zeros(148 * 16, dtype=torch.int64, device=dev)
    st = torch.cuda.current_stream().cuda_stream

    def run():
        rc = lib.dflash_verify_qmm(x.data_ptr(), wq.data_ptr(), s.data_ptr(), b.data_ptr(), None, y.data_ptr(), M, K, N, G,
                                   _lib.BF16, ws.data_ptr(), ws.numel(), st)
        _lib.check(rc, "dflash_verify_qmm")

    run()                                   # creates tensor maps and kernel attributes
    flush.fill_(1)                          # evicts the weights from L2
    torch.cuda.synchronize()
    lib.dflash_set_pdl(0)                   # a plain launch with nothing before it: the kernel alone
    lib.dflash_verify_qmm_set_stamps(stamps.data_ptr())
    run()
    torch.cuda.synchronize()
    lib.dflash_verify_qmm_set_stamps(None)
    lib.dflash_set_pdl(1)
    h = stamps.cpu().view(148, 16)
    live = h[h[:, 0] != 0]
    if live.numel() == 0:
        raise RuntimeError("no stamps: this shape did not run the tcgen05 kernel")
    t0, t1 = int(live[:, 0].min()), int(live[:, 1].max())
    ns_per_clk = (live[:, 1] - live[:, 0]).double() / (live[:, 10] - live[:, 2]).double()
    rel = (live[:, 3:11] - live[:, 2:3]).double() * ns_per_clk[:, None] / 1e3      # us from entry
    return {"blocks": int(live.shape[0]), "avg": rel.mean(dim=0).tolist(), "max": rel.max(dim=0).values.tolist(),
            "kernel_us": (t1 - t0) / 1e3}


def main(argv):
    shapes = [(4096, 12288), (5120, 151936), (2048, 256)]
    if len(argv) >= 2:
        shapes = [(int(argv[i]), int(argv[i + 1])) for i in range(0, len(argv) - 1, 2)]
    print("| shape | blocks | " + " | ".join(NAMES) + " | kernel |")
    print("|---|---|" + "---|" * (len(NAMES) + 1))
    for K, N in shapes:
        r = stamps_for(K, N)
        cells = " | ".join("%.2f / %.2f" % (a, m) for a, m in zip(r["avg"], r["max"]))
        print(f"| {K} -> {N} | {r['blocks']} | {cells} | {r['kernel_us']:.1f} |")


if __name__ == "__main__":
    main(sys.argv[1:])
