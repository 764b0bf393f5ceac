"""Prints the phase time stamps that one CTA of the attention kernels records (tuning aid).

    python -m torchmpi_b200.utils.attention_trace [--batch 8] [--seq 1024] [--heads 16] [--backward]

Forward: the CTA of the last query block (it walks every key block); backward: the CTA of the first key block (it meets
every query block).  Times are nanoseconds from the CTA's first stamp, read from the GPU's global timer (32 ns steps);
a stamp costs a timer read and a store, so traced launches are a little slower than untraced ones.
"""
from __future__ import annotations

import argparse

import torch

FWD = {0: "waits for S", 1: "has S", 2: "row maximum known", 3: "P written", 4: "P announced", 10: "mma: has P",
       11: "mma: has V", 12: "mma: P V issued", 5: "has O_j", 6: "output updated", 8: "mma: S was read",
       9: "mma: next S issued"}
BWD = {0: "waits for S, dP", 1: "has S, dP", 2: "P, dS announced", 10: "mma: has P, dS", 12: "mma: three products issued",
       3: "waits for dQ", 4: "has dQ", 5: "reductions issued", 8: "mma: S, dP were read", 9: "mma: next S, dP issued"}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--backward", action="store_true")
    args = ap.parse_args()
    from torchmpi_b200.ops import attention
    from torchmpi_b200._lib import lib
    B, T, H = args.batch, args.seq, args.heads
    qkv = torch.randn(B, T, 3 * H * 64, device="cuda").to(torch.bfloat16)
    out, lse = attention.attention_forward(qkv, H)
    dout = torch.randn_like(out)
    blocks = T // 128
    buf = torch.zeros(blocks * 16, dtype=torch.int64, device="cuda")
    run = (lambda: attention.attention_backward(qkv, out, lse, dout, H)) if args.backward else \
        (lambda: attention.attention_forward(qkv, H))
    setter = lib.tmpi_attention_bwd_set_trace if args.backward else lib.tmpi_attention_set_trace
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    setter(buf.data_ptr())
    try:
        run()
        torch.cuda.synchronize()
    finally:
        setter(None)
    attention.check_status()
    t = buf.cpu().view(blocks, 16)
    t0 = min(int(v) for v in t.flatten().tolist() if v)
    names = BWD if args.backward else FWD
    for j in range(blocks):
        cells = [f"{name} {int(t[j, e]) - t0}" for e, name in names.items() if int(t[j, e])]
        print(f"{'pair' if args.backward else 'key block'} {j}: " + "; ".join(cells))


if __name__ == "__main__":
    main()
