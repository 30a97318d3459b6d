"""Small, self-ending case of the hot path for profiler captures.

    python -m wmma_extension_b200.profile_case --size 6144 --policy fp16_ec --reps 3

Runs `reps` full calls (split of A, split of B, GEMM) of one square SGEMM on cuda:0
with a few hundred MB on the device, prints the event-timed throughput, and exits.
"""
import argparse

import torch

from . import tcec


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--size", type=int, default=6144)
    ap.add_argument("--policy", default="fp16_ec")
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--batch", type=int, default=0, help="if > 0: strided batch of size x size x size")
    args = ap.parse_args()
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev)
    g.manual_seed(2)
    n = args.size
    shape = (args.batch, n, n) if args.batch else (n, n)
    a = torch.rand(shape, generator=g, device=dev) * 2 - 1
    b = torch.rand(shape, generator=g, device=dev) * 2 - 1
    c = torch.empty(shape, device=dev)
    call = tcec.sgemm_strided_batched if args.batch else tcec.sgemm
    call(a, b, c, policy=args.policy)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.reps):
        call(a, b, c, policy=args.policy)
    e1.record()
    torch.cuda.synchronize()
    tcec.device_status()
    ms = e0.elapsed_time(e1) / args.reps
    flop = 2.0 * n * n * n * max(1, args.batch)
    print(f"size {n} batch {args.batch} policy {args.policy}: {ms:.3f} ms/call, {flop / ms * 1e-9:.1f} TFLOP/s")


if __name__ == "__main__":
    main()
