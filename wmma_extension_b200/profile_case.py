"""Small, self-ending case of the hot path for profiler captures.

    python -m wmma_extension_b200.profile_case --size 6144 --policy fp16_ec --reps 3

Runs `reps` full calls (split of A, split of B, GEMM) of one square SGEMM on cuda:0
with a few hundred MB on the device, prints the event-timed throughput, and exits.
"""
import argparse

import torch

from . import tcec


def _time(fn, reps):
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def late_ctas(size: int, reps: int) -> None:
    """What a kernel that holds 8 SMs when the GEMM starts costs it, with tiles drawn from the
    device-wide counter (default) and with static striding (option static_tiles = 1)."""
    dev = torch.device("cuda:0")
    m, n, k = 2048, size, size
    a = torch.rand((m, k), device=dev) * 2 - 1
    b = torch.rand((k, n), device=dev) * 2 - 1
    c = torch.empty((m, n), device=dev)
    ap_, bp_ = tcec.pack_a(a), tcec.pack_b(b)
    dm, dn, dk = 128, 2048, 24576  # 8 tiles: 8 CTAs, each owning an SM for a few hundred microseconds
    da, db = torch.rand((dm, dk), device=dev), torch.rand((dk, dn), device=dev)
    dc = torch.empty((dm, dn), device=dev)
    dap, dbp = tcec.pack_a(da), tcec.pack_b(db)
    side = torch.cuda.Stream()
    print(f"8-CTA GEMM alone: {_time(lambda: tcec.sgemm_packed(dap, dbp, dm, dn, dk, dc), reps):.3f} ms")

    def both():
        ev = torch.cuda.Event()
        ev.record()
        with torch.cuda.stream(side):
            side.wait_event(ev)
            tcec.sgemm_packed(dap, dbp, dm, dn, dk, dc)
        tcec.sgemm_packed(ap_, bp_, m, n, k, c)
        torch.cuda.current_stream().wait_stream(side)

    try:
        for _ in range(3):
            for static in (0, 1):
                tcec.set_option("static_tiles", static)
                alone = _time(lambda: tcec.sgemm_packed(ap_, bp_, m, n, k, c), reps)
                print(f"{'static striding' if static else 'tile counter   '}: {m}x{n}x{k} alone {alone:.3f} ms, "
                      f"with the 8-CTA GEMM started just before it {_time(both, reps):.3f} ms", flush=True)
    finally:
        tcec.set_option("static_tiles", 0)
    tcec.device_status()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--size", type=int, default=6144)
    ap.add_argument("--policy", default="fp16_ec")
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--batch", type=int, default=0, help="if > 0: strided batch of size x size x size")
    ap.add_argument("--late-ctas", action="store_true",
                    help="time a 2048 x size x size GEMM alone and with an 8-CTA GEMM started just before it "
                         "on another stream, for both tile orders")
    args = ap.parse_args()
    if args.late_ctas:
        late_ctas(args.size, args.reps)
        return
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
