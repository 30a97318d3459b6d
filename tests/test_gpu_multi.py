"""The sharded drivers over NCCL on two GPUs of one box (skipped where fewer are visible):
column shards with A broadcast in row panels, and batch shards with no collective."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import datetime

    from wmma_extension_b200 import sharded, tcec

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=120))
    try:
        m, n, k = 1500, 1100, 640
        g = torch.Generator(device="cpu").manual_seed(31)
        a = torch.randn((m, k), generator=g)
        b = torch.randn((k, n), generator=g)
        c0, cn = sharded.column_shard(n, rank, world)
        b_local = b[:, c0:c0 + cn].contiguous().to(dev)
        c_local = torch.full((m, cn), float("nan"), device=dev)
        a_root = a.to(dev) if rank == 0 else None
        tcec.set_option("comm_panel_rows", 256)  # six panels at this size: flags and the helper launch are exercised
        sharded.sgemm_column_sharded(a_root, b_local, c_local, m, k, root=0)
        tcec.device_status()
        want = tcec.sgemm(a.to(dev), b_local)  # the same block computed without communication
        assert torch.equal(c_local, want)
        # the same from host memory through the pipelined entry
        bh, ch = b_local.cpu().pin_memory(), torch.full((m, cn), float("nan")).pin_memory()
        tcec.sgemm_column_shard_host(a.pin_memory() if rank == 0 else None, bh, ch, m, k, root=0, panel_rows=256)
        torch.cuda.current_stream().synchronize()
        tcec.device_status()
        assert torch.equal(ch, want.cpu())
        np.save(os.path.join(out_dir, f"c{rank}.npy"), c_local.cpu().numpy())
        np.save(os.path.join(out_dir, f"cols{rank}.npy"), np.array([c0, cn]))
        # batch shards
        nb = 37
        ab = torch.randn((nb, 96, 64), generator=g)
        bb = torch.randn((nb, 64, 300), generator=g)
        first, count = sharded.batch_shard(nb, rank, world)
        got = sharded.sgemm_batch_sharded(ab[first:first + count].to(dev), bb[first:first + count].to(dev))
        tcec.device_status()
        np.save(os.path.join(out_dir, f"b{rank}.npy"), got.cpu().numpy())
        np.save(os.path.join(out_dir, f"brange{rank}.npy"), np.array([first, count]))
    finally:
        tcec.comm_destroy()
        dist.destroy_process_group()


def test_one_process_drives_two_gpus_through_the_c_abi():
    """tcec_sgemm_multi and tcec_sgemm_batched_multi (device list, library-owned NCCL
    communicators): bit-equal to the single-GPU calls on the same blocks."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from wmma_extension_b200 import sharded, tcec

    m, n, k = 1500, 1100, 640
    g = torch.Generator(device="cpu").manual_seed(32)
    a = torch.randn((m, k), generator=g)
    b = torch.randn((k, n), generator=g)
    devs = [torch.device("cuda", 0), torch.device("cuda", 1)]
    cols = [sharded.column_shard(n, r, 2) for r in range(2)]
    b_blocks = [b[:, c0:c0 + cn].contiguous().to(d) for (c0, cn), d in zip(cols, devs)]
    try:
        for panel_rows in (256, 2048):
            tcec.set_option("comm_panel_rows", panel_rows)
            c_blocks = [torch.full((m, cn), float("nan"), device=d) for (_, cn), d in zip(cols, devs)]
            tcec.sgemm_multi(a.to(devs[0]), b_blocks, c_blocks)
            for d in devs:
                torch.cuda.synchronize(d)
                with torch.cuda.device(d):
                    tcec.device_status()
            for d, bb, cc in zip(devs, b_blocks, c_blocks):
                assert torch.equal(cc, tcec.sgemm(a.to(d), bb)), panel_rows
    finally:
        tcec.set_option("comm_panel_rows", 2048)
    # batch shards: no collective
    nb = 37
    ab = torch.randn((nb, 96, 64), generator=g)
    bb = torch.randn((nb, 64, 300), generator=g)
    parts = [sharded.batch_shard(nb, r, 2) for r in range(2)]
    a_parts = [ab[f:f + c].to(d) for (f, c), d in zip(parts, devs)]
    b_parts = [bb[f:f + c].to(d) for (f, c), d in zip(parts, devs)]
    c_parts = [torch.empty((c, 96, 300), device=d) for (_, c), d in zip(parts, devs)]
    tcec.sgemm_batched_multi(a_parts, b_parts, c_parts)
    for d, x, y, z in zip(devs, a_parts, b_parts, c_parts):
        torch.cuda.synchronize(d)
        assert torch.equal(z, tcec.sgemm_strided_batched(x, y))
    tcec.destroy()


def test_sharded_drivers_over_nccl_on_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    g = torch.Generator(device="cpu").manual_seed(31)
    a = torch.randn((1500, 640), generator=g)
    b = torch.randn((640, 1100), generator=g)
    exact = a.double() @ b.double()
    got = torch.full((1500, 1100), float("nan"))
    for r in range(world):
        c0, cn = np.load(tmp_path / f"cols{r}.npy")
        got[:, c0:c0 + cn] = torch.from_numpy(np.load(tmp_path / f"c{r}.npy"))
    assert ((got.double() - exact).abs().max() / exact.abs().max()).item() < 1e-6
    ab = torch.randn((37, 96, 64), generator=g)
    bb = torch.randn((37, 64, 300), generator=g)
    exact_b = torch.matmul(ab.double(), bb.double())
    parts = {}
    for r in range(world):
        first, count = np.load(tmp_path / f"brange{r}.npy")
        parts[int(first)] = torch.from_numpy(np.load(tmp_path / f"b{r}.npy"))
        assert parts[int(first)].shape[0] == count
    got_b = torch.cat([parts[key] for key in sorted(parts)])
    assert got_b.shape == exact_b.shape
    assert ((got_b.double() - exact_b).abs().max() / exact_b.abs().max()).item() < 1e-6
