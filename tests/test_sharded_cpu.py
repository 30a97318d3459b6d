"""The multi-GPU host logic on CPU: shard arithmetic, the column-sharded driver run as two
``gloo`` ranks with the oracle standing in for the local GEMM, and what the driver does when a
rank's compute fails or a rank leaves (failures are made on the host; no GPU is involved)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from wmma_extension_b200 import sharded


def test_batch_shard_covers_everything_once():
    for batch in (0, 1, 7, 8, 8192, 8191):
        for world in (1, 2, 3, 8):
            seen = []
            for r in range(world):
                first, cnt = sharded.batch_shard(batch, r, world)
                seen += list(range(first, first + cnt))
            assert seen == list(range(batch))
    with pytest.raises(ValueError):
        sharded.batch_shard(4, 2, 2)


def test_column_shard_is_tile_aligned_and_complete():
    for n in (0, 1, 255, 256, 1000, 65536, 65537):
        for world in (1, 2, 4, 8):
            cols = []
            for r in range(world):
                first, cnt = sharded.column_shard(n, r, world)
                if cnt:
                    assert first % 256 == 0
                cols += list(range(first, first + cnt))
            assert cols == list(range(n))
    assert sharded.column_shard(65536, 3, 8) == (3 * 8192, 8192)


def test_row_panels():
    assert sharded.row_panels(300, 100) == [(0, 128), (128, 128), (256, 44)]
    assert sharded.row_panels(0, 128) == []
    assert sum(r for _, r in sharded.row_panels(65536, 2048)) == 65536


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, m, n, k, panel_rows, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import cpu

        rng = np.random.default_rng(21)
        a = rng.standard_normal((m, k)).astype(np.float32)
        b = rng.standard_normal((k, n)).astype(np.float32)
        c0, cn = sharded.column_shard(n, rank, world, align=64)
        b_local = torch.from_numpy(np.ascontiguousarray(b[:, c0:c0 + cn]))
        c_local = torch.full((m, cn), float("nan"))
        calls = []

        def prepare_b(bl):
            calls.append("prepare")
            return bl.numpy().copy()

        def gemm_panel(a_panel, prepared, c_rows):
            calls.append(a_panel.shape[0])
            c_rows.copy_(torch.from_numpy(cpu.tcec_gemm(a_panel.numpy(), prepared)))

        ops = sharded.LocalOps(prepare_b, gemm_panel)
        a_root = torch.from_numpy(a) if rank == 0 else None
        sharded.sgemm_column_sharded(a_root, b_local, c_local, m, k, root=0, panel_rows=panel_rows, ops=ops)
        assert calls[0] == "prepare" and calls.count("prepare") == 1  # B is prepared once, not per panel
        assert sum(calls[1:]) == m
        np.save(os.path.join(out_dir, f"c{rank}.npy"), c_local.numpy())
        np.save(os.path.join(out_dir, f"cols{rank}.npy"), np.array([c0, cn]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("m,n,k,panel_rows", [(300, 200, 96, 128), (128, 130, 64, 4096)])
def test_column_sharded_two_ranks_gloo(tmp_path, m, n, k, panel_rows):
    from oracle import cpu

    world = 2
    mp.spawn(_worker, args=(world, _free_port(), m, n, k, panel_rows, str(tmp_path)), nprocs=world, join=True)
    rng = np.random.default_rng(21)
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal((k, n)).astype(np.float32)
    want = cpu.tcec_gemm(a, b)
    got = np.full((m, n), np.nan, dtype=np.float32)
    for r in range(world):
        c0, cn = np.load(tmp_path / f"cols{r}.npy")
        got[:, c0:c0 + cn] = np.load(tmp_path / f"c{r}.npy")
    # each output element depends only on its own row of A and column of B: bit-identical to one rank
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert cpu.errors(got, cpu.gemm_f64(a, b))["max_rel"] < 1e-6


def _failing_worker(rank, world, port, mode, out_dir):
    """mode 'local': rank 1's gemm_panel raises on its second panel.  mode 'leave': rank 1 takes part
    in one call and then leaves, between calls, with nothing of its own in flight."""
    import datetime

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    m, n, k = 384, 256, 64
    rng = np.random.default_rng(5)
    a = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32))
    b = torch.from_numpy(rng.standard_normal((k, n)).astype(np.float32))
    c0, cn = sharded.column_shard(n, rank, world, align=64)
    b_local = b[:, c0:c0 + cn].contiguous()
    calls = {"n": 0}

    def gemm_panel(a_panel, prepared, c_rows):
        calls["n"] += 1
        if mode == "local" and rank == 1 and calls["n"] == 2:
            raise RuntimeError("injected failure of the local GEMM")
        c_rows.copy_(a_panel @ prepared)

    ops = sharded.LocalOps(lambda bl: bl.clone(), gemm_panel)
    result = "ok"
    try:
        for step in range(2):
            if mode == "leave" and rank == 1 and step == 1:
                break  # leaves between calls
            c_local = torch.zeros((m, cn))
            sharded.sgemm_column_sharded(a if rank == 0 else None, b_local, c_local, m, k, root=0, panel_rows=128,
                                         ops=ops)
            if mode == "leave":
                assert torch.allclose(c_local, a @ b_local, atol=1e-4)
    except sharded.ShardError as e:
        result = f"shard_error {e.status}"
    with open(os.path.join(out_dir, f"r{rank}.txt"), "w") as f:
        f.write(result)
    if mode == "local":
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["local", "leave"])
def test_failures_surface_as_a_status_on_every_rank(tmp_path, mode):
    world = 2
    ctx = mp.spawn(_failing_worker, args=(world, _free_port(), mode, str(tmp_path)), nprocs=world, join=False)
    import time

    deadline = time.time() + 120
    while not ctx.join(timeout=5):
        assert time.time() < deadline, "a rank is blocked"
    got = [open(tmp_path / f"r{r}.txt").read() for r in range(world)]
    if mode == "local":
        # the failing rank reports its own error, the other one learns of it; nobody blocks
        assert got[1] == f"shard_error {sharded.ERR_LOCAL}"
        assert got[0] == f"shard_error {sharded.ERR_PEER}"
    else:
        # the rank that stays gets a communication error from its next collective instead of waiting forever
        assert got[1] == "ok"
        assert got[0] == f"shard_error {sharded.ERR_COMM}"
