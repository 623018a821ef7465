"""Row-range sharding used for N > 1 GPUs: host logic on CPU, including a 2-rank gloo run in which every rank
computes only its shard (with the CPU oracle standing in for the GPU engine) and the gathered result must be
bit-identical to the unsharded one -- the path bench.py takes under torchrun, minus the device."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

from dphpc_b200 import Dataset
from dphpc_b200.partition import block_grid, block_shard, coo_cuts, row_cuts, shard

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("cfg,scale", [(2, 0.05), (4, 0.01), (5, 0.01)])
@pytest.mark.parametrize("parts", [1, 2, 4, 8])
def test_cuts_cover_and_balance(cfg, scale, parts):
    d = Dataset(cfg, 4, scale)
    cuts = row_cuts(d.row_ptr, parts)
    assert cuts[0] == 0 and cuts[-1] == d.M and len(cuts) == parts + 1
    assert (np.diff(cuts) >= 0).all()
    per = np.diff(d.row_ptr[cuts])
    assert per.sum() == d.nnz
    longest = int(np.diff(d.row_ptr).max())
    assert per.max() <= d.nnz / parts + longest  # no shard exceeds its share by more than one row


def test_aligned_cuts_stay_on_the_tile_grid():
    d = Dataset(2, 4, 0.3)
    cuts = row_cuts(d.row_ptr, 4, align=64)
    assert cuts[0] == 0 and cuts[-1] == d.M and (np.diff(cuts) >= 0).all()
    assert all(int(c) % 64 == 0 for c in cuts[1:-1])
    per = np.diff(d.row_ptr[cuts])
    assert per.max() <= d.nnz / 4 + 64 * int(np.diff(d.row_ptr).max())


def test_cuts_on_degenerate_patterns():
    assert row_cuts(np.array([0, 0, 0, 5], np.int32), 2).tolist() == [0, 2, 3]      # all nonzeros in the last row
    assert row_cuts(np.array([0, 4, 4, 4], np.int32), 4).tolist() == [0, 0, 1, 1, 3]     # one heavy row: it goes to one shard, the others stay (nearly) empty
    cuts = row_cuts(np.arange(9, dtype=np.int32), 8)                                     # diagonal: one row each
    assert cuts.tolist() == list(range(9))
    assert row_cuts(np.zeros(5, np.int32), 2)[[0, -1]].tolist() == [0, 4]                # empty matrix


@pytest.mark.parametrize("parts", [1, 2, 3, 8])
def test_coo_cuts_find_row_boundaries_without_a_row_ptr(parts):
    d = Dataset(5, 4, 0.01)
    rows = d.row_idx()
    cuts, offs = coo_cuts(rows, d.M, parts)
    assert cuts[0] == 0 and cuts[-1] == d.M and offs[0] == 0 and offs[-1] == d.nnz
    assert (np.diff(cuts) >= 0).all() and (np.diff(offs) >= 0).all()
    assert np.array_equal(offs, d.row_ptr[cuts])                       # every part starts at the first entry of its first row
    longest = int(np.diff(d.row_ptr).max())
    assert np.diff(offs).max() <= d.nnz / parts + longest
    # aligned cuts, degenerate inputs, unsorted rows
    cuts64, offs64 = coo_cuts(rows, d.M, parts, align=64)
    assert all(int(c) % 64 == 0 for c in cuts64[1:-1]) and np.array_equal(offs64, d.row_ptr[cuts64])
    c, o = coo_cuts(np.array([2, 2, 2, 2, 2], np.int32), 3, 2)
    assert c.tolist() == [0, 2, 3] and o.tolist() == [0, 0, 5]          # all entries in the last row
    c, o = coo_cuts(np.zeros(0, np.int32), 4, 2)
    assert c[[0, -1]].tolist() == [0, 4] and o.tolist() == [0, 0, 0]   # empty matrix
    with pytest.raises(ValueError):
        coo_cuts(np.array([0, 1, 2, 9, 3, 3], np.int32), 4, 2)          # the entry a cut looks at lies outside [0, M)


def test_block_grid_cuts_columns_only_where_b_exceeds_l2_and_rows_are_long():
    assert block_grid(8, 1453908, 1453908, 32, 37497844) == (2, 4)      # Poisson rows, B 186 MB: slices of 46 MB
    assert block_grid(4, 1453908, 1453908, 32, 37497844) == (1, 4)
    assert block_grid(2, 1453908, 1453908, 32, 37497844) == (1, 2)
    assert block_grid(1, 1453908, 1453908, 32, 37497844) == (1, 1)
    assert block_grid(8, 2601977, 2601977, 32, 36200056) == (8, 1)      # power-law rows, mean 14: row ranges (the engine cuts the long rows itself)
    assert block_grid(8, 14340, 14340, 32, 18070000) == (8, 1)          # B fits L2
    assert block_grid(8, 503712, 503712, 64, 36799047) == (8, 1)        # B about the size of L2
    assert block_grid(8, 1453908, 1453908, 64, 37497844) == (2, 4)
    assert block_grid(2, 1453908, 1453908, 64, 37497844) == (2, 1)      # a half of B (186 MB) would still not fit L2
    assert block_grid(8, 1453908, 1453908, 128, 37497844) == (8, 1)     # rows of 512 bytes: A would be re-read once per column part
    assert block_grid(8, 1453908, 1453908, 64, 37497844, elem_bytes=2) == (8, 1)   # bf16 storage


@pytest.mark.parametrize("world,grid", [(4, (1, 4)), (8, (2, 4)), (2, (2, 1)), (6, (3, 2))])
def test_blocks_of_a_grid_assemble_the_whole_result(world, grid):
    """Every block is a problem of its own (local row_ptr, re-based columns, its rows of A and B); computing each with
    the CPU oracle and writing the pieces back through `sel` gives the unsharded result bit for bit."""
    sys.path.insert(0, str(ROOT / "oracle"))
    import oracle_lib
    orc = oracle_lib.Oracle()
    d = Dataset(5, 8, 0.02)
    want = orc.sddmm_csr(d.M, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B)
    got = np.full(d.nnz, np.nan, np.float32)
    total = 0
    for r in range(world):
        b = block_shard(d.row_ptr, d.col_idx, d.s_val, d.A, d.B, r, grid)
        assert b["rp"][0] == 0 and b["rp"][-1] == b["nnz"] == b["col"].size == b["val"].size
        assert b["A"].shape[0] == b["M"] and b["B"].shape[0] == b["N"] == b["c1"] - b["c0"]
        assert b["nnz"] == 0 or (0 <= b["col"].min() and b["col"].max() < b["N"])
        p = orc.sddmm_csr(b["M"], d.K, b["rp"], b["col"], b["val"], np.ascontiguousarray(b["A"]), np.ascontiguousarray(b["B"]))
        if b["sel"] is None:
            got[b["j0"]:b["j1"]] = p
        else:
            got[b["sel"]] = p
        total += b["nnz"]
    assert total == d.nnz and np.array_equal(got, want)


def test_shard_slices_rebase_row_ptr():
    d = Dataset(5, 8, 0.005)
    pieces = [shard(d.row_ptr, d.col_idx, d.s_val, d.A, r, 3) for r in range(3)]
    assert sum(p[3].size for p in pieces) == d.nnz
    for r0, r1, rp, ci, sv, A in pieces:
        assert rp[0] == 0 and rp[-1] == ci.size == sv.size and A.shape[0] == r1 - r0 and rp.size == r1 - r0 + 1
    assert np.array_equal(np.concatenate([p[3] for p in pieces]), d.col_idx)


def _rank_main(rank, world, port, out_dir):
    import torch.distributed as dist

    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "oracle"))
    import oracle_lib

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import torch

    d = Dataset(4, 32, 0.004)
    orc = oracle_lib.Oracle()
    # rank 0 owns B and broadcasts it once, like the NCCL broadcast before the timed region
    B = torch.from_numpy(np.ascontiguousarray(d.B).copy()) if rank == 0 else torch.empty((d.N, d.K), dtype=torch.float32)
    dist.broadcast(B, src=0)
    r0, r1, rp, ci, sv, A = shard(d.row_ptr, d.col_idx, d.s_val, d.A, rank, world)
    p_local = orc.sddmm_csr(r1 - r0, d.K, rp, ci, sv, A, B.numpy())
    sizes = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(sizes, torch.tensor([p_local.size], dtype=torch.int64))
    bufs = [torch.empty(int(s.item()), dtype=torch.float32) for s in sizes]
    dist.all_gather(bufs, torch.from_numpy(p_local)) if len({int(s.item()) for s in sizes}) == 1 else None
    if len({int(s.item()) for s in sizes}) != 1:  # ragged shards: gather through rank 0 with point-to-point sends
        if rank == 0:
            bufs[0] = torch.from_numpy(p_local)
            for r in range(1, world):
                dist.recv(bufs[r], src=r)
        else:
            dist.send(torch.from_numpy(p_local), dst=0)
    if rank == 0:
        full = orc.sddmm_csr(d.M, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B)
        got = np.concatenate([b.numpy() for b in bufs])
        np.save(Path(out_dir) / "ok.npy", np.array([np.array_equal(full, got), got.size == d.nnz]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gloo_sharded_sddmm(tmp_path):
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_rank_main, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    ok = np.load(tmp_path / "ok.npy")
    assert ok.all()
