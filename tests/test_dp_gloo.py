"""The data-parallel reduction order, on CPU ranks (gloo, world_size 2 and 4).

The device path packs one LoRA-gradient set per chunk, reduces the local chunks in a
binary tree over the chunk index, all-gathers the per-rank partial sums and finishes the
tree in rank order. The claim under test: because the tree is over CHUNKS, every world
size produces the bits of the single-process tree — and every rank ends with the same
bits. Host model of the device kernels: see_ml_b200.dp.tree_sum_host."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from see_ml_b200.dp import gradient_spans, tree_sum_host
from see_ml_b200 import formats as F

K, FPS = 8, 1000


def _chunk_sets():
    rng = np.random.default_rng(42)
    # wide dynamic range so that summation order changes the bits
    return (rng.standard_normal((K, FPS)) * np.exp(rng.uniform(-8, 8, (K, FPS)))).astype(np.float32)


def _rank_main(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sets = _chunk_sets()
    local = K // world
    mine = sets[rank * local:(rank + 1) * local]           # consecutive chunks per rank
    partial = torch.from_numpy(tree_sum_host(mine))        # local subtree
    gathered = [torch.empty(FPS) for _ in range(world)]
    dist.all_gather(gathered, partial)
    total = tree_sum_host(np.stack([g.numpy() for g in gathered])) * np.float32(1.0 / K)
    np.save(os.path.join(out_dir, f"r{rank}.npy"), total)
    dist.barrier()
    dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world", [2, 4])
def test_chunk_tree_is_world_size_invariant(world, tmp_path):
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    want = tree_sum_host(_chunk_sets()) * np.float32(1.0 / K)      # the one-process tree
    naive = _chunk_sets().sum(0, dtype=np.float32) * np.float32(1.0 / K)
    assert not np.array_equal(want, naive), "inputs too tame to tell summation orders apart"
    for r in range(world):
        got = np.load(tmp_path / f"r{r}.npy")
        np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))


def test_gradient_spans_follow_the_optimiser_instructions(golden_dir):
    z = np.load(os.path.join(golden_dir, "plans.npz"))
    p = F.parse_plan(z["llama_tiny"].tobytes())
    offs, counts = gradient_spans(p.train)
    n_opt = int(np.sum(p.train["opcode"] == int(F.Op.ADAMW)))
    assert len(offs) == n_opt == 24
    # one (A, B) pair per adapter; every span inside the arena and 4-byte aligned
    assert np.all(offs % 4 == 0) and np.all(offs + counts * 4 <= p.header.arena_size)
