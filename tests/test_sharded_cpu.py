"""The N > 1 path on CPU: two gloo ranks follow the library's shard plan, each computes its row
block with the CPU oracle, the slices are all-gathered, and the assembled y must equal the
unsharded oracle result bit for bit (rows are independent, so sharding changes no number)."""
import os
import socket

import numpy as np
import pytest

from demonic_b200 import sharded, synth


def test_shard_plan_covers_every_row_once():
    for n in (65536, 8192, 10, 7, 1, 100003):
        for world in (1, 2, 3, 4, 8):
            edges = [sharded.shard_range(n, r, world) for r in range(world)]
            assert edges[0][0] == 0 and edges[-1][1] == n
            for (a0, a1), (b0, b1) in zip(edges, edges[1:]):
                assert a1 == b0 and a0 <= a1
            sizes = [b - a for a, b in edges]
            assert max(sizes) - min(sizes) <= 1
    assert sharded.shard_range(65536, 3, 8) == (24576, 32768)


def test_every_rank_chooses_the_same_exchange():
    """The exchange (fused into the kernel, or NCCL) is chosen from facts that are equal on every
    rank, never from a rank's own slice: with fewer rows than ranks some slices are empty, and a rank
    that went the other way would leave its peers waiting for it."""
    from demonic_b200 import _lib
    lib = _lib.load()
    for world in (2, 4, 8):
        for n in (1, 3, world - 1, world, 65536):
            for knob in (-1, 0, 1):
                for peers_ok in (0, 1):
                    want = lib.dmc_cuda_shard_path(world, peers_ok, knob, 8192, n)
                    # the rule takes no rank and no slice, so it cannot differ between ranks; empty slices keep it
                    empty = [r for r in range(world) if sharded.shard_range(n, r, world)[0] == sharded.shard_range(n, r, world)[1]]
                    assert (n < world) == bool(empty)
                    assert want == int(peers_ok and knob != 0 and n > 0)
    assert lib.dmc_cuda_shard_path(1, 1, -1, 8192, 100) == 0        # a world of one exchanges nothing by default
    assert lib.dmc_cuda_shard_path(1, 1, 1, 8192, 100) == 1         # ... unless asked (the single-GPU tests do)
    assert lib.dmc_cuda_shard_path(8, 1, -1, 0, 100) == 0           # empty contraction: y is zero, nothing to exchange


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, n, k, out_dir):
    import torch
    import torch.distributed as dist

    import oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(77)                     # every rank draws the same full problem
    w = synth.bf16_weights(rng, (n, k))
    x = synth.activations(rng, (1, k))
    r0, r1 = sharded.shard_range(n, rank, world)
    mine = oracle.gemm_bf16_fma(x, np.ascontiguousarray(w[r0:r1].T))[0]
    # ragged all-gather the way the library does it: every rank broadcasts its slice
    y = torch.zeros(n, dtype=torch.float32)
    y[r0:r1] = torch.from_numpy(mine)
    for r in range(world):
        a, b = sharded.shard_range(n, r, world)
        if b > a:
            piece = y[a:b].clone()
            dist.broadcast(piece, src=r)
            y[a:b] = piece
    full = oracle.gemm_bf16_fma(x, np.ascontiguousarray(w.T))[0]
    ok = np.array_equal(y.numpy().view(np.uint32), full.view(np.uint32))
    np.save(os.path.join(out_dir, f"ok{rank}.npy"), np.array([ok]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("n", [64, 61])
def test_two_gloo_ranks_assemble_the_unsharded_result(tmp_path, n):
    import torch.multiprocessing as mp
    port = _free_port()
    mp.spawn(_rank_main, args=(2, port, n, 256, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        assert bool(np.load(tmp_path / f"ok{r}.npy")[0]), f"rank {r}: assembled y differs from the unsharded result"
