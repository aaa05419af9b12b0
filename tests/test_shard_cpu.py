"""Multi-GPU partitioning logic on CPU: split arithmetic, and a world_size-2
gloo run in which each rank computes its shard with the oracle and the gathered
result must equal the unsharded computation bit for bit (the path has no
reduction, so sharding may not change a single byte)."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import fp8_sources
from llmmm_b200 import shard

ROOT = Path(__file__).resolve().parent.parent


def test_split_groups_cover_and_balance():
    for n, w in [(28, 8), (296, 8), (48, 4), (5, 8), (20, 2), (152, 8)]:
        parts = [shard.split_groups(n, w, r) for r in range(w)]
        assert parts[0][0] == 0 and parts[-1][1] == n
        assert all(parts[i][1] == parts[i + 1][0] for i in range(w - 1))
        sizes = [b - a for a, b in parts]
        assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)


def test_split_n_is_on_group_boundaries():
    # 7B down-projection: N = 3584 = 28 groups over 8 ranks -> 4,4,4,4,3,3,3,3 groups
    cols = [shard.split_n(3584, 8, r) for r in range(8)]
    assert [(b - a) // 128 for a, b in cols] == [4, 4, 4, 4, 3, 3, 3, 3]
    assert all(a % 128 == 0 and b % 128 == 0 for a, b in cols)
    with pytest.raises(ValueError):
        shard.split_n(100, 2, 0)
    with pytest.raises(ValueError):
        shard.split_groups(4, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, mode, q):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import oracle as o
        o.set_num_threads(2)
        M, N, K = 24, 384, 256  # 3 output groups over 2 ranks: an uneven N-split
        x, w = fp8_sources(21, M, N, K, w_std=0.02)
        A_q, A_s = o.quant_1x128(x)
        B_q, B_s = o.quant_128x128(w)
        full_q, full_s, _ = o.fp8_blockwise_mm(A_q, A_s, B_q, B_s)
        tA_q, tA_s, tB_q, tB_s = map(torch.from_numpy, (A_q, A_s, B_q, B_s))
        if mode == "nb":
            # even split (the first two of the three groups, one per rank) gathered in the blocked layout
            N2 = 256
            full2_q, full2_s, _ = o.fp8_blockwise_mm(A_q, A_s, B_q[:N2], B_s[:2])
            bq, bs = shard.shard_weights_n(tB_q[:N2], tB_s[:2], world, rank)
            cq, cs, _ = o.fp8_blockwise_mm(A_q, A_s, bq.numpy(), bs.numpy())
            blk, gs = shard.all_gather_c_n_blocked(torch.from_numpy(cq), torch.from_numpy(cs))
            assert tuple(blk.shape) == (world, M, N2 // world)
            gq = torch.cat([shard.unblock_c_n(blk), torch.from_numpy(full_q[:, N2:])], dim=1)
            gs = torch.cat([gs, torch.from_numpy(full_s[2:])], dim=0)
            assert (shard.unblock_c_n(blk).numpy() == full2_q).all() and (gs[:2].numpy() == full2_s).all()
        elif mode == "n":
            bq, bs = shard.shard_weights_n(tB_q, tB_s, world, rank)
            cq, cs, _ = o.fp8_blockwise_mm(A_q, A_s, bq.numpy(), bs.numpy())
            gq, gs = shard.all_gather_c_n(torch.from_numpy(cq), torch.from_numpy(cs), N)
        else:
            aq, as_ = shard.shard_activations_m(tA_q, tA_s, world, rank)
            cq, cs, _ = o.fp8_blockwise_mm(aq.numpy(), as_.numpy(), B_q, B_s)
            gq, gs = shard.all_gather_c_m(torch.from_numpy(cq), torch.from_numpy(cs), M)
        ok = bool((gq.numpy() == full_q).all() and (gs.numpy().view(np.uint32) == full_s.view(np.uint32)).all())
        q.put((rank, ok, tuple(gq.shape), tuple(gs.shape)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["n", "m", "nb"])
def test_two_rank_gloo_shard_and_gather(mode, oracle):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, mode, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok, qs, ss in results:
        assert ok, f"rank {rank}: gathered shards differ from the unsharded result"
        assert qs == (24, 384) and ss == (3, 24)
