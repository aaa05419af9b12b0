"""Partitioning of the FP8 blockwise GEMM across the GPUs of one box.

The path shards without any reduction:

* N-split (column-parallel weights): rank r owns a contiguous run of 128-wide
  output groups, i.e. the row slab B_q[n0:n1, :] and B_s[n0/128:n1/128, :]; A
  is replicated; the rank produces C_q[:, n0:n1] and C_s[n0/128:n1/128, :].
  The cut is made on 128-column boundaries so that no 1x128 output group and no
  128x128 weight block straddles two ranks; when the number of groups is not a
  multiple of the world size the first ranks take one group more.
* M-split (independent rows): rank r owns rows [m0, m1) of A_q; the scale
  arrays are M-minor ([K/128, M], [N/128, M]), so a rank's part is a column
  band that is re-packed to the local leading dimension m1 - m0.

A collective is needed only when the caller wants the whole C on every rank:
`all_gather_c_n` / `all_gather_c_m` use torch.distributed (NCCL over NVLink on
GPUs, gloo in the CPU tests).

The reference has no multi-GPU code; the layouts cut here are the ones its
kernels define (examples/005.fp8.mm.cu:1059-1063 for A_s/B_s, :1136 for C_s).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def split_groups(n_groups: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous, near-even split of `n_groups` items; returns [g0, g1)."""
    if not (0 <= rank < world):
        raise ValueError("rank out of range")
    base, extra = divmod(n_groups, world)
    g0 = rank * base + min(rank, extra)
    g1 = g0 + base + (1 if rank < extra else 0)
    return g0, g1


def split_n(N: int, world: int, rank: int) -> tuple[int, int]:
    """Column range [n0, n1) of rank `rank`, cut on 128-column group boundaries."""
    if N % 128:
        raise ValueError("N must be a multiple of 128")
    g0, g1 = split_groups(N // 128, world, rank)
    return g0 * 128, g1 * 128


def split_m(M: int, world: int, rank: int) -> tuple[int, int]:
    """Row range [m0, m1) of rank `rank`."""
    return split_groups(M, world, rank)


def shard_weights_n(B_q: torch.Tensor, B_s: torch.Tensor, world: int, rank: int):
    """Rank's slab of B_q[N,K] and B_s[N/128,K/128] (views, contiguous)."""
    n0, n1 = split_n(B_q.shape[0], world, rank)
    return B_q[n0:n1], B_s[n0 // 128:n1 // 128]


def shard_activations_m(A_q: torch.Tensor, A_s: torch.Tensor, world: int, rank: int):
    """Rank's rows of A_q[M,K] and the matching band of A_s[K/128,M], re-packed
    so that the local leading dimension of the scales is the local row count."""
    m0, m1 = split_m(A_q.shape[0], world, rank)
    return A_q[m0:m1].contiguous(), A_s[:, m0:m1].contiguous()


def _all_gather_var(t: torch.Tensor, dim: int, sizes: list[int], group=None) -> torch.Tensor:
    """all_gather of tensors whose extent along `dim` differs per rank
    (`sizes[r]`); pads to the largest, gathers, trims and concatenates."""
    world = dist.get_world_size(group)
    big = max(sizes)
    moved = t.movedim(dim, 0).contiguous()
    pad_shape = (big,) + tuple(moved.shape[1:])
    buf = torch.zeros(pad_shape, dtype=t.dtype, device=t.device)
    buf[:moved.shape[0]] = moved
    out = [torch.empty_like(buf) for _ in range(world)]
    dist.all_gather(out, buf, group=group)
    parts = [o[:sizes[r]] for r, o in enumerate(out)]
    return torch.cat(parts, dim=0).movedim(0, dim).contiguous()


def all_gather_c_n(C_q: torch.Tensor, C_s: torch.Tensor, N: int, group=None):
    """N-split outputs -> full C_q[M,N] and C_s[N/128,M] on every rank."""
    world = dist.get_world_size(group)
    cols = [split_n(N, world, r) for r in range(world)]
    q = _all_gather_var(C_q, 1, [b - a for a, b in cols], group)
    s = _all_gather_var(C_s, 0, [(b - a) // 128 for a, b in cols], group)
    return q, s


def all_gather_c_m(C_q: torch.Tensor, C_s: torch.Tensor, M: int, group=None):
    """M-split outputs -> full C_q[M,N] and C_s[N/128,M] on every rank."""
    world = dist.get_world_size(group)
    rows = [split_m(M, world, r) for r in range(world)]
    q = _all_gather_var(C_q, 0, [b - a for a, b in rows], group)
    s = _all_gather_var(C_s, 1, [b - a for a, b in rows], group)
    return q, s


class PeerOutputs:
    """Full-size outputs C_q [M, N] / C_s [N/128, M] on every rank of an N-split, each rank's pair mapped into
    every other rank's process (CUDA IPC through torch's storage sharing, peer access enabled), for
    `capi.fp8_blockwise_mm_gather`: a rank's GEMM stores its column shard into all of them, so the all-gather
    is done by the epilogue's peer stores.  One process per GPU, all GPUs of one box visible to every process.

    `dsts()` gives the destination lists (own buffers first); after the GEMM, `wait_all()` (stream
    synchronisation + a barrier of the group) is the point from which every rank may read its whole C."""

    def __init__(self, M: int, N: int, device, group=None):
        if N % 128:
            raise ValueError("N must be a multiple of 128")
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.device = torch.device(device)
        self.C_q = torch.empty(M, N, dtype=torch.uint8, device=self.device)
        self.C_s = torch.empty(N // 128, M, dtype=torch.float32, device=self.device)
        mine = (self.device.index, self.C_q.untyped_storage()._share_cuda_(), self.C_s.untyped_storage()._share_cuda_())
        everyone = [None] * self.world
        dist.all_gather_object(everyone, mine, group=group)
        self.peer_q, self.peer_s, self._keep = [], [], []
        for r, (dev_index, hq, hs) in enumerate(everyone):
            if r == self.rank:
                continue
            _enable_peer_access(self.device.index, dev_index)
            sq = torch.UntypedStorage._new_shared_cuda(*hq)
            ss = torch.UntypedStorage._new_shared_cuda(*hs)
            self._keep += [sq, ss]
            self.peer_q.append(torch.empty(0, dtype=torch.uint8, device=f"cuda:{dev_index}").set_(sq, 0, (M, N)))
            self.peer_s.append(torch.empty(0, dtype=torch.float32, device=f"cuda:{dev_index}").set_(ss, 0, (N // 128, M)))
        dist.barrier(group=group)

    def dsts(self):
        """(C_q destinations, C_s destinations) as raw device addresses, own buffers first."""
        return ([self.C_q.data_ptr()] + [t.data_ptr() for t in self.peer_q],
                [self.C_s.data_ptr()] + [t.data_ptr() for t in self.peer_s])

    def wait_all(self) -> None:
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)

    def close(self) -> None:
        """Unmaps the peers' buffers (every rank must call it, before the owners free theirs)."""
        self.wait_all()
        self.peer_q, self.peer_s, self._keep = [], [], []
        torch.cuda.ipc_collect()
        dist.barrier(group=self.group)


def _enable_peer_access(device_index: int, peer_index: int) -> None:
    """cudaDeviceEnablePeerAccess(peer) with `device_index` current (kernels, unlike copies, need it explicitly)."""
    import ctypes
    if device_index == peer_index:
        return
    if not torch.cuda.can_device_access_peer(device_index, peer_index):
        raise RuntimeError(f"GPU {device_index} cannot access GPU {peer_index} directly")
    rt = ctypes.CDLL("libcudart.so.12")
    with torch.cuda.device(device_index):
        torch.cuda.current_stream().synchronize()  # the context exists
        rc = rt.cudaDeviceEnablePeerAccess(ctypes.c_int(peer_index), ctypes.c_uint(0))
        if rc not in (0, 704):  # 704: peer access already enabled
            raise RuntimeError(f"cudaDeviceEnablePeerAccess({peer_index}) failed with CUDA error {rc}")
        rt.cudaGetLastError()
