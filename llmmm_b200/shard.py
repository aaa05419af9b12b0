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


def all_gather_c_n_blocked(C_q: torch.Tensor, C_s: torch.Tensor, group=None):
    """N-split outputs of equal width -> (C_q blocked [R, M, N_r], C_s [N/128, M]) on every rank with one
    all_gather_into_tensor each: rank r's slab C_q[:, n0:n1] lands as block r, unchanged, and the C_s slabs
    concatenate along dim 0 as they are.  No transpose, padding or copy around the collective: this is the plain
    NCCL all-gather a consumer that accepts the blocked layout pays (block r, row m holds columns
    [r N_r, (r+1) N_r) of row m).  Uneven splits go through all_gather_c_n."""
    world = dist.get_world_size(group)
    out_q = torch.empty((world * C_q.shape[0], C_q.shape[1]), dtype=C_q.dtype, device=C_q.device)
    out_s = torch.empty((world * C_s.shape[0], C_s.shape[1]), dtype=C_s.dtype, device=C_s.device)
    dist.all_gather_into_tensor(out_q, C_q.contiguous(), group=group)
    dist.all_gather_into_tensor(out_s, C_s.contiguous(), group=group)
    return out_q.view(world, C_q.shape[0], C_q.shape[1]), out_s


def unblock_c_n(C_blocked: torch.Tensor) -> torch.Tensor:
    """[R, M, N_r] -> row-major [M, R * N_r] (one copy), for consumers that need it."""
    R, M, Nr = C_blocked.shape
    return C_blocked.permute(1, 0, 2).reshape(M, R * Nr)


def all_gather_c_m(C_q: torch.Tensor, C_s: torch.Tensor, M: int, group=None):
    """M-split outputs -> full C_q[M,N] and C_s[N/128,M] on every rank."""
    world = dist.get_world_size(group)
    rows = [split_m(M, world, r) for r in range(world)]
    q = _all_gather_var(C_q, 0, [b - a for a, b in rows], group)
    s = _all_gather_var(C_s, 1, [b - a for a, b in rows], group)
    return q, s


class PeerOutputs:
    """Full-size outputs C_q [M, N] / C_s [N/128, M] on every rank of an N-split, each rank's pair mapped into
    every other rank's address space, for `capi.fp8_blockwise_mm_gather`: a rank's GEMM stores its column shard
    into all of them, so the all-gather is done by the epilogue's peer stores.  The buffers come from torch's
    symmetric memory (`torch.distributed._symmetric_memory`: device memory created with the virtual-memory API,
    exported to the other processes of the group and mapped with access for this GPU); one process per GPU.

    `dsts()` gives the destination address lists (every rank once); after the GEMM, `wait_all()` (stream
    synchronisation + a barrier of the group) is the point from which every rank may read its whole C."""

    def __init__(self, M: int, N: int, device, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        if N % 128:
            raise ValueError("N must be a multiple of 128")
        self.group = dist.group.WORLD if group is None else group
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.device = torch.device(device)
        with torch.cuda.device(self.device):
            self._q = symm_mem.empty(M * N, dtype=torch.uint8, device=self.device)
            self._s = symm_mem.empty((N // 128) * M, dtype=torch.float32, device=self.device)
            self._hq = symm_mem.rendezvous(self._q, self.group)
            self._hs = symm_mem.rendezvous(self._s, self.group)
        self.C_q = self._q.view(M, N)
        self.C_s = self._s.view(N // 128, M)
        if len(self._hq.buffer_ptrs) != self.world or self._hq.buffer_ptrs[self.rank] != self._q.data_ptr():
            raise RuntimeError("symmetric memory rendezvous returned an unexpected set of buffers")
        dist.barrier(group=self.group)

    def dsts(self):
        """(C_q destinations, C_s destinations) as raw device addresses valid on this GPU, every rank once, starting
        with the rank after this one: the kernel stores to the destinations in list order, and if all ranks began
        with rank 0 they would all push into the same GPU's NVLink ports at the same time."""
        order = [(self.rank + 1 + i) % self.world for i in range(self.world)]
        return [self._hq.buffer_ptrs[r] for r in order], [self._hs.buffer_ptrs[r] for r in order]

    def wait_all(self) -> None:
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)

    def close(self) -> None:
        """Every rank calls it before the buffers go away: no rank may still be storing into a peer."""
        self.wait_all()
