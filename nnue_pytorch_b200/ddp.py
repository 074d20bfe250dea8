"""Gradient exchange between data-parallel ranks (one process per GPU).

The reference wraps its model in `DistributedDataParallel`
(trainer/engine.py:149-162 of the reference project): every gradient is
averaged over the ranks during backward and every rank then runs the same
optimizer step.  `make_grad_hook` gives `TrainStep` the same result: the small
dense-layer gradients travel as one flat bucket, the feature-transformer
table gradient (23232 x 3080 fp32, 286 MB) as its own all-reduce.  NCCL over
NVLink/NVSwitch does the wire work; with one rank nothing is exchanged.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

_BIG = 1 << 22  # elements; tensors at least this large are reduced on their own


def make_grad_hook(model: torch.nn.Module, world: int, average: bool = True, skip=()):
    """`average=False` leaves rank SUMS in `.grad`; the caller then folds the
    division by `world` into the scalar its optimizer multiplies gradients by
    (`TrainStep` does), which saves a read-modify-write pass over the table."""
    if world <= 1:
        return None
    inv = 1.0 / world if average else 1.0
    skipped = {id(p) for p in skip}  # parameters another mechanism exchanges

    def hook(m: torch.nn.Module) -> None:
        grads = [p.grad for p in m.parameters() if p.grad is not None and id(p) not in skipped]
        small = [g for g in grads if g.numel() < _BIG]
        for g in grads:
            if g.numel() >= _BIG:
                dist.all_reduce(g)
                if inv != 1.0:
                    g.mul_(inv)
        if small:
            flat = torch.cat([g.reshape(-1) for g in small])
            dist.all_reduce(flat)
            if inv != 1.0:
                flat.mul_(inv)
            at = 0
            for g in small:
                n = g.numel()
                g.copy_(flat[at : at + n].view_as(g))
                at += n

    return hook


def _map_peers(local: torch.Tensor, group) -> tuple[list[int], object]:
    """Device pointers of `local`'s counterpart on every rank of `group`, valid in
    this process.  `local` must come from `_alloc_shared`.  Returns the pointer
    list and an object that must stay alive as long as the pointers are used."""
    handle = getattr(local, "_nnue_symm_handle", None)
    if handle is not None:
        return [int(p) for p in handle.buffer_ptrs], handle
    # CUDA IPC: every rank exports its allocation, everyone opens everyone else's
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    exported = local.untyped_storage()._share_cuda_()
    gathered: list = [None] * world
    dist.all_gather_object(gathered, exported, group=group)
    keep, ptrs = [], []
    for r in range(world):
        if r == rank:
            ptrs.append(local.data_ptr())
            continue
        storage = torch.UntypedStorage._new_shared_cuda(*gathered[r])
        keep.append(storage)
        ptrs.append(storage.data_ptr())
    return ptrs, keep


def _alloc_shared(numel: int, device: torch.device, group) -> torch.Tensor:
    """A float32 buffer every rank of `group` can map: torch symmetric memory when
    it is available, a plain allocation (shared through CUDA IPC) otherwise."""
    try:
        import torch.distributed._symmetric_memory as symm_mem

        t = symm_mem.empty(numel, dtype=torch.float32, device=device)
        t._nnue_symm_handle = symm_mem.rendezvous(t, group)
        return t
    except Exception:  # noqa: BLE001 - any failure here means "use IPC instead"
        return torch.empty(numel, dtype=torch.float32, device=device)


def shard_range(n_rows: int, width: int, world: int, rank: int) -> tuple[int, int]:
    """Element range [begin, end) of rank's row shard: whole rows, ceil-split."""
    per = (n_rows + world - 1) // world
    r0, r1 = min(n_rows, rank * per), min(n_rows, (rank + 1) * per)
    return r0 * width, r1 * width


class ShardedTableExchange:
    """Owner of the feature-transformer table under data parallelism.

    Every rank keeps the full table (the forward gathers from anywhere) but
    optimizer state only for its own shard of rows.  Per step:
      reduce()  peer-load reduce-scatter of the gradient + squared norm,
      update()  RangerLite on the shard + peer-store all-gather of the rows.
    The table parameter's storage and the gradient buffer live in memory all
    ranks have mapped; `install()` points the kernels' gradient sink at it."""

    def __init__(self, param: torch.nn.Parameter, group=None, pnm: bool = True, lookahead: bool = True):
        assert param.is_cuda and param.dim() == 2 and param.dtype == torch.float32
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.param = param
        n, w = param.shape
        assert w % 4 == 0, "table width must be a multiple of 4 floats"
        dev = param.device
        self.table = _alloc_shared(n * w, dev, self.group)
        self.grad = _alloc_shared(n * w, dev, self.group)
        self.table.copy_(param.data.reshape(-1))
        param.data = self.table.view(n, w)  # the model now reads the shared table
        self.table_ptrs, self._keep_t = _map_peers(self.table, self.group)
        self.grad_ptrs, self._keep_g = _map_peers(self.grad, self.group)
        self.begin, self.end = shard_range(n, w, self.world, self.rank)
        m = self.end - self.begin
        self.grad_ma = torch.zeros(m, device=dev)
        self.variance_ma = torch.zeros(m, device=dev)
        self.neg_grad_ma = torch.zeros(m, device=dev) if pnm else None
        self.slow = self.table[self.begin : self.end].clone() if lookahead else None
        self.step = 0
        self.ft_sumsq = torch.zeros(1, device=dev)
        self._token = torch.zeros(1, device=dev)
        self.grad_view = self.grad.view(n, w)

    def install(self) -> None:
        from . import _launch

        _launch.GRAD_SINK = self.grad_view

    def reduce(self) -> torch.Tensor:
        """After every rank's backward (the caller has put a collective in between):
        sums this rank's shard over the ranks.  Returns the squared norm of the whole
        summed gradient (all-reduced scalar), which also fences the phase."""
        from . import _launch

        self.ft_sumsq.zero_()
        _launch.ddp_reduce_shard(self.grad_ptrs, self.rank, self.begin, self.end, self.ft_sumsq)
        dist.all_reduce(self.ft_sumsq, group=self.group)
        return self.ft_sumsq

    def update(self, hp, grad_scale: torch.Tensor | None) -> None:
        from . import _launch

        _launch.ddp_update_shard(self.table_ptrs, self.rank, self.begin, self.end, self.grad, self.grad_ma,
                                 self.neg_grad_ma, self.variance_ma, self.slow, grad_scale, hp)
        # nobody may read its table before every rank has stored its shard into it
        dist.all_reduce(self._token, group=self.group)

    def state_dict(self) -> dict:
        """Full-size optimizer state of the table, gathered from the shards (same keys as RangerLite)."""
        out = {"step": self.step}
        for key, t in (("grad_ma", self.grad_ma), ("variance_ma", self.variance_ma),
                       ("neg_grad_ma", self.neg_grad_ma), ("lookahead_params", self.slow)):
            if t is None:
                continue
            per = (self.param.shape[0] + self.world - 1) // self.world * self.param.shape[1]
            padded = torch.zeros(per, device=t.device)
            padded[: t.numel()] = t
            parts = [torch.empty_like(padded) for _ in range(self.world)]
            dist.all_gather(parts, padded, group=self.group)
            out[key] = torch.cat(parts)[: self.param.numel()].view_as(self.param).clone()
        return out
