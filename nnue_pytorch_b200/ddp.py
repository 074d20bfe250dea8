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
            views, at = [], 0
            for g in small:
                n = g.numel()
                views.append(flat[at : at + n].view_as(g))
                at += n
            torch._foreach_copy_(small, views)  # one multi-tensor launch instead of one copy per tensor

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


def shard_ranges(bounds: list[int], width: int, world: int, rank: int) -> list[tuple[int, int]]:
    """One element range per row slice [bounds[i], bounds[i+1]): rank's ceil-split
    share of that slice.  Every rank owns a part of every slice, so all ranks
    reduce a slice at the same time."""
    out = []
    for b0, b1 in zip(bounds[:-1], bounds[1:]):
        e0, e1 = shard_range(b1 - b0, width, world, rank)
        out.append((b0 * width + e0, b0 * width + e1))
    return out


def gather_sharded(local: torch.Tensor, bounds: list[int], width: int, group) -> torch.Tensor:
    """Full [bounds[-1] * width] tensor from every rank's shares.  `local` is this rank's shares of all
    slices back to back (the layout of `ShardedTableExchange`'s optimizer state); collective."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    full = torch.zeros(bounds[-1] * width, dtype=local.dtype, device=local.device)
    at = 0
    for b0, b1 in zip(bounds[:-1], bounds[1:]):
        per = (b1 - b0 + world - 1) // world * width  # the largest share of this slice
        e0, e1 = shard_range(b1 - b0, width, world, rank)
        if per == 0:
            continue
        padded = torch.zeros(per, dtype=local.dtype, device=local.device)
        padded[: e1 - e0] = local[at : at + (e1 - e0)]
        at += e1 - e0
        parts = [torch.empty_like(padded) for _ in range(world)]
        dist.all_gather(parts, padded, group=group)
        # shares are ceil-split: every rank but the last ones holds `per` elements, so the padded
        # concatenation has the slice's elements in front
        full[b0 * width : b1 * width] = torch.cat(parts)[: (b1 - b0) * width]
    return full


def scatter_full(full: torch.Tensor, bounds: list[int], width: int, world: int, rank: int) -> torch.Tensor:
    """This rank's shares of `full` ([bounds[-1] * width] or [rows, width]), slice after slice: the
    inverse of `gather_sharded`; no communication."""
    flat = full.reshape(-1)
    return torch.cat([flat[e0:e1] for e0, e1 in shard_ranges(bounds, width, world, rank)])


class ShardedTableExchange:
    """Owner of the feature-transformer table under data parallelism.

    Every rank keeps the full table (the forward gathers from anywhere) but
    optimizer state only for its own share of the rows.  Per step:
      reduce()  peer-load reduce-scatter of the gradient + squared norm,
      update()  RangerLite on the share + peer-store all-gather of the rows.
    The table parameter's storage and the gradient buffer live in memory all
    ranks have mapped; `install()` points the kernels' gradient sink at it.

    `slices` (row bounds, first 0, last the row count) makes the backward
    deliver the gradient slice by slice (`nnue_ft_fused_bwd_sliced`) and the
    reduce of slice i run on a second stream while slice i + 1 is still being
    computed.  With the flat HalfKAv2_hm^ table, [0, 22528, 23232] puts the 704
    factor rows, which collect half of all entries, last: nearly the whole
    reduce traffic then hides behind their computation."""

    def __init__(self, param: torch.nn.Parameter, group=None, pnm: bool = True, lookahead: bool = True,
                 slices: list[int] | None = None, reduce_ctas: int = 32, col_slices: list[int] | None = None):
        """`reduce_ctas`: grid cap of the peer-load reduce while it runs beside the sliced backward
        (it needs few SMs to fill the links and takes them from the gather kernel); measured on
        8 GPUs: 32 -> 3.42 ms per step, 64 -> 3.43, 96 -> 3.53, uncapped and unsliced 3.55.
        `col_slices` (column bounds in floats, first 0, last the row width, inner ones multiples of
        `_launch.bwd_column_tile`) slices the gradient by columns instead: the backward's gather-sum walks the
        columns tile by tile anyway, so the slices cost it nothing, every rank keeps ONE share of whole rows, and
        the reduce of column slice i (this rank's rows, those columns) runs beside the computation of slice i + 1."""
        assert param.is_cuda and param.dim() == 2 and param.dtype == torch.float32
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.param = param
        n, w = param.shape
        assert w % 4 == 0, "table width must be a multiple of 4 floats"
        self.bounds = [0, n] if not slices else [int(b) for b in slices]
        assert self.bounds[0] == 0 and self.bounds[-1] == n and all(
            a <= b for a, b in zip(self.bounds[:-1], self.bounds[1:])), "slices must run from 0 to the row count"
        assert len(self.bounds) - 1 <= 16
        self.col_bounds = None
        if col_slices:
            assert not slices, "row slices and column slices exclude each other"
            self.col_bounds = [int(b) for b in col_slices]
            assert self.col_bounds[0] == 0 and self.col_bounds[-1] == w and len(self.col_bounds) - 1 <= 16 and all(
                a <= b and a % 4 == 0 for a, b in zip(self.col_bounds[:-1], self.col_bounds[1:])), "bad column slices"
        dev = param.device
        self.table = _alloc_shared(n * w, dev, self.group)
        self.grad = _alloc_shared(n * w, dev, self.group)
        self.table.copy_(param.data.reshape(-1))
        param.data = self.table.view(n, w)  # the model now reads the shared table
        self.table_ptrs, self._keep_t = _map_peers(self.table, self.group)
        self.grad_ptrs, self._keep_g = _map_peers(self.grad, self.group)
        self.ranges = shard_ranges(self.bounds, w, self.world, self.rank)
        self.begin, self.end = self.ranges[0][0], self.ranges[-1][1]  # extent (one slice: the shard itself)
        sizes = [e1 - e0 for e0, e1 in self.ranges]
        self.state_at = [0]
        for m_ in sizes:
            self.state_at.append(self.state_at[-1] + m_)
        m = self.state_at[-1]
        self.grad_ma = torch.zeros(m, device=dev)
        self.variance_ma = torch.zeros(m, device=dev)
        self.neg_grad_ma = torch.zeros(m, device=dev) if pnm else None
        self.slow = torch.cat([self.table[e0:e1] for e0, e1 in self.ranges]).clone() if lookahead else None
        self.step = 0
        self.ft_sumsq = torch.zeros(1, device=dev)
        self._token = torch.zeros(1, device=dev)
        self.grad_view = self.grad.view(n, w)
        self.sliced = len(self.ranges) > 1 or self.col_bounds is not None
        self.reduce_ctas = int(reduce_ctas)
        if self.sliced:
            self.comm_stream = torch.cuda.Stream(dev, priority=-1)  # its CTAs go first when an SM frees up
            n_events = len(self.col_bounds) - 1 if self.col_bounds is not None else len(self.ranges)
            self.slice_events = [torch.cuda.Event() for _ in range(n_events)]
            for e in self.slice_events:
                e.record()  # creates the CUDA event the library will record
            self._reduced = torch.cuda.Event()
            self._zeroed = torch.cuda.Event()
            self._zeroed.record()
            self._local_reader = torch.cuda.Event()
        self._local_reader_pending = False
        self._emit = None            # set by ship_integer_rows
        self.fp32_rows_valid = True  # False: rows outside this rank's shares are older than their owner's

    def ship_integer_rows(self, l1_size: int, scale_main: float, scale_psqt: float, fp32_to_peers: bool = False) -> None:
        """From now on `update()` sends the other ranks the rows their forward actually gathers when weights are
        fake-quantized: the int16 table and the fake-quantized PSQT columns (`nnue_ft_quantize_table`'s format,
        (2 L1 + 4 P) bytes per row instead of 4 (L1 + P)), written by the update kernel from the new weights it
        holds in registers.  The forward's values do not change by a bit.

        With `fp32_to_peers=False` the fp32 rows no longer cross NVLink: every rank's parameter tensor stays
        current only inside its own shares until `sync_table()` (called by `uninstall()` and `state_dict()`; call
        it before anything else reads the parameter: evaluation through the fp32 table, serialization).  A weight
        that leaves the packed int16 range (|w * scale| > 4095) has no fp32 route then: `device_status` reports it.
        Collective; the ranks' tables must agree when it is called."""
        from . import _launch

        n, w = self.param.shape
        l1, p = int(l1_size), w - int(l1_size)
        assert l1 % 16 == 0 and p >= 0 and p % 4 == 0, "needs L1 % 16 == 0 and a PSQT width that is a multiple of 4"
        dev = self.table.device
        self._q16_buf = _alloc_shared((n + 1) * l1 // 2, dev, self.group)
        self._psqt_buf = _alloc_shared(max(n * p, 4), dev, self.group)
        self._stats_buf = _alloc_shared(max(2 * (self.world + 1), 4), dev, self.group)
        q16 = self._q16_buf.view(torch.int16).view(n + 1, l1)
        psqt = self._psqt_buf[: n * p].view(n, p)
        stats = self._stats_buf.view(torch.int32)[: 2 * (self.world + 1)]
        q16_ptrs, self._keep_q = _map_peers(self._q16_buf, self.group)
        psqt_ptrs, self._keep_p = _map_peers(self._psqt_buf, self.group)
        stats_ptrs, self._keep_s = _map_peers(self._stats_buf, self.group)
        self._stats_local = torch.zeros(2, dtype=torch.int32, device=dev)
        self._emit = _launch.ddp_emit_struct(q16_ptrs, psqt_ptrs, stats_ptrs, self._stats_local, l1, l1, p,
                                             scale_main, scale_psqt, fp32_to_peers)
        self._emit_key = (l1, float(scale_main), float(scale_psqt))
        self._fp32_to_peers = bool(fp32_to_peers)
        self.cache = _launch.QuantTableCache(owner=self)
        self.cache.q16, self.cache.psqt, self.cache.stats = q16, psqt, stats
        self.param._nnue_q16_cache = self.cache
        self.fp32_rows_valid = True
        self.rebuild_integer_rows()

    def rebuild_integer_rows(self) -> None:
        """The integer table again from the fp32 parameter, on every rank (after something other than `update()`
        changed it: clipping, loading a checkpoint).  Collective."""
        from . import _launch

        assert self._emit is not None
        self.sync_table()
        l1, sm, sp = self._emit_key
        c = self.cache
        whole = torch.zeros(2, dtype=torch.int32, device=self.table.device)
        _launch.quantize_blocks([(self.param.detach(), None)], l1, sm, sp, overflow=whole, out=(c.q16, c.psqt))
        c.stats.view(self.world + 1, 2)[: self.world] = whole  # every rank's part: the whole table's figures
        c.stats[-2:].zero_()
        c.store(self.param, l1, sm, sp, c.q16, c.psqt, c.stats)
        dist.all_reduce(self._token, group=self.group)  # nobody updates (stores into peers) before all have rebuilt

    def sync_table(self) -> None:
        """Every rank's fp32 parameter current again (the owners' rows gathered).  Collective; a no-op while the
        fp32 rows travel with every update."""
        if self.fp32_rows_valid:
            return
        n, w = self.param.shape
        mine = torch.cat([self.table[e0:e1] for e0, e1 in self.ranges])
        self.table.copy_(gather_sharded(mine, self.bounds, w, self.group).reshape(-1))
        self.fp32_rows_valid = True

    def install(self) -> None:
        """Marks the table parameter: the fused backward of every op that reads it (or a table
        derived from it) then writes the gradient into the shared buffer, slice by slice when
        the exchange is sliced."""
        from . import _lib

        self.param._nnue_exchange = self
        if self.sliced:
            _lib.tune("ddp_reduce_ctas", self.reduce_ctas)

    def uninstall(self) -> None:
        """Back to plain gradients: no shared buffer, no slices."""
        from . import _lib

        self.sync_table()
        if self._emit is not None and getattr(self.param, "_nnue_q16_cache", None) is self.cache:
            del self.param._nnue_q16_cache  # the buffers are no longer kept up to date
        if getattr(self.param, "_nnue_exchange", None) is self:
            del self.param._nnue_exchange
        _lib.tune("ddp_reduce_ctas", 0)

    def slice_spec(self):
        """(bounds, events, by_columns) for `nnue_ft_fused_bwd_sliced`, or None when the gradient is taken whole."""
        if not self.sliced:
            return None
        if self.col_bounds is not None:
            return (self.col_bounds, self.slice_events, True)
        return (self.bounds, self.slice_events, False)

    def note_local_reader(self) -> None:
        """Called after a kernel of THIS rank that reads the unsummed gradient buffer has been
        enqueued on the current stream (the factor-row gradient of a folded table): the sliced
        reduce, which runs on its own stream and overwrites this rank's share with rank sums,
        waits for it."""
        if self.sliced:
            self._local_reader.record(torch.cuda.current_stream(self.table.device))
            self._local_reader_pending = True

    def reduce(self) -> torch.Tensor:
        """After every rank's backward has been ENQUEUED: sums this rank's share over the
        ranks.  Returns the squared norm of the whole summed gradient (all-reduced scalar),
        which also fences the phase.  One slice: the caller has put a collective between the
        backward and this call.  Several: a tiny collective per slice, on the second stream,
        tells that every rank has finished that slice."""
        from . import _launch

        if not self.sliced:
            self.ft_sumsq.zero_()
            e0, e1 = self.ranges[0]
            _launch.ddp_reduce_shard(self.grad_ptrs, self.rank, e0, e1, self.ft_sumsq)
        else:
            cur = torch.cuda.current_stream(self.table.device)
            comm = self.comm_stream
            comm.wait_event(self._zeroed)  # ft_sumsq was cleared after its last reader
            if self._local_reader_pending:
                comm.wait_event(self._local_reader)
                self._local_reader_pending = False
            with torch.cuda.stream(comm):
                if self.col_bounds is not None:
                    w = self.param.shape[1]
                    r0, r1 = self.ranges[0][0] // w, self.ranges[0][1] // w
                    for ev, c0, c1 in zip(self.slice_events, self.col_bounds[:-1], self.col_bounds[1:]):
                        comm.wait_event(ev)
                        dist.all_reduce(self._token, group=self.group)
                        _launch.ddp_reduce_block(self.grad_ptrs, self.rank, r0, r1, c0, c1, w, self.ft_sumsq)
                else:
                    for ev, (e0, e1) in zip(self.slice_events, self.ranges):
                        comm.wait_event(ev)                           # this rank has finished the slice ...
                        dist.all_reduce(self._token, group=self.group)  # ... and so has every other rank
                        _launch.ddp_reduce_shard(self.grad_ptrs, self.rank, e0, e1, self.ft_sumsq)
                self._reduced.record(comm)
            cur.wait_event(self._reduced)
        dist.all_reduce(self.ft_sumsq, group=self.group)
        return self.ft_sumsq

    def update(self, hp, grad_scale: torch.Tensor | None) -> None:
        from . import _launch

        emit = self._emit
        if emit is not None:
            self._stats_local.zero_()
        for (e0, e1), o0, o1 in zip(self.ranges, self.state_at[:-1], self.state_at[1:]):
            if e1 == e0:
                continue
            _launch.ddp_update_shard(
                self.table_ptrs, self.rank, e0, e1, self.grad, self.grad_ma[o0:o1],
                None if self.neg_grad_ma is None else self.neg_grad_ma[o0:o1], self.variance_ma[o0:o1],
                None if self.slow is None else self.slow[o0:o1], grad_scale, hp, emit=emit)
        cache = getattr(self.param, "_nnue_q16_cache", None)
        if emit is not None:
            _launch.ddp_publish_stats(emit, self.world, self.rank, self.table.device)
            # every row has been rewritten from its owner's new weights once the fence below has passed
            self.cache.store(self.param, *self._emit_key, self.cache.q16, self.cache.psqt, self.cache.stats)
            if not self._fp32_to_peers and self.world > 1:
                self.fp32_rows_valid = False
        elif cache is not None:
            cache.invalidate()  # the table changed through raw (peer) stores: the forward quantizes it again
        # nobody may read its table before every rank has stored its share into it
        dist.all_reduce(self._token, group=self.group)
        if self.sliced:
            self.ft_sumsq.zero_()
            self._zeroed.record()

    _STATE_KEYS = (("grad_ma", "grad_ma"), ("variance_ma", "variance_ma"), ("neg_grad_ma", "neg_grad_ma"),
                   ("lookahead_params", "slow"))

    def state_dict(self) -> dict:
        """Full-size optimizer state of the table, gathered from the shares: the keys and shapes the
        reference's RangerLite keeps per parameter (model/optimizers/ranger_lite.py:268-278), so a checkpoint
        written under the exchange resumes without it and the other way round.  Collective."""
        self.sync_table()  # the model's state dict is usually taken right beside this one
        out = {"step": self.step}
        n, w = self.param.shape
        for key, attr in self._STATE_KEYS:
            t = getattr(self, attr)
            if t is not None:
                out[key] = gather_sharded(t, self.bounds, w, self.group).view(n, w)
        return out

    def load_state_dict(self, state: dict) -> None:
        """Inverse of `state_dict`: every rank keeps its shares of the full-size tensors (any device;
        missing moments start from zero as in a fresh optimizer, a missing lookahead copy from the table).
        The table itself is the model parameter and is loaded with the model's state dict; call this after it."""
        n, w = self.param.shape
        self.step = int(state.get("step", 0))
        for key, attr in self._STATE_KEYS:
            t = getattr(self, attr)
            if t is None:
                continue
            if key in state and state[key] is not None:
                src = state[key]
                if tuple(src.shape) != (n, w) and src.numel() != n * w:
                    raise ValueError(f"{key}: expected {n} x {w} elements, got {tuple(src.shape)}")
                t.copy_(scatter_full(src.to(device=t.device, dtype=t.dtype), self.bounds, w, self.world, self.rank))
            elif attr == "slow":
                t.copy_(scatter_full(self.table, self.bounds, w, self.world, self.rank))
            else:
                t.zero_()
