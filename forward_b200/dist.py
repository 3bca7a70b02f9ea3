"""Multi-GPU EmbeddingBag: row-sharded tables and table-wise placement.

One process per GPU.  `torch.distributed` carries the rendezvous (IPC handle exchange) and, for
the plain variants, the collective; the fused variants move data with the pooling kernels' own
peer stores (include/fwd_eb_shard.h).

Row shards (one huge table): rank r holds rows [r*rows/G, (r+1)*rows/G); every rank gets the whole
batch, pools what it owns into partial bags, and bag b ends up, summed, on rank b // bags_per_rank.
  exchange="nccl"  partial [B, D] fp32 in local memory, then ncclReduceScatter
  exchange="a2a"   all-to-all of the partial slices, then a fixed-order fold (deterministic)
  exchange="push"  fwd_eb_pipeline_step_rowshard: partial rows go straight into the owner's slots
                   over NVLink from inside the pooling kernel; the flag exchange and the fold run on
                   a side stream beside the next call's pooling
  exchange="compact" fwd_eb_pipeline_step_rowshard_compact (sum / mean; the fastest): a streaming
                   pass keeps this rank's indices as dense sub-bags, the pooling kernel walks those
                   and pushes the partial rows to their owners; flags and fold as "push"
  exchange="stage" fwd_eb_pipeline_step_rowshard_staged: the plain pooling kernel writes the partial
                   bags locally and the copy engines carry each owner's block over NVLink (side
                   stream, beside the next call's pooling); same flags and fold as "push"

Table-wise (many tables): whole tables are assigned to ranks; each rank pools the full batch for
its tables and the pooled outputs are exchanged so that rank g ends with [B/G, T, D].
"""
from __future__ import annotations

import ctypes as C

from . import capi

MAX_PEERS = 16
SHARD_BUFFERS = 16         # FWD_EB_SHARD_BUFFERS: parts of a receive buffer, results in rotation
LAYOUT_ROW_SHARD, LAYOUT_TABLE_WISE = 0, 1
SHARD_TIMEOUT = 1


# ---- host-side geometry (pure Python; covered by CPU tests) ---------------------------------------

def shard_rows(num_rows: int, world: int, rank: int) -> tuple[int, int]:
    """(first logical row, row count) of `rank`: equal windows, the last takes the remainder."""
    per = -(-num_rows // world)
    lo = min(rank * per, num_rows)
    return lo, min(per, num_rows - lo)


def bags_per_rank(num_bags: int, world: int) -> int:
    return max(1, -(-num_bags // world))


def owned_bags(num_bags: int, world: int, rank: int) -> tuple[int, int]:
    per = bags_per_rank(num_bags, world)
    lo = min(rank * per, num_bags)
    return lo, min(per, num_bags - lo)


REPLICATED = -1   # owner value of a table that every rank holds


def place_tables(table_bytes: list[int], world: int, lookups: list[int] | None = None,
                 replicate_below_bytes: int = 0) -> list[int]:
    """Owner rank of every table.  Greedy longest-processing-time on the per-call cost (lookups per
    table; equal when None) with ties broken towards the rank holding fewer bytes, so both time
    and capacity stay balanced.  Deterministic.

    Tables smaller than `replicate_below_bytes` get REPLICATED instead of an owner: every rank
    holds them and pools its own bags only, so they cost no exchange and spread evenly whatever
    the table count (a few hundred MB per table is nothing next to 180 GB of HBM)."""
    n = len(table_bytes)
    cost = list(lookups) if lookups is not None else [1] * n
    owner = [0] * n
    placed = []
    for t in range(n):
        if world > 1 and table_bytes[t] < replicate_below_bytes:
            owner[t] = REPLICATED
        else:
            placed.append(t)
    order = sorted(placed, key=lambda t: (-cost[t], -table_bytes[t], t))
    load = [0] * world
    held = [0] * world
    for t in order:
        r = min(range(world), key=lambda k: (load[k], held[k], k))
        owner[t] = r
        load[r] += cost[t]
        held[r] += table_bytes[t]
    return owner


# ---- C structs -----------------------------------------------------------------------------------

class CompactScratch(C.Structure):
    """Mirror of struct fwd_eb_compact_scratch."""
    _fields_ = [("kept", C.c_void_p), ("kept_weights", C.c_void_p), ("bounds", C.c_void_p),
                ("counts", C.c_void_p)]


class ShardExchange(C.Structure):
    """Mirror of struct fwd_eb_shard_exchange."""
    _fields_ = [
        ("world", C.c_int32), ("rank", C.c_int32), ("bags_per_rank", C.c_int64),
        ("wire_dtype", C.c_int32), ("epoch", C.c_uint32),
        ("peer_slots", C.c_void_p * MAX_PEERS), ("peer_flags", C.c_void_p * MAX_PEERS),
        ("status", C.c_void_p), ("max_spins", C.c_int64),
        ("layout", C.c_int32), ("num_tables", C.c_int32), ("table_index", C.c_int32),
        ("raise_from_push", C.c_int32), ("tickets", C.c_void_p),
        ("stage", C.c_void_p), ("stage_tables", C.c_int32), ("stage_slot", C.c_int32),
    ]


SIGNATURES = {
    "fwd_eb_shard_slots_bytes": (C.c_size_t, [C.c_int32, C.c_int64, C.c_int32, C.c_int32]),
    "fwd_eb_shard_tablewise_bytes": (C.c_size_t, [C.c_int64, C.c_int32, C.c_int32, C.c_int32]),
    "fwd_eb_shard_push": (C.c_int, [C.POINTER(capi.Params), C.POINTER(ShardExchange), C.c_void_p]),
    "fwd_eb_shard_combine": (C.c_int, [C.POINTER(ShardExchange), C.c_int32, C.c_int64, C.c_void_p,
                                       C.c_int32, C.c_void_p]),
    "fwd_eb_shard_combine_div": (C.c_int, [C.POINTER(ShardExchange), C.c_int32, C.c_int64, C.c_void_p,
                                           C.c_void_p, C.c_int32, C.c_void_p]),
    "fwd_eb_pipeline_step_rowshard_compact": (C.c_int, [C.c_void_p, C.POINTER(capi.Params),
                                                        C.POINTER(ShardExchange), C.c_int64,
                                                        C.POINTER(CompactScratch), C.POINTER(C.c_void_p),
                                                        C.c_int32, C.c_void_p, C.POINTER(C.c_int32)]),
    "fwd_eb_shard_stage_bytes": (C.c_size_t, [C.c_int32, C.c_int64, C.c_int32, C.c_int32, C.c_int32]),
    "fwd_eb_shard_ship": (C.c_int, [C.POINTER(ShardExchange), C.c_int32, C.c_int64, C.c_void_p, C.c_void_p]),
    "fwd_eb_shard_wait": (C.c_int, [C.POINTER(ShardExchange), C.c_int32, C.POINTER(C.c_void_p),
                                    C.c_void_p]),
    "fwd_eb_shard_signal": (C.c_int, [C.POINTER(ShardExchange), C.c_void_p]),
    "fwd_eb_shard_send_staged": (C.c_int, [C.POINTER(ShardExchange), C.c_int32, C.c_int64, C.c_void_p,
                                           C.c_void_p]),
    "fwd_eb_pipeline_create": (C.c_int, [C.POINTER(C.c_void_p)]),
    "fwd_eb_pipeline_destroy": (None, [C.c_void_p]),
    "fwd_eb_pipeline_side_stream": (C.c_void_p, [C.c_void_p]),
    "fwd_eb_pipeline_set_lookback": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32]),
    "fwd_eb_pipeline_step_rowshard": (C.c_int, [C.c_void_p, C.POINTER(capi.Params), C.POINTER(ShardExchange),
                                                C.c_int64, C.POINTER(C.c_void_p), C.c_int32, C.c_void_p,
                                                C.POINTER(C.c_int32)]),
    "fwd_eb_pipeline_step_rowshard_staged": (C.c_int, [C.c_void_p, C.POINTER(capi.Params),
                                                       C.POINTER(ShardExchange), C.c_int64,
                                                       C.POINTER(C.c_void_p), C.POINTER(C.c_void_p),
                                                       C.c_int32, C.c_void_p, C.POINTER(C.c_int32)]),
    "fwd_eb_pipeline_step_tablewise": (C.c_int, [C.c_void_p, C.POINTER(C.POINTER(capi.Params)),
                                                 C.POINTER(C.c_int32), C.c_int32,
                                                 C.POINTER(ShardExchange), C.c_int32, C.c_void_p,
                                                 C.POINTER(C.c_void_p)]),
    "fwd_eb_pipeline_step_tablewise_hybrid": (C.c_int, [C.c_void_p, C.POINTER(C.POINTER(capi.Params)),
                                                        C.POINTER(C.c_int32), C.c_int32,
                                                        C.POINTER(C.POINTER(capi.Params)),
                                                        C.POINTER(C.c_int32), C.c_int32,
                                                        C.POINTER(ShardExchange), C.c_int32, C.c_void_p,
                                                        C.POINTER(C.c_void_p)]),
    "fwd_eb_pipeline_set_local_streams": (C.c_int, [C.c_void_p, C.c_int32]),
    "fwd_eb_shard_pool_local": (C.c_int, [C.POINTER(capi.Params), C.POINTER(ShardExchange), C.c_void_p]),
    "fwd_eb_pipeline_sync_result": (C.c_int, [C.c_void_p, C.c_void_p]),
    "fwd_eb_pipeline_drain": (C.c_int, [C.c_void_p]),
    "fwd_eb_ipc_alloc": (C.c_int, [C.c_size_t, C.POINTER(C.c_void_p), C.c_char_p]),
    "fwd_eb_ipc_open": (C.c_int, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "fwd_eb_ipc_close": (C.c_int, [C.c_void_p]),
    "fwd_eb_ipc_free": (C.c_int, [C.c_void_p]),
}

_bound = False


def _lib():
    global _bound
    lib = capi.lib()
    if not _bound:
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _bound = True
    return lib


# ---- peer-mapped buffers ---------------------------------------------------------------------------

class PeerBuffers:
    """This rank's receive slots + flag words, and every peer's view of theirs.

    With a process group the buffers are cudaMalloc'ed here, their CUDA IPC handles all-gathered
    and the peers' buffers opened.  Without one (`local_world` given) all "ranks" live on this GPU
    and the peer pointers are ordinary local pointers — used to test the kernels on one GPU by
    running the ranks' launches one after another."""

    def __init__(self, slot_bytes: int, world: int, rank: int, group=None, local_world=None):
        import torch
        lib = _lib()
        self.world, self.rank = world, rank
        self.slots = [0] * world
        self.flags = [0] * world
        self._opened = []
        self._own = []
        self._keep = []
        if local_world is not None:
            for r in range(world):
                s = torch.zeros(slot_bytes, dtype=torch.uint8, device="cuda")
                f = torch.zeros(MAX_PEERS, dtype=torch.int32, device="cuda")
                self._keep += [s, f]
                self.slots[r], self.flags[r] = s.data_ptr(), f.data_ptr()
            return
        import torch.distributed as dist
        handles = []
        for nbytes in (slot_bytes, MAX_PEERS * 4):
            ptr = C.c_void_p()
            h = C.create_string_buffer(64)
            capi.check(lib.fwd_eb_ipc_alloc(nbytes, C.byref(ptr), h))
            self._own.append(ptr.value)
            handles.append(h.raw)
        gathered = [None] * world
        dist.all_gather_object(gathered, handles, group=group)
        for r in range(world):
            if r == rank:
                self.slots[r], self.flags[r] = self._own
                continue
            got = []
            for raw in gathered[r]:
                ptr = C.c_void_p()
                capi.check(lib.fwd_eb_ipc_open(raw, C.byref(ptr)))
                self._opened.append(ptr.value)
                got.append(ptr.value)
            self.slots[r], self.flags[r] = got
        dist.barrier(group=group)

    def close(self):
        lib = _lib()
        for p in self._opened:
            lib.fwd_eb_ipc_close(C.c_void_p(p))
        for p in self._own:
            lib.fwd_eb_ipc_free(C.c_void_p(p))
        self._opened, self._own, self._keep = [], [], []


def make_exchange(buffers: PeerBuffers, rank: int, per_rank_bags: int, wire_dtype: int,
                  status, *, layout=LAYOUT_ROW_SHARD, num_tables=0, max_spins=0, tickets=None) -> ShardExchange:
    x = ShardExchange()
    x.world, x.rank = buffers.world, rank
    x.bags_per_rank = per_rank_bags
    x.wire_dtype = wire_dtype
    x.epoch = 0
    for r in range(buffers.world):
        x.peer_slots[r] = buffers.slots[r]
        x.peer_flags[r] = buffers.flags[r]
    x.status = status.data_ptr()
    x.max_spins = max_spins
    x.layout = layout
    x.num_tables = num_tables
    # zeroed device words of this rank: with them the pipeline lets the pooling grid raise the flag
    x.tickets = tickets.data_ptr() if tickets is not None else None
    return x


class _StepLanes:
    """Consecutive steps are independent batches.  Queued on one stream, a step's pooling grid starts
    only when the last CTA (and the last peer store) of the step before has finished; on two
    alternating streams it runs beside that tail.  Each step's stream is first put behind the
    caller's current stream (whatever produced the inputs), then the step is queued on it; the
    pipeline keeps flags, waits and folds in call order on its own side stream."""

    def __init__(self, lanes: int, dev):
        import torch
        self.streams = [torch.cuda.Stream(device=dev) for _ in range(lanes)] if lanes > 1 else []
        self.events = [torch.cuda.Event() for _ in self.streams]
        self.calls = 0

    def fork(self):
        """Put every lane behind the current stream's position once (then steps may be issued with
        inputs_ready=True until the current stream produces something they need again)."""
        import torch
        cur = torch.cuda.current_stream()
        for ev, st in zip(self.events, self.streams):
            ev.record(cur)
            st.wait_event(ev)

    def next(self, inputs_ready: bool = False):
        """(lane number, stream) of the next step; the current stream itself with one lane.
        `inputs_ready`: the caller vouches that nothing queued on the current stream produces this
        step's inputs (device-resident batches), which saves the event that orders the lane behind it."""
        import torch
        if not self.streams:
            return 0, torch.cuda.current_stream()
        lane = self.calls % len(self.streams)
        self.calls += 1
        if not inputs_ready:
            self.events[lane].record(torch.cuda.current_stream())
            self.streams[lane].wait_event(self.events[lane])
        return lane, self.streams[lane]


# ---- row-sharded table -------------------------------------------------------------------------------

class RowShardedBag:
    """EmbeddingBag over a table split by rows across the ranks of `group`."""

    def __init__(self, table_local, row_lo: int, *, mode: int, max_bags: int, group=None,
                 exchange: str = "push", wire_dtype: int = capi.F32, padding_idx: int = -1,
                 out_dtype=None, max_indices: int = 0, flag_from_pool: bool = False, ship: bool = False,
                 lookback: tuple[int, int] | None = None, lanes: int = 1):
        import torch
        import torch.distributed as dist
        if mode == capi.MODE_MAX:
            # a shard's partial is {value, position}: only the staged exchange carries it
            if exchange != "stage":
                raise ValueError("row-sharded max needs exchange='stage'")
            wire_dtype = capi.F32_POS
        elif mode not in (capi.MODE_SUM, capi.MODE_MEAN):
            raise ValueError("row-sharded pooling supports sum, mean and max")
        elif wire_dtype == capi.F32_POS:
            raise ValueError("the value + position wire type belongs to max")
        self.table, self.row_lo, self.mode, self.padding_idx = table_local, row_lo, mode, padding_idx
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.exchange = exchange
        self.dim = table_local.shape[1]
        self.max_bags = max_bags
        self.per = bags_per_rank(max_bags, self.world)
        self.out_dtype = out_dtype or torch.float32
        dev = table_local.device
        self.out = torch.empty((self.per, self.dim), dtype=self.out_dtype, device=dev)
        self.side = None
        self.ready = None
        self.piped = exchange in ("push", "stage", "compact")
        if lanes < 1 or lanes > 2:
            raise ValueError("1 or 2 lanes")
        # steps alternate over `lanes` private streams (see _StepLanes); the plain NCCL exchanges stay
        # on the caller's stream
        self._lanes = _StepLanes(lanes if self.piped else 1, dev)
        if exchange == "compact" and max_indices <= 0:
            raise ValueError("exchange='compact' needs max_indices (its scratch is sized up front)")
        if self.piped:
            # The fold runs on the pipeline's side stream so that the next call's pooling does
            # not queue behind this call's flag exchange; results rotate through SHARD_BUFFERS buffers.
            self.outs = [self.out] + [torch.empty_like(self.out) for _ in range(SHARD_BUFFERS - 1)]
            self._out_ptrs = (C.c_void_p * SHARD_BUFFERS)(*[o.data_ptr() for o in self.outs])
            self._pl = C.c_void_p()
            capi.check(_lib().fwd_eb_pipeline_create(C.byref(self._pl)))
            if lanes > 1 and not lookback:
                # with two steps in flight a look-back of two calls is a stall on every wait: measured on
                # two B200s, table-wise step 22.2 us with (6, 2), 19.7 with (8, 8), 20.3 with (12, 4)
                lookback = (8, 8)
            if lookback:
                capi.check(_lib().fwd_eb_pipeline_set_lookback(self._pl, *lookback))
            self.side = torch.cuda.ExternalStream(_lib().fwd_eb_pipeline_side_stream(self._pl), device=dev)
            self._which = C.c_int32(0)
            nbytes = _lib().fwd_eb_shard_slots_bytes(self.world, self.per, self.dim, wire_dtype)
            self.buffers = PeerBuffers(nbytes, self.world, self.rank, group=group)
            self.status = torch.zeros(1, dtype=torch.int32, device=dev)
            # flag_from_pool: the pooling grid raises the flag itself (ticket counter); measured
            # slower than the kernel behind the grid raising it, so off unless asked for
            self.tickets = torch.zeros(SHARD_BUFFERS, dtype=torch.int32, device=dev) if flag_from_pool else None
            self.x = make_exchange(self.buffers, self.rank, self.per, wire_dtype, self.status,
                                   tickets=self.tickets)
            self._stage = None
            if ship and exchange in ("push", "compact"):
                # ship: the pooling kernel stores every partial row locally and a small copy kernel
                # on the side stream sends them on (a pooling warp that stores to a peer has to wait
                # for the acknowledgement before it can exit)
                nbytes = _lib().fwd_eb_shard_stage_bytes(self.world, self.per, 1, self.dim, wire_dtype)
                self._stage = torch.empty(nbytes, dtype=torch.uint8, device=dev)
                self.x.stage = self._stage.data_ptr()
                self.x.stage_tables = 1
            if exchange == "compact":
                # scratch of the window compaction: kept indices, sub-bag bounds, and for a mean
                # the bags' full counts (one part per step in flight: a fold reads them beside later steps)
                nb_all = self.per * self.world
                # kept indices and bounds are read by the step's own pooling only: one set per lane
                self._kept = [torch.empty(max_indices, dtype=torch.int32, device=dev) for _ in range(lanes)]
                self._bounds = [torch.empty((nb_all, 2), dtype=torch.int32, device=dev) for _ in range(lanes)]
                self._counts = torch.zeros((SHARD_BUFFERS, nb_all), dtype=torch.int32, device=dev)
                self._scratch = [CompactScratch(k.data_ptr(), None, b.data_ptr(), self._counts.data_ptr())
                                 for k, b in zip(self._kept, self._bounds)]
                self.max_indices = max_indices
            if exchange == "stage":
                # "stage": the plain pooling kernel writes all partial bags here and the copy
                # engines carry each owner's block over NVLink beside the next call's pooling
                wire = torch.float16 if wire_dtype == capi.F16 else torch.float32
                cols = self.dim * (2 if wire_dtype == capi.F32_POS else 1)   # pairs: 8 bytes a column
                self.stages = [torch.empty((self.per * self.world, cols), dtype=wire, device=dev)
                               for _ in range(SHARD_BUFFERS)]
                self._stage_ptrs = (C.c_void_p * SHARD_BUFFERS)(*[t.data_ptr() for t in self.stages])
        elif exchange in ("nccl", "a2a"):
            self.partial = torch.empty((self.per * self.world, self.dim), dtype=torch.float32,
                                       device=dev)
            if exchange == "a2a":
                self.recv = torch.empty_like(self.partial)
            self.out32 = (self.out if self.out_dtype == torch.float32 else
                          torch.empty((self.per, self.dim), dtype=torch.float32, device=dev))
        else:
            raise ValueError(exchange)

    def params(self, indices, offsets, out):
        return capi.make_params(self.table, indices, offsets, out=out, mode=self.mode,
                                padding_idx=self.padding_idx, row_lo=self.row_lo)

    def prepare(self, indices, offsets):
        """Argument block for forward() on these tensors, built once for inputs that are reused
        (the tensors must stay alive and in place)."""
        num_bags = offsets.numel()
        if num_bags > self.max_bags:
            raise ValueError("batch larger than max_bags")
        if self.exchange == "compact" and indices.numel() > self.max_indices:
            raise ValueError("batch holds more indices than max_indices")
        _, mine = owned_bags(self.per * self.world, self.world, self.rank)
        mine = max(0, min(mine, num_bags - self.rank * self.per))
        out = self.out if self.piped else self.partial
        return (self.params(indices, offsets, out), mine, num_bags)

    def forward(self, indices, offsets=None, pool_events=None, inputs_ready: bool = False):
        """Returns this rank's [bags_owned, dim] slice of the pooled output (a buffer reused
        SHARD_BUFFERS calls later).  `indices` may be a prepare()d argument block.  `pool_events` = (start, end)
        CUDA events recorded around the pooling launch.  `inputs_ready`: see _StepLanes.next."""
        import torch
        import torch.distributed as dist
        p, mine, num_bags = indices if isinstance(indices, tuple) else self.prepare(indices, offsets)
        lane, main = self._lanes.next(inputs_ready)
        stream = main.cuda_stream
        if self.piped:
            if pool_events:
                pool_events[0].record(main)
            if self.exchange == "compact":
                capi.check(_lib().fwd_eb_pipeline_step_rowshard_compact(
                    self._pl, C.byref(p), C.byref(self.x), mine, C.byref(self._scratch[lane]), self._out_ptrs,
                    capi._torch_dtype_code(self.out), C.c_void_p(stream), C.byref(self._which)))
            elif self.exchange == "stage":
                capi.check(_lib().fwd_eb_pipeline_step_rowshard_staged(
                    self._pl, C.byref(p), C.byref(self.x), mine, self._stage_ptrs, self._out_ptrs,
                    capi._torch_dtype_code(self.out), C.c_void_p(stream), C.byref(self._which)))
            else:
                capi.check(_lib().fwd_eb_pipeline_step_rowshard(
                    self._pl, C.byref(p), C.byref(self.x), mine, self._out_ptrs,
                    capi._torch_dtype_code(self.out), C.c_void_p(stream), C.byref(self._which)))
            if pool_events:
                pool_events[1].record(main)   # after the push launch (the fold went to the side stream)
            self.ready = True
            return self.outs[self._which.value][:mine]
        if num_bags < self.per * self.world:
            self.partial[num_bags:].zero_()
        if pool_events:
            pool_events[0].record()
        capi.forward(p, stream)
        if pool_events:
            pool_events[1].record()
        if self.exchange == "nccl":
            dist.reduce_scatter_tensor(self.out32, self.partial, group=self.group)
        else:
            dist.all_to_all_single(self.recv, self.partial, group=self.group)
            capi.combine_partials(self.recv.view(self.world, self.per, self.dim), self.out32)
        if self.out32 is not self.out:
            self.out.copy_(self.out32)
        return self.out[:mine]

    def order_behind_current(self):
        """Steps issued from now on start behind whatever is queued on the current stream (see
        _StepLanes.fork); forward(..., inputs_ready=True) relies on it."""
        self._lanes.fork()

    def sync_result(self):
        """Make the current stream wait until the result of the last forward() is complete.
        (With exchange="push" the fold runs on `self.side`; work queued on that stream needs no
        call.)  Consume a result before the next forward()."""
        if self.piped and self.ready:
            capi.check(_lib().fwd_eb_pipeline_sync_result(self._pl, C.c_void_p(capi.current_stream_ptr())))

    def check_status(self) -> int:
        """Non-zero when a bounded wait gave up (reads one device word; synchronises)."""
        if not self.piped:
            return 0
        capi.check(_lib().fwd_eb_pipeline_drain(self._pl))
        return int(self.status.item())

    def close(self):
        if self.piped:
            _lib().fwd_eb_pipeline_destroy(self._pl)
            self._pl = C.c_void_p()
            self.buffers.close()


def exchange_partials(partial, world: int, per: int, group=None, method: str = "a2a", fold=None):
    """Combine per-rank partial bags [world*per, dim] into this rank's [per, dim] slice.

    "nccl": reduce-scatter (the library picks the order of the additions).  "a2a": all-to-all of
    the slices, then `fold` adds the `world` received slices in source-rank order (default: the
    CUDA fold kernel; CPU tensors need a caller-supplied fold, there is no CPU path here)."""
    import torch
    import torch.distributed as dist
    dim = partial.shape[1]
    if method == "nccl":
        out = torch.empty((per, dim), dtype=partial.dtype, device=partial.device)
        dist.reduce_scatter_tensor(out, partial, group=group)
        return out
    recv = torch.empty_like(partial)
    dist.all_to_all_single(recv, partial, group=group)
    recv = recv.view(world, per, dim)
    if fold is not None:
        return fold(recv)
    if not partial.is_cuda:
        raise RuntimeError("exchange_partials: folding on the host needs an explicit `fold`")
    out = torch.empty((per, dim), dtype=partial.dtype, device=partial.device)
    capi.combine_partials(recv, out)
    return out


class _DeviceView:
    """Lets torch wrap device memory this library allocated (CUDA array interface)."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr,
                                         "data": (ptr, False), "version": 2}


class TableWiseBags:
    """Many tables, each held whole by one rank (owner[t] = that rank) or by every rank (owner[t] =
    REPLICATED: no exchange, each rank pools the bags it owns); pooled outputs land as
    [bags_owned, T, dim].

    exchange="push": each pooling kernel writes its table's column block of every owner's result
    buffer over NVLink (no staging copy, no separate all-to-all kernel).  exchange="nccl": pooled
    [B, T_local, dim] then ncclAllToAll and a local re-layout."""

    def __init__(self, local_tables: dict, owner: list[int], *, dim: int, max_bags: int, group=None,
                 exchange: str = "push", wire_dtype: int = capi.F32, mode: int = capi.MODE_SUM,
                 fixed_len: int = 0, padding_idx: int = -1, flag_from_pool: bool = False,
                 ship: bool = False, lookback: tuple[int, int] | None = None,
                 local_streams: int | None = None, lanes: int = 1):
        import torch
        import torch.distributed as dist
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.owner = list(owner)
        self.num_tables = len(owner)
        self.mine = [t for t, r in enumerate(owner) if r == self.rank]
        self.replicated = [t for t, r in enumerate(owner) if r == REPLICATED]
        if sorted(local_tables) != sorted(self.mine + self.replicated):
            raise ValueError("local_tables must hold exactly the tables this rank owns and the replicated ones")
        if self.replicated and flag_from_pool:
            raise ValueError("replicated tables need the flag raised behind the step's last kernel")
        self.tables = local_tables
        self.dim, self.mode, self.fixed_len, self.padding_idx = dim, mode, fixed_len, padding_idx
        self.per = bags_per_rank(max_bags, self.world)
        self.exchange = exchange
        self.wire_dtype = wire_dtype
        dev = torch.device("cuda", torch.cuda.current_device())
        if lanes < 1 or lanes > 2:
            raise ValueError("1 or 2 lanes")
        self._lanes = _StepLanes(lanes if exchange == "push" else 1, dev)   # see _StepLanes
        self.side = None
        self.ready = None
        self._views = {}
        if exchange == "push":
            self._pl = C.c_void_p()
            capi.check(_lib().fwd_eb_pipeline_create(C.byref(self._pl)))
            if lanes > 1 and not lookback:
                # with two steps in flight a look-back of two calls is a stall on every wait: measured on
                # two B200s, table-wise step 22.2 us with (6, 2), 19.7 with (8, 8), 20.3 with (12, 4)
                lookback = (8, 8)
            if lookback:
                capi.check(_lib().fwd_eb_pipeline_set_lookback(self._pl, *lookback))
            if local_streams is not None:
                capi.check(_lib().fwd_eb_pipeline_set_local_streams(self._pl, local_streams))
            # the flag exchange runs on the pipeline's side stream, beside the next pooling
            self.side = torch.cuda.ExternalStream(_lib().fwd_eb_pipeline_side_stream(self._pl), device=dev)
            nbytes = _lib().fwd_eb_shard_tablewise_bytes(self.per, self.num_tables, dim, wire_dtype)
            self.buffers = PeerBuffers(nbytes, self.world, self.rank, group=group)
            self.status = torch.zeros(1, dtype=torch.int32, device=dev)
            self.tickets = torch.zeros(SHARD_BUFFERS, dtype=torch.int32, device=dev) if flag_from_pool else None
            self.x = make_exchange(self.buffers, self.rank, self.per, wire_dtype, self.status,
                                   layout=LAYOUT_TABLE_WISE, num_tables=self.num_tables,
                                   tickets=self.tickets)
            self._stage = None
            if ship and self.mine:
                nbytes = _lib().fwd_eb_shard_stage_bytes(self.world, self.per, len(self.mine), dim, wire_dtype)
                self._stage = torch.empty(nbytes, dtype=torch.uint8, device=dev)
                self.x.stage = self._stage.data_ptr()
        else:
            tl = max(1, len(self.mine))
            self.send = torch.zeros((self.per * self.world, tl, dim), dtype=torch.float32, device=dev)
            placed = sum(1 for r in owner if r != REPLICATED)
            self.recv = torch.empty((self.per * placed, dim), dtype=torch.float32, device=dev)
            self.result = torch.empty((self.per, self.num_tables, dim), dtype=torch.float32, device=dev)
            self._max_bags = max_bags
            counts = [sum(1 for r in owner if r == src) for src in range(self.world)]
            self.in_splits = [self.per * len(self.mine)] * self.world
            self.out_splits = [self.per * c for c in counts]
            self.by_src = [[t for t, r in enumerate(owner) if r == src] for src in range(self.world)]

    def _own_bags(self, idx, off, w):
        """The part of a whole-batch input that describes the bags this rank owns: (indices,
        offsets, weights, include_last_offset), or None when it owns none of them."""
        lo = self.rank * self.per
        if self.fixed_len > 0:
            L = self.fixed_len
            nb = idx.numel() // L
            hi = min(nb, lo + self.per)
            if hi <= lo:
                return None
            flat = idx.reshape(-1)
            return flat[lo * L:hi * L], None, (w.reshape(-1)[lo * L:hi * L] if w is not None else None), False
        nb = off.numel()
        hi = min(nb, lo + self.per)
        if hi <= lo:
            return None
        # offsets stay absolute: the indices (and weights) are passed whole; a next bag's start, where
        # there is one, closes this rank's last bag
        if hi < nb:
            return idx, off[lo:hi + 1], w, True
        return idx, off[lo:hi], w, False

    def prepare(self, inputs: dict):
        """Argument blocks for forward() on these tensors, built once for inputs that are reused
        (the tensors must stay alive and in place).  inputs[t] describes the WHOLE batch, for the
        replicated tables too."""
        blocks = []
        for k, t in enumerate(self.mine):
            idx, off, w = inputs[t]
            # with "push" `out` is ignored by the entry point; any CUDA tensor satisfies the binding
            out = self.tables[t][:1] if self.exchange == "push" else self.send[:, k, :]
            blocks.append((t, capi.make_params(self.tables[t], idx, off, out=out, mode=self.mode,
                                               fixed_len=self.fixed_len, per_sample_weights=w,
                                               padding_idx=self.padding_idx)))
        n = len(blocks)
        ptrs = (C.POINTER(capi.Params) * max(n, 1))(*[C.pointer(p) for _, p in blocks])
        tabs = (C.c_int32 * max(n, 1))(*[t for t, _ in blocks])
        local, keep = [], []
        for t in self.replicated:
            own = self._own_bags(*inputs[t])
            if own is None:
                continue
            idx, off, w, incl = own
            keep.append(own)
            nb = idx.numel() // self.fixed_len if self.fixed_len > 0 else off.numel() - (1 if incl else 0)
            out = self.tables[t][:1] if self.exchange == "push" else self.result[:nb, t, :]
            local.append((t, capi.make_params(self.tables[t], idx, off, out=out, mode=self.mode,
                                              fixed_len=self.fixed_len, per_sample_weights=w,
                                              padding_idx=self.padding_idx, include_last_offset=incl)))
        m = len(local)
        lptrs = (C.POINTER(capi.Params) * max(m, 1))(*[C.pointer(p) for _, p in local])
        ltabs = (C.c_int32 * max(m, 1))(*[t for t, _ in local])
        return [blocks, ptrs, tabs, n, local, lptrs, ltabs, m, keep]

    def forward(self, inputs, pool_events=None, inputs_ready: bool = False):
        """inputs[t] = (indices, offsets_or_None, weights_or_None) for every table this rank owns,
        or a prepare()d list.  Returns [per, T, dim] (rows past the bags this rank owns are
        unspecified).  `pool_events` = (start, end) CUDA events recorded around the pooling
        launches."""
        import torch
        import torch.distributed as dist
        prepared = inputs if isinstance(inputs, list) else self.prepare(inputs)
        blocks, ptrs, tabs, n, local, lptrs, ltabs, m, _ = prepared
        _, main = self._lanes.next(inputs_ready)
        stream = main.cuda_stream
        if self.exchange == "push":
            if pool_events:
                pool_events[0].record(main)
            res = C.c_void_p()
            capi.check(_lib().fwd_eb_pipeline_step_tablewise_hybrid(
                self._pl, ptrs, tabs, n, lptrs, ltabs, m, C.byref(self.x), self.dim, C.c_void_p(stream),
                C.byref(res)))
            if pool_events:
                pool_events[1].record(main)   # after the push launches (the flag exchange is on the side stream)
            self.ready = True
            view = self._views.get(res.value)
            if view is None:
                typestr = "<f2" if self.wire_dtype == capi.F16 else "<f4"
                view = torch.as_tensor(_DeviceView(res.value, (self.per, self.num_tables, self.dim), typestr),
                                       device="cuda")
                self._views[res.value] = view
            return view
        tl = len(self.mine)
        if pool_events:
            pool_events[0].record()
        for t, p in blocks + local:
            capi.forward(p, stream)
        if pool_events:
            pool_events[1].record()
        send = self.send.view(self.per * self.world * max(1, tl), self.dim) if tl else \
            self.send.view(-1, self.dim)[:0]
        dist.all_to_all_single(self.recv, send, output_split_sizes=self.out_splits,
                               input_split_sizes=self.in_splits if tl else [0] * self.world,
                               group=self.group)
        pos = 0
        for src in range(self.world):
            ts = self.by_src[src]
            if not ts:
                continue
            block = self.recv[pos:pos + self.per * len(ts)].view(self.per, len(ts), self.dim)
            self.result[:, ts, :] = block
            pos += self.per * len(ts)
        return self.result

    def order_behind_current(self):
        """Steps issued from now on start behind whatever is queued on the current stream (see
        _StepLanes.fork); forward(..., inputs_ready=True) relies on it."""
        self._lanes.fork()

    def sync_result(self):
        """Make the current stream wait until the result of the last forward() is complete (the
        flag exchange runs on `self.side`).  Consume a result before the next forward()."""
        if self.exchange == "push" and self.ready:
            capi.check(_lib().fwd_eb_pipeline_sync_result(self._pl, C.c_void_p(capi.current_stream_ptr())))

    def check_status(self) -> int:
        if self.exchange != "push":
            return 0
        capi.check(_lib().fwd_eb_pipeline_drain(self._pl))
        return int(self.status.item())

    def close(self):
        if self.exchange == "push":
            _lib().fwd_eb_pipeline_destroy(self._pl)
            self._pl = C.c_void_p()
            self.buffers.close()
