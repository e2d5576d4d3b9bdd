"""Expert-parallel host logic: which experts (and which slice of the shared expert) a rank holds, and how the ranks'
partial MoE outputs are combined.

Experts are split into contiguous ranges, rank r of N holding [r * E / N, (r + 1) * E / N) (the reference model's
`n_local_experts` split, model.py:869-872).  The router and every dense/attention weight are replicated, so all ranks
see the same ids and weights; the shared expert's intermediate rows are split N ways as well, so each rank's MoE kernels
produce a partial y whose sum over ranks is the layer's output (model.py:903-904).

Two combines:
  * `EpComm` + `encode_combine`: the MoE down kernel stores its partial into every rank's exchange buffer over NVLink
    peer memory and a small kernel adds the slots (no collective library on the path);
  * `combine_routed`: one all-reduce of the partial (the baseline; works under any torch.distributed backend).
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist


def expert_range(n_experts: int, world: int, rank: int) -> tuple[int, int]:
    """[lo, hi) of the experts resident on `rank`."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("rank %d outside a world of %d" % (rank, world))
    if n_experts % world:
        raise ValueError("%d experts do not split evenly over %d ranks" % (n_experts, world))
    per = n_experts // world
    return rank * per, (rank + 1) * per


def shared_range(inter: int, world: int, rank: int, granule: int = 256) -> tuple[int, int]:
    """[lo, hi) of the shared expert's intermediate rows computed by `rank`: granules of 256 rows (one super-block of
    the down matrix's K dimension) dealt out as evenly as possible, the first ranks taking the remainder; a rank beyond
    the number of granules gets an empty range."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("rank %d outside a world of %d" % (rank, world))
    if inter % granule:
        raise ValueError("inter %d is not a multiple of %d" % (inter, granule))
    g = inter // granule
    base, rem = divmod(g, world)
    lo = rank * base + min(rank, rem)
    hi = lo + base + (1 if rank < rem else 0)
    return lo * granule, hi * granule


def local_slots(ids, lo: int, hi: int) -> list[int]:
    """Positions k of the router's top-k whose expert ids[k] is resident in [lo, hi) (host mirror of the kernels'
    on-GPU resolution; used by tests and byte models)."""
    return [k for k, e in enumerate(ids) if lo <= int(e) < hi]


def combine_routed(y_part: torch.Tensor, group=None) -> torch.Tensor:
    """Sum the ranks' partial outputs in place (one all-reduce of dim floats; 16 KB at dim 4096)."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(y_part, op=dist.ReduceOp.SUM, group=group)
    return y_part


class EpComm:
    """The ranks' exchange buffers as seen from this process.  `EpComm(dim, group)` allocates the local buffer,
    exchanges CUDA IPC handles through the process group (host side, any backend) and maps the peers' buffers.
    `EpComm.local(dim, world)` builds `world` communicators over buffers of ONE device, for running the ranks one after
    the other on a single GPU (tests)."""

    def __init__(self, dim: int, group=None, _bases=None, _rank=0, _owned=None):
        from . import _lib
        self._lib = _lib
        self.dim = dim
        self._imported = []
        if _bases is not None:
            self.world, self.rank, self._owned = len(_bases), _rank, _owned or []
            bases = list(_bases)
        else:
            self.world = dist.get_world_size(group)
            self.rank = dist.get_rank(group)
            if self.world > 8:
                raise ValueError("at most 8 ranks")
            nbytes = _lib.lib.msb_ep_exchange_bytes(dim, self.world)
            p = C.c_void_p()
            _lib.check(_lib.lib.msb_ep_alloc(nbytes, C.byref(p)))
            self._owned = [p.value]
            h = C.create_string_buffer(64)
            _lib.check(_lib.lib.msb_ipc_export(p, h))
            handles = [None] * self.world
            dist.all_gather_object(handles, h.raw, group=group)
            bases = []
            for r in range(self.world):
                if r == self.rank:
                    bases.append(p.value)
                else:
                    q = C.c_void_p()
                    _lib.check(_lib.lib.msb_ipc_import(handles[r], C.byref(q)))
                    self._imported.append(q.value)
                    bases.append(q.value)
            dist.barrier(group=group)
        self.c = _lib.EpCommC()
        self.c.world, self.c.rank = self.world, self.rank
        for r, b in enumerate(bases):
            self.c.base[r] = b

    @classmethod
    def local(cls, dim: int, world: int):
        from . import _lib
        nbytes = _lib.lib.msb_ep_exchange_bytes(dim, world)
        bases = []
        for _ in range(world):
            p = C.c_void_p()
            _lib.check(_lib.lib.msb_ep_alloc(nbytes, C.byref(p)))
            bases.append(p.value)
        return [cls(dim, _bases=bases, _rank=r, _owned=bases if r == 0 else []) for r in range(world)]

    def close(self):
        for q in self._imported:
            self._lib.lib.msb_ipc_release(q)
        for p in self._owned:
            self._lib.lib.msb_ep_free(p)
        self._imported, self._owned = [], []


def encode_combine(e, comm: EpComm, h: torch.Tensor):
    """h += sum over ranks of the partial outputs that the ranks' MoE down launches stored for this exchange."""
    comm._lib.check(comm._lib.lib.msb_ep_combine(C.byref(comm.c), h.data_ptr(), h.numel(), e.handle))


class HostExchange:
    """The exchange protocol of the peer combine, on the host: what `moe_down_kernel`'s epilogue and `ep_combine_kernel`
    do with peer stores and arrival counters, restated over a torch.distributed key-value store so that the protocol (epochs,
    double-buffered slots, rank-ordered sum, BOUNDED wait with a status instead of a hang) can be exercised by CPU ranks.

    publish(partial): this rank's partial of the current epoch becomes visible to every rank (slot write + arrival mark).
    combine(h, timeout_s): wait -- at most timeout_s -- for every rank's arrival in the current epoch, add the partials to h in
    rank order and advance the epoch.  Returns 0, or STATUS_PEER_WAIT (3, the device status word's value for the same
    event) with h untouched when a rank's contribution did not arrive in time; the epoch does not advance then."""

    STATUS_PEER_WAIT = 3

    def __init__(self, store, world: int, rank: int, prefix: str = "msb_ep"):
        self.store, self.world, self.rank, self.prefix = store, world, rank, prefix
        self.epoch = 0

    def _key(self, epoch, rank):
        # two buffers, by epoch parity: a rank may publish epoch e + 1 while a slower rank still reads epoch e
        return "%s/%d/%d" % (self.prefix, epoch & 1, rank)

    def publish(self, partial: torch.Tensor):
        import io
        buf = io.BytesIO()
        torch.save((self.epoch + 1, partial.detach().cpu().to(torch.float32)), buf)
        self.store.set(self._key(self.epoch, self.rank), buf.getvalue())

    def combine(self, h: torch.Tensor, timeout_s: float = 1.0) -> int:
        import io
        import time
        deadline = time.monotonic() + timeout_s
        parts = []
        for r in range(self.world):                       # fixed rank order, as the kernel sums
            while True:
                got = None
                try:
                    if self.store.check([self._key(self.epoch, r)]):
                        flag, part = torch.load(io.BytesIO(self.store.get(self._key(self.epoch, r))))
                        if flag == self.epoch + 1:        # the flag carries the epoch: a stale slot does not count
                            got = part
                except Exception:
                    got = None
                if got is not None:
                    parts.append(got)
                    break
                if time.monotonic() >= deadline:
                    return self.STATUS_PEER_WAIT
                time.sleep(0.002)
        for part in parts:
            h += part.to(h.dtype)
        self.epoch += 1
        return 0
