"""Communicator: the symmetric heaps of all ranks of one NVSwitch box, mapped into this process.

Heap layout of every rank (identical offsets on all ranks)::

    [ sync page | fused-kernel flag page | LL staging (2 x nranks slots) | FIFO area | arena for symmetric tensors ]

Two ways to build one:

* ``Communicator.emulated(world)`` - all ranks live on the current device of this process; the
  interpreter kernel then runs every rank's threadblocks in one cooperative launch.  Used for
  single-GPU testing of multi-rank programs.
* ``Communicator.from_process_group()`` - one process per GPU under ``torch.distributed``
  (rendezvous, descriptor exchange and barriers only; no data goes through it).  Heaps are CUDA
  VMM allocations shared as file descriptors over Unix sockets, optionally bound to an NVLink
  multicast object for ``multimem`` instructions; cudaIpc is the fallback.

The reference leaves all of this to an external NCCL fork
(msccl/autosynth/__init__.py:96-114 only exports environment variables).
"""
import os
import struct
import uuid

import torch

from msccl.runtime.native import load

SYNC_BYTES = 128 * 1024
_RANKCTX = struct.Struct('<2Q3Q3q')


def _align(v, a):
    return (v + a - 1) // a * a


class CommError(RuntimeError):
    pass


class Communicator:
    def __init__(self):
        self.native = load()
        self.rank = 0
        self.world = 1
        self.device = 0
        self.local_ranks = [0]
        self.emulated_mode = False
        self.heap_ptrs = []          # base address of every rank's heap in this process
        self.heap_bytes = 0
        self.ll_slot_bytes = 0
        self.fifo_bytes = 0
        self.arena_bytes = 0
        self.mc_base = 0             # multicast window (0: none)
        self.group = None
        self.mode = 'emulated'
        self._arena_used = 0
        self._owned = []             # (kind, payload) for teardown
        self._dev_tables = {}
        self.timeout_ns = int(float(os.environ.get('MSCCL_TIMEOUT_S', '20')) * 1e9)

    # ------------------------------------------------------------------ layout
    def _set_layout(self, world, ll_max_bytes, fifo_bytes, arena_bytes):
        self.ll_slot_bytes = _align(2 * ll_max_bytes, 1024)
        self.off_fused = SYNC_BYTES
        self.off_staging = 2 * SYNC_BYTES
        self.off_fifo = _align(self.off_staging + 2 * world * self.ll_slot_bytes, 1 << 16)
        self.fifo_bytes = fifo_bytes
        self.off_arena = _align(self.off_fifo + fifo_bytes, 1 << 21)
        self.arena_bytes = arena_bytes
        self.heap_bytes = self.off_arena + arena_bytes
        assert self.native.layout()['sizeof_SyncPage'] <= SYNC_BYTES

    def sync_ptr(self, r):
        return self.heap_ptrs[r]

    def fused_ptr(self, r):
        return self.heap_ptrs[r] + self.off_fused

    def staging_ptr(self, r):
        return self.heap_ptrs[r] + self.off_staging

    def fifo_ptr(self, r):
        return self.heap_ptrs[r] + self.off_fifo

    def arena_ptr(self, r):
        return self.heap_ptrs[r] + self.off_arena

    @property
    def ll_max_bytes(self):
        return self.ll_slot_bytes // 2

    # ---------------------------------------------------------------- builders
    @classmethod
    def emulated(cls, world, fifo_bytes=32 << 20, arena_bytes=0, ll_max_bytes=64 << 10, device=None):
        """All ``world`` ranks on one device of this process."""
        self = cls()
        self.world = world
        self.local_ranks = list(range(world))
        self.emulated_mode = True
        self.device = torch.cuda.current_device() if device is None else device
        torch.cuda.set_device(self.device)
        self._set_layout(world, ll_max_bytes, fifo_bytes, arena_bytes)
        for _ in range(world):
            ptr = self.native.device_malloc(self.heap_bytes, False)
            self.native.device_memset(ptr, 0, self.off_arena)      # flags and FIFOs (packets carry their flags)
            self.heap_ptrs.append(ptr)
            self._owned.append(('malloc', ptr))
        self._upload_tables()
        return self

    @classmethod
    def from_process_group(cls, group=None, fifo_bytes=256 << 20, arena_bytes=0, ll_max_bytes=None,
                           mode=None, multicast=None):
        """One process per GPU; ``torch.distributed`` must be initialised (any backend)."""
        import torch.distributed as dist
        self = cls()
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.local_ranks = [self.rank]
        self.device = torch.cuda.current_device()
        if ll_max_bytes is None:
            # largest block of the one-shot LL kernels.  Measured: with 8 ranks blocks of 128 KB still beat the
            # barrier-based kernels and NCCL (17 us against 27 us for a 1 MB all-gather), blocks of 512 KB do
            # not (38 us against 28-30 us); with 2 ranks 1 MB blocks do (12.5 us against 17 us).
            # (2 ranks: 2 MB blocks; measured 27 us for the barrier-based kernels on 2 MB blocks against 24 us for NCCL)
            ll_max_bytes = (2 << 20) if self.world == 2 else max(256 << 10, (2 << 20) // self.world)
        self._set_layout(self.world, ll_max_bytes, fifo_bytes, arena_bytes)
        mode = mode or os.environ.get('MSCCL_SYMM', 'auto')
        errors = []
        if mode in ('auto', 'vmm'):
            ok, why = self._try_collectively(self._build_vmm, multicast)
            if ok:
                self.mode = 'vmm'
            else:
                errors.append(f'vmm: {why}')
                if mode == 'vmm':
                    raise CommError('; '.join(errors))
        if self.mode != 'vmm':
            ok, why = self._try_collectively(self._build_ipc, None)
            if not ok:
                raise CommError('; '.join(errors + [f'ipc: {why}']))
            self.mode = 'ipc'
        self._upload_tables()
        self.barrier()
        try:
            from msccl.runtime.liveness import Liveness
            self.liveness = Liveness.from_default_store(group)
        except Exception:      # noqa: BLE001 - a job without a rendezvous store simply has no host-side liveness
            self.liveness = None
        return self

    def require_peers(self, max_age=None):
        """Host-side check before a launch: raises ``PeerLostError`` if a peer announced its departure
        (or, with ``max_age``, stopped reporting).  A store round trip: call it between steps, not per kernel."""
        if getattr(self, 'liveness', None) is not None:
            self.liveness.require_all(max_age)

    def leave(self, reason='left'):
        """Tell the other ranks that this rank stops taking part (between steps, nothing in flight)."""
        if getattr(self, 'liveness', None) is not None:
            self.liveness.leave(reason)

    def _try_collectively(self, fn, arg):
        """Run ``fn`` on every rank; succeed only if all ranks succeeded."""
        import torch.distributed as dist
        try:
            fn(arg)
            mine = None
        except Exception as e:     # noqa: BLE001 - reported to all ranks below
            mine = f'rank {self.rank}: {type(e).__name__}: {e}'
        results = [None] * self.world
        dist.all_gather_object(results, mine, group=self.group)
        bad = [r for r in results if r is not None]
        return (not bad), '; '.join(bad[:2])

    def barrier(self):
        if self.group is not None or (not self.emulated_mode):
            import torch.distributed as dist
            torch.cuda.synchronize()
            dist.barrier(group=self.group)

    def _build_vmm(self, multicast):
        import torch.distributed as dist
        nat = self.native
        want_mc = nat.multicast_supported(self.device) if multicast is None else multicast
        want_mc = want_mc and os.environ.get('MSCCL_NVLS', '1') != '0' and self.world > 1
        flags = [None] * self.world
        dist.all_gather_object(flags, bool(want_mc), group=self.group)
        want_mc = all(flags)
        gran = nat.vmm_granularity(self.device, want_mc, self.world)
        self.heap_bytes = _align(self.heap_bytes, gran)
        mine = nat.vmm_create(self.device, self.heap_bytes, gran)
        self._owned.append(('vmm', mine))
        nat.device_memset(mine['ptr'], 0, self.off_arena)          # flags and FIFOs (packets carry their flags)
        # descriptor exchange over abstract Unix sockets
        token = [uuid.uuid4().hex if self.rank == 0 else None]
        dist.broadcast_object_list(token, src=dist.get_global_rank(self.group, 0) if self.group else 0, group=self.group)
        names = [f'msccl-{token[0]}-{r}' for r in range(self.world)]
        sock = nat.fd_socket_open(names[self.rank])
        try:
            dist.barrier(group=self.group)
            for r in range(self.world):
                if r != self.rank:
                    nat.fd_socket_send(sock, names[r], mine['fd'], self.rank)
            blocks = {self.rank: mine}
            for _ in range(self.world - 1):
                fd, src = nat.fd_socket_recv(sock)
                blocks[src] = nat.vmm_import(self.device, fd, self.heap_bytes, gran)
                self._owned.append(('vmm', blocks[src]))
            self.heap_ptrs = [blocks[r]['ptr'] for r in range(self.world)]
            dist.barrier(group=self.group)
            if want_mc:
                if self.rank == 0:
                    mc, mc_fd = nat.multicast_create(self.world, self.heap_bytes)
                    for r in range(1, self.world):
                        nat.fd_socket_send(sock, names[r], mc_fd, 1000)
                else:
                    mc_fd, tag = nat.fd_socket_recv(sock)
                    assert tag == 1000
                    mc = nat.multicast_import(mc_fd)
                nat.multicast_add_device(mc, self.device)
                dist.barrier(group=self.group)          # every device joined before anyone binds
                nat.multicast_bind(mc, mine['handle'], self.heap_bytes)
                dist.barrier(group=self.group)
                self.mc_base = nat.multicast_map(mc, self.heap_bytes, gran, self.device)
                self._owned.append(('mc', (self.mc_base, self.heap_bytes, mc, self.device)))
        finally:
            nat.fd_socket_close(sock)

    def _build_ipc(self, _unused):
        import torch.distributed as dist
        nat = self.native
        ptr = nat.device_malloc(self.heap_bytes, False)
        nat.device_memset(ptr, 0, self.off_arena)                  # flags and FIFOs (packets carry their flags)
        self._owned.append(('malloc', ptr))
        handles = [None] * self.world
        dist.all_gather_object(handles, nat.ipc_export(ptr), group=self.group)
        self.heap_ptrs = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.heap_ptrs.append(ptr)
            else:
                mapped = nat.ipc_import(h)
                self._owned.append(('ipc', mapped))
                self.heap_ptrs.append(mapped)
        self.mc_base = 0

    # ------------------------------------------------------------ device tables
    def _upload_tables(self):
        nat = self.native
        self.dev_heap_bases = nat.upload(struct.pack(f'<{self.world}Q', *self.heap_ptrs))
        self.dev_syncs = nat.upload(struct.pack(f'<{self.world}Q', *[self.sync_ptr(r) for r in range(self.world)]))
        self.dev_staging = nat.upload(struct.pack(f'<{self.world}Q', *[self.staging_ptr(r) for r in range(self.world)]))
        self.dev_rankctx = nat.upload(self.rankctx_bytes({}))
        for p in (self.dev_heap_bases, self.dev_syncs, self.dev_staging, self.dev_rankctx):
            self._owned.append(('malloc', p))

    def rankctx_bytes(self, buffers, sizes=None):
        """``buffers[rank] = (in_ptr, out_ptr, scratch_ptr)`` for ranks this process runs, ``sizes[rank]`` their
        element counts (the bounds the kernel checks every step against)."""
        out = []
        sizes = sizes or {}
        for r in range(self.world):
            b = buffers.get(r, (0, 0, 0))
            n = sizes.get(r, (0, 0, 0))
            out.append(_RANKCTX.pack(self.sync_ptr(r), self.fifo_ptr(r), b[0], b[1], b[2], n[0], n[1], n[2]))
        return b''.join(out)

    # -------------------------------------------------------- symmetric tensors
    def symmetric_empty(self, numel, dtype):
        """A tensor inside this rank's arena at an offset that is the same on every rank (all
        ranks must call this in the same order with the same sizes)."""
        nbytes = _align(numel * torch.empty((), dtype=dtype).element_size(), 256)
        if self._arena_used + nbytes > self.arena_bytes:
            raise CommError(f'symmetric arena exhausted ({self._arena_used}+{nbytes} > {self.arena_bytes})')
        offset = self.off_arena + self._arena_used
        self._arena_used += nbytes
        return self.tensor_at(self.rank if not self.emulated_mode else 0, offset, numel, dtype), offset

    def tensor_at(self, rank, offset, numel, dtype):
        """View ``numel`` elements of ``rank``'s heap at ``offset`` as a torch tensor (no copy)."""
        esize = torch.empty((), dtype=dtype).element_size()
        holder = _DevicePointer(self.heap_ptrs[rank] + offset, numel * esize)
        return torch.as_tensor(holder, device=f'cuda:{self.device}').view(dtype)

    def heap_offset_of(self, tensor):
        """Offset of ``tensor`` inside this rank's heap, or None if it lives elsewhere."""
        base = self.heap_ptrs[self.rank if not self.emulated_mode else 0]
        ptr = tensor.data_ptr()
        if base + self.off_arena <= ptr and ptr + tensor.numel() * tensor.element_size() <= base + self.heap_bytes:
            return ptr - base
        return None

    # ------------------------------------------------------------------ status
    STATUS_NAMES = {0: 'ok', 1: 'timeout waiting for a free FIFO slot', 2: 'timeout waiting for data',
                    3: 'timeout waiting for another threadblock', 4: 'timeout waiting for the peer to drain',
                    5: 'aborted after another threadblock failed', 6: 'out-of-bounds step', 7: 'timeout in barrier'}

    def check(self):
        """Synchronise and raise if any local rank's kernel reported a failure."""
        torch.cuda.synchronize()
        for r in self.local_ranks:
            st = self.native.read_status(self.sync_ptr(r))
            if st[0] != 0:
                raise ExecutorError(st, self.STATUS_NAMES.get(st[0], '?'))

    def reset_after_failure(self):
        """Zero flags, counters, staging slots and FIFOs of the local ranks (all ranks must do this together).  The
        FIFOs are part of it because the launch epoch restarts: a flag-in-data packet left by an earlier launch
        must not carry a flag that a later launch expects."""
        torch.cuda.synchronize()
        for r in self.local_ranks:
            self.native.device_memset(self.sync_ptr(r), 0, self.off_arena)
        if not self.emulated_mode:
            self.barrier()

    def close(self):
        torch.cuda.synchronize()
        nat = self.native
        for kind, payload in reversed(self._owned):
            try:
                if kind == 'malloc':
                    nat.device_free(payload)
                elif kind == 'ipc':
                    nat.ipc_close(payload)
                elif kind == 'vmm':
                    nat.vmm_release(payload['ptr'], payload['size'], payload['handle'], payload['fd'])
                elif kind == 'mc':
                    nat.multicast_unmap(*payload)
            except Exception:      # noqa: BLE001 - teardown is best effort
                pass
        self._owned = []


class ExecutorError(RuntimeError):
    def __init__(self, status, text):
        self.code, self.rank, self.tb, self.step, self.iteration, self.aux0, self.aux1 = status
        super().__init__(f'executor kernel failed on rank {self.rank}: {text} (tb {self.tb}, step {self.step}, '
                         f'iteration {self.iteration}, peer/dep {self.aux0}, channel/step {self.aux1})')


class _DevicePointer:
    """Minimal __cuda_array_interface__ holder (raw bytes) so torch can wrap foreign device memory."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {'shape': (nbytes,), 'typestr': '|u1', 'data': (ptr, False), 'version': 2}
