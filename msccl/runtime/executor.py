"""Executor: runs MSCCL-IR programs and the direct kernels on a ``Communicator``.

``Executor.run(plan, ...)`` launches the interpreter kernel for one compiled program (a program made of
in-switch steps, ``msccl.language.ext_nvls``, goes to the native multimem kernel instead).
``Executor.all_reduce / all_gather / reduce_scatter / all_to_all`` dispatch by size and placement:

* blocks <= ``comm.ll_max_bytes``            -> one-shot LL kernel: flag-in-data packets, no barrier, any
                                               device memory (all four collectives);
* tensor inside the symmetric arena          -> all-reduce / reduce-scatter: two-shot (NVLS multimem when the
                                               heap is bound to a multicast object, peer loads in rank order
                                               otherwise); all-gather / all-to-all: stores straight into the
                                               peers' output between two barriers;
* otherwise                                  -> the interpreter with the program registered for that size (the
                                               ``<msccl_algos>`` table ``msccl.init`` writes, reference
                                               ``msccl/autosynth/__init__.py:75-94``).

As with any collective library, every rank issues the same collectives in the same order, and calls on one
communicator do not overlap in time (staging slots, FIFOs and barrier counters are shared between them).
``last_algorithm`` tells which path the last call took.
"""
import math
import os

import torch

from msccl.runtime.comm import Communicator
from msccl.runtime.plan import (HostPlan, PlanError, access_width, chunk_geometry, compile_plan, tile_geometry,
                                K_FIFO_SLOTS)
from msccl.xml.loader import AlgoIR, load_plan_table, load_xml

DTYPE_CODES = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
MAX_SLOT_BYTES = 4 << 20


class DevicePlan:
    """A ``HostPlan`` uploaded to the device, bound to one communicator."""

    def __init__(self, comm: Communicator, algo: AlgoIR):
        self.comm = comm
        self.algo = algo
        if algo.ngpus != comm.world:
            raise PlanError(f'program is for {algo.ngpus} GPUs, communicator has {comm.world}')
        from msccl.language.ext_nvls import classify
        from msccl.runtime.plan import fifo_index_tables
        # A program made of in-switch steps (mmar / mmb / mmr between barriers) is not interpreted: it is
        # exactly what one native kernel does, and Executor.run hands it to that kernel.
        self.nvls_kind = classify(algo)
        if self.nvls_kind is not None:
            self.host = None
            self.dev_tbs = self.dev_steps = 0
            self.grid = 0
            self.slot_bytes = 0
            self.scratch = {}
            return
        conns = max((len(t) for t in fifo_index_tables(algo).values()), default=0)
        slot = MAX_SLOT_BYTES if conns == 0 else min(MAX_SLOT_BYTES, comm.fifo_bytes // (conns * K_FIFO_SLOTS))
        self.slot_bytes = slot // 1024 * 1024
        if self.slot_bytes < 1024:
            raise PlanError('FIFO area too small for this program')
        self.host: HostPlan = compile_plan(algo, comm.local_ranks, self.slot_bytes)
        nat = comm.native
        self.dev_tbs = nat.upload(self.host.tb_bytes)
        self.dev_steps = nat.upload(self.host.step_bytes)
        self.grid = self.host.total_tbs()
        self.scratch = {}

    def close(self):
        for p in (self.dev_tbs, self.dev_steps):
            if p:
                self.comm.native.device_free(p)
        self.scratch = {}


class Executor:
    def __init__(self, comm: Communicator):
        self.comm = comm
        self.table = {}            # collective -> [(min_bytes, max_bytes, DevicePlan)]
        self.launches = 0          # kernels launched by this executor (for reporting)
        self._checked_grid = {}
        # Threadblocks of a program wait on one another, so they are launched cooperatively (the driver
        # guarantees co-residency).  MSCCL_EXEC_COOPERATIVE=0 is a diagnostic switch for an otherwise idle GPU.
        self.cooperative = os.environ.get('MSCCL_EXEC_COOPERATIVE', '1') != '0'
        self.last_algorithm = None  # what the last collective call dispatched to
        self._ctx_cache = {}       # emulated mode: buffer pointers of all ranks -> device copy of the rank table
        self.last_direct_mask = 0  # buffers (bit 0 input, 1 output, 2 scratch) the last run() stored into directly
        self._trace = None
        # how the warps of a CTA learn that a step may start: 'poll' shared memory, or at a CTA 'barrier'
        self.wait_mode = 0 if os.environ.get('MSCCL_EXEC_WAIT', 'barrier') == 'poll' else 1
        self._scratch_pool = None  # registered scratch shared by all plans (one process per GPU)
        self._stage = None         # registered staging slices for in-switch programs on ordinary tensors
        self.launches_staged = 0

    # ------------------------------------------------------------------ plans
    def compile(self, algo_or_xml) -> DevicePlan:
        algo = load_xml(algo_or_xml) if isinstance(algo_or_xml, str) else algo_or_xml
        return DevicePlan(self.comm, algo)

    def register(self, algo_or_xml, min_bytes=0, max_bytes=math.inf):
        plan = self.compile(algo_or_xml)
        self.table.setdefault(plan.algo.coll, []).append((min_bytes, max_bytes, plan))
        return plan

    def load_plan_table(self, path=None):
        """Install the plans of an ``<msccl_algos>`` file (default: ``$MSCCL_CONFIG``)."""
        path = path or os.environ.get('MSCCL_CONFIG')
        if not path:
            raise PlanError('no plan table: call msccl.init(...) first or pass a path')
        for entry in load_plan_table(path):
            if entry.algo.ngpus == self.comm.world:
                self.register(entry.algo, entry.min_bytes, entry.max_bytes)
        return self

    def select(self, collective, nbytes):
        for lo, hi, plan in self.table.get(collective, []):
            if lo <= nbytes < hi:
                return plan
        return None

    # ------------------------------------------------------------- interpreter
    def run(self, plan: DevicePlan, inputs, outputs=None, stream=None, direct='auto', trace=False, declared_elems=None):
        """Execute ``plan``.  ``inputs`` / ``outputs`` map every local rank to a contiguous CUDA
        tensor (a bare tensor is accepted when this process runs one rank).  For in-place
        programs ``outputs`` may be omitted.  Returns the output tensors by rank.

        ``direct``: sends whose matching receive is ``r`` / ``rcs`` store straight into the receiver's slot when the
        receiving buffer is mapped on the sender - always in emulation; with one process per GPU when the tensor
        (and, if the program receives into scratch, the plan's scratch) comes from ``Communicator.symmetric_empty``,
        i.e. lies at the same heap offset on every rank.  ``'auto'`` decides per buffer, ``False`` forces the FIFO
        path.  ``trace=True`` records per-step device time stamps, read back with ``last_trace()``.
        ``declared_elems`` (rank -> (input, output, scratch) element counts) overrides the buffer sizes the kernel
        checks every step against (a testing aid for the bounds check)."""
        comm, algo = self.comm, plan.algo
        if torch.is_tensor(inputs):
            inputs = {comm.local_ranks[0]: inputs}
        if torch.is_tensor(outputs):
            outputs = {comm.local_ranks[0]: outputs}
        outputs = outputs or {}
        if plan.nvls_kind is not None:
            return self._run_in_switch(plan, inputs, outputs, stream)
        first = inputs[comm.local_ranks[0]]
        dtype = first.dtype
        if dtype not in DTYPE_CODES:
            raise PlanError(f'unsupported dtype {dtype}')
        esize = first.element_size()
        if algo.inplace and algo.coll == 'allgather':
            # the caller passes the gathered buffer with its own part already in place
            chunk = first.numel() // max(algo.gpus[comm.local_ranks[0]].o_chunks, 1)
        else:
            chunk = chunk_geometry(algo, comm.local_ranks[0], first.numel())
        if direct == 'auto':
            direct = os.environ.get('MSCCL_DIRECT', '1') != '0'
        buffers, sizes, results, tensors = {}, {}, {}, {}
        for r in comm.local_ranks:
            g = algo.gpus[r]
            t_in = inputs[r]
            assert t_in.is_cuda and t_in.is_contiguous() and t_in.dtype == dtype
            used = plan.host.extents[r]
            in_ptr, out_ptr = t_in.data_ptr(), 0
            in_elems, out_elems = t_in.numel(), 0
            out_t = None
            if algo.inplace and algo.coll == 'allgather':
                # the caller's tensor is the gathered buffer; its own part is already in place
                out_t = outputs.get(r, t_in)
                if out_t.numel() != g.o_chunks * chunk:
                    raise PlanError(f'in-place all-gather needs the full {g.o_chunks * chunk}-element buffer')
                in_ptr, out_ptr, results[r] = 0, out_t.data_ptr(), out_t
                in_elems, out_elems = 0, out_t.numel()
            else:
                if t_in.numel() < used['i'] * chunk:
                    raise PlanError(f'rank {r}: input of {t_in.numel()} elements, program reads {used["i"] * chunk}')
                if used['o'] > 0:
                    out_t = outputs.get(r)
                    if out_t is None:
                        out_t = torch.empty(g.o_chunks * chunk, dtype=dtype, device=t_in.device)
                    if out_t.numel() < used['o'] * chunk:
                        raise PlanError(f'rank {r}: output of {out_t.numel()} elements, program writes {used["o"] * chunk}')
                    out_ptr, results[r] = out_t.data_ptr(), out_t
                    out_elems = out_t.numel()
                else:
                    results[r] = t_in
            scratch_ptr, scratch_elems, scratch_t = 0, 0, None
            if used['s'] > 0:
                need = used['s'] * chunk * esize
                scratch_t = plan.scratch.get(r)
                if scratch_t is None or scratch_t.numel() < need:
                    scratch_t = self._new_scratch(plan, r, need, t_in.device, direct)
                    plan.scratch[r] = scratch_t
                scratch_ptr, scratch_elems = scratch_t.data_ptr(), scratch_t.numel() // esize
            for ptr in (in_ptr, out_ptr, scratch_ptr):
                if ptr % esize != 0:
                    raise PlanError('buffers must be aligned to their element size')
            buffers[r] = (in_ptr, out_ptr, scratch_ptr)
            sizes[r] = tuple(declared_elems[r]) if declared_elems else (in_elems, out_elems, scratch_elems)
            tensors[r] = (None if in_ptr == 0 else t_in, out_t, scratch_t)
        width = access_width(chunk, esize, [p for r in comm.local_ranks for p in buffers[r]])
        proto = plan.host.proto
        if proto == 2 and width != 16:
            proto = 1                         # LL128 lines need 16-byte chunks; such calls run on the LL packets
        tile, iterations = tile_geometry(plan.host, chunk, esize, plan.slot_bytes, width, proto)
        stream_h = (stream or torch.cuda.current_stream()).cuda_stream
        nat = comm.native
        key = (DTYPE_CODES[dtype], proto, width)
        if key not in self._checked_grid:
            self._checked_grid[key] = nat.max_coresident_ctas(*key)
        if plan.grid > self._checked_grid[key]:
            raise PlanError(f'{plan.grid} threadblocks cannot be co-resident on this device '
                            f'(limit {self._checked_grid[key]})')
        trace_ptr, trace_steps = 0, 0
        if trace:
            trace_steps = max(1, max(len(tb.steps) for g in algo.gpus for tb in g.tbs))
            self._trace = torch.zeros(plan.grid * trace_steps * 6, dtype=torch.int64, device=first.device)
            self._trace_shape = (plan, trace_steps)
            trace_ptr = self._trace.data_ptr()
        geom = [chunk, tile, plan.slot_bytes, iterations, comm.world, 0, plan.grid, key[0], proto, width]
        if comm.emulated_mode:
            # the per-rank buffer table lives on the device, one copy per distinct set of buffers: a
            # host-to-device copy per launch would queue behind any large input copy in flight
            table = tuple(buffers[r] + sizes[r] for r in comm.local_ranks)
            rankctx = self._ctx_cache.get(table)
            if rankctx is None:
                if len(self._ctx_cache) >= 64:
                    nat.device_free(self._ctx_cache.pop(next(iter(self._ctx_cache))))
                rankctx = self._ctx_cache[table] = nat.upload(comm.rankctx_bytes(buffers, sizes))
            self.last_direct_mask = 7 if direct else 0
            nat.launch(plan.dev_tbs, plan.dev_steps, rankctx, geom, comm.timeout_ns, stream_h, self.cooperative,
                       direct_mask=self.last_direct_mask, trace=trace_ptr, trace_steps=trace_steps, wait_mode=self.wait_mode)
        else:
            r = comm.rank
            sym_off, mask = [-1, -1, -1], 0
            if direct:
                for b, t in enumerate(tensors[r]):
                    off = comm.heap_offset_of(t) if t is not None else None
                    if off is not None:
                        sym_off[b], mask = off, mask | (1 << b)
            self.last_direct_mask = mask
            nat.launch(plan.dev_tbs, plan.dev_steps, comm.dev_rankctx, geom, comm.timeout_ns, stream_h, self.cooperative,
                       bufs=list(buffers[r]), elems=list(sizes[r]), peer_heaps=list(comm.heap_ptrs), sym_off=sym_off,
                       direct_mask=mask, trace=trace_ptr, trace_steps=trace_steps, wait_mode=self.wait_mode)
        self.launches += 1
        return results

    def _new_scratch(self, plan, rank, nbytes, device, direct):
        """Scratch of a plan.  When the program receives into scratch, one registered region of the symmetric arena
        serves all plans of this executor (collectives on one communicator never overlap in time, and every rank
        grows the region with the same sizes in the same order, so the offsets agree); otherwise, or when the
        arena has no room, ordinary memory."""
        comm = self.comm
        wants_symmetric = direct and not comm.emulated_mode and 's' in plan.host.direct_bufs.get(rank, ())
        if wants_symmetric:
            pool = self._scratch_pool
            if pool is None or pool.numel() < nbytes:
                try:
                    pool = self._scratch_pool = comm.symmetric_empty(max(nbytes, 8 << 20), torch.uint8)[0]
                except Exception:      # noqa: BLE001 - arena exhausted: the FIFO path needs no registered scratch
                    pool = None
            if pool is not None:
                return pool[:nbytes]
        return torch.empty(nbytes, dtype=torch.uint8, device=device)

    def last_trace(self):
        """Step trace of the last ``run(..., trace=True)``: one dict per (rank, threadblock, step) with the first start
        and last end (ns of the GPU's global timer, relative to the earliest start) and the total ns spent waiting,
        moving data (up to the barrier that ends the step) and signalling over all iterations."""
        if getattr(self, '_trace', None) is None:
            return []
        plan, steps = self._trace_shape
        raw = self._trace.cpu().view(-1, steps, 6)
        starts = raw[:, :, 0][raw[:, :, 0] > 0]
        origin = int(starts.min()) if starts.numel() else 0
        rows, cta = [], 0
        for r in self.comm.local_ranks:
            for tb in plan.algo.gpus[r].tbs:
                for si, st in enumerate(tb.steps):
                    t0, t1, wait, move, signal, _ = (int(v) for v in raw[cta, si])
                    if t1 or t0:
                        rows.append({'rank': r, 'tb': tb.id, 'step': si, 'type': st.type, 'start_ns': t0 - origin,
                                     'end_ns': t1 - origin, 'wait_ns': wait, 'move_ns': move, 'signal_ns': signal})
                cta += 1
        return rows

    def _run_in_switch(self, plan, inputs, outputs, stream):
        """A program of in-switch steps (``msccl.language.ext_nvls``) on the native kernel of the same shape."""
        comm = self.comm
        if comm.emulated_mode or (not comm.mc_base and plan.nvls_kind != 'allreduce'):
            raise PlanError('in-switch programs need one process per GPU and a communicator with NVLink multicast')
        rank, world = comm.rank, comm.world
        t_in = inputs[rank]
        offset = comm.heap_offset_of(t_in)
        nbytes = t_in.numel() * t_in.element_size()
        if not t_in.is_contiguous() or nbytes % (16 * world) or t_in.dtype not in DTYPE_CODES:
            raise PlanError('in-switch programs need a contiguous tensor whose size is a multiple of 16 bytes per rank')
        if offset is None:
            if plan.nvls_kind != 'allreduce':
                raise PlanError('in-switch all-gather / reduce-scatter programs need tensors from Communicator.symmetric_empty')
            return {rank: self._staged_in_switch_allreduce(t_in, stream)}
        stream_h = (stream or torch.cuda.current_stream()).cuda_stream
        code = DTYPE_CODES[t_in.dtype]
        nat = comm.native
        if plan.nvls_kind == 'allreduce':
            # without a multicast window the same two-shot all-reduce runs on peer loads and stores
            nat.twoshot_allreduce(comm.dev_heap_bases, comm.mc_base, offset, nbytes, code, rank, world, comm.dev_syncs,
                                  comm.timeout_ns, self._twoshot_ctas(nbytes), stream_h,
                                  pipelined=bool(comm.mc_base) and os.environ.get('MSCCL_TWOSHOT_PIPE', '0') == '1')
            result = t_in
        elif plan.nvls_kind == 'allgather':            # in place: the own block already sits at its position
            block = nbytes // world
            nat.push_blocks(t_in.data_ptr() + rank * block, True, comm.dev_heap_bases, comm.mc_base, offset, block, rank,
                            world, comm.dev_syncs, comm.timeout_ns, self._direct_ctas(nbytes), stream_h)
            result = t_in
        else:
            out = outputs.get(rank)
            if out is None:
                out = torch.empty(t_in.numel() // world, dtype=t_in.dtype, device=t_in.device)
            if out.numel() * world != t_in.numel() or not out.is_contiguous() or out.data_ptr() % 16:
                raise PlanError('reduce-scatter output must hold 1/world of the input')
            nat.twoshot_allreduce(comm.dev_heap_bases, comm.mc_base, offset, nbytes, code, rank, world, comm.dev_syncs,
                                  comm.timeout_ns, 8, stream_h, out.data_ptr())
            result = out
        self.launches += 1
        self.last_algorithm = f'in-switch {plan.nvls_kind}'
        return {rank: result}

    def _twoshot_ctas(self, nbytes):
        """CTAs of the two-shot kernel: the in-switch reduction is saturated by a few, peer loads want many in flight."""
        if self.comm.mc_base:
            return 8
        return max(1, min(128, nbytes // (32 << 10) or 1))

    STAGE_SLICE_BYTES = 64 << 20

    def _staged_in_switch_allreduce(self, tensor, stream):
        """The in-switch all-reduce on a tensor that is not registered memory: the tensor passes through two registered
        slices of 64 MB.  A tensor that fits into one slice is copied in, reduced and copied back on the caller's stream.
        Larger ones are cut into slices whose copies run on two side streams, so the copy-in of slice i + 1 and the
        copy-out of slice i - 1 overlap the in-switch kernel of slice i (which keeps 8 SMs busy); a slice is reused only
        after its copy-out, and the kernel's closing barrier means no peer still reads it."""
        comm = self.comm
        world, rank = comm.world, comm.rank
        esize = tensor.element_size()
        nbytes = tensor.numel() * esize
        slice_bytes = self.STAGE_SLICE_BYTES // (16 * world) * (16 * world)
        if self._stage is None:
            buf = comm.symmetric_empty(2 * slice_bytes, torch.uint8)[0]
            self._stage = (buf, comm.heap_offset_of(buf), torch.cuda.Stream(), torch.cuda.Stream(),
                           [torch.cuda.Event(), torch.cuda.Event()])
        buf, base, s_in, s_out, freed = self._stage
        main = stream or torch.cuda.current_stream()
        flat = tensor.view(-1).view(torch.uint8)
        code = DTYPE_CODES[tensor.dtype]
        pipelined = bool(comm.mc_base) and os.environ.get('MSCCL_TWOSHOT_PIPE', '0') == '1'
        if nbytes <= slice_bytes:
            if self.launches_staged:
                main.wait_event(freed[0])                       # an earlier, sliced call may still copy out of slice 0
            stage = buf[:nbytes]
            with torch.cuda.stream(main):
                stage.copy_(flat, non_blocking=True)
                comm.native.twoshot_allreduce(comm.dev_heap_bases, comm.mc_base, base, nbytes, code, rank, world, comm.dev_syncs,
                                              comm.timeout_ns, self._twoshot_ctas(nbytes), main.cuda_stream, pipelined=pipelined)
                flat.copy_(stage, non_blocking=True)
                freed[0].record(main)
            self.launches += 1
            self.launches_staged += 1
            self.last_algorithm = 'in-switch allreduce (staged)'
            return tensor
        start = torch.cuda.Event()
        start.record(main)
        s_in.wait_event(start)                                  # the tensor's producer
        pieces = [(o, min(slice_bytes, nbytes - o)) for o in range(0, nbytes, slice_bytes)]
        for i, (off, size) in enumerate(pieces):
            half = i & 1
            stage = buf[half * slice_bytes: half * slice_bytes + size]
            if i >= 2 or self.launches_staged:
                s_in.wait_event(freed[half])                    # the copy-out that last used this slice
            with torch.cuda.stream(s_in):
                stage.copy_(flat[off:off + size], non_blocking=True)
                loaded = torch.cuda.Event()
                loaded.record(s_in)
            main.wait_event(loaded)
            comm.native.twoshot_allreduce(comm.dev_heap_bases, comm.mc_base, base + half * slice_bytes, size, code, rank, world,
                                          comm.dev_syncs, comm.timeout_ns, self._twoshot_ctas(size), main.cuda_stream,
                                          pipelined=pipelined)
            reduced = torch.cuda.Event()
            reduced.record(main)
            s_out.wait_event(reduced)
            with torch.cuda.stream(s_out):
                flat[off:off + size].copy_(stage, non_blocking=True)
                freed[half].record(s_out)
            self.launches += 1
        for ev in freed[:min(2, len(pieces))]:
            main.wait_event(ev)
        self.launches_staged += 1
        self.last_algorithm = 'in-switch allreduce (staged)'
        return tensor

    # -------------------------------------------------------------- collectives
    def all_reduce(self, tensor, stream=None, algorithm='auto'):
        """In-place sum over all ranks.  ``algorithm``: auto | oneshot | twoshot | xml."""
        comm = self.comm
        if comm.emulated_mode:
            raise PlanError('collective entry points need one process per GPU; use run() with an emulated communicator')
        nbytes = tensor.numel() * tensor.element_size()
        if tensor.dtype not in DTYPE_CODES:
            raise PlanError(f'no reduction kernel for {tensor.dtype} (sums of fp32, bf16 and fp16 only)')
        stream_h = (stream or torch.cuda.current_stream()).cuda_stream
        code = DTYPE_CODES[tensor.dtype]
        if comm.world == 1:
            return tensor
        offset = comm.heap_offset_of(tensor)
        if algorithm == 'auto':
            if nbytes <= comm.ll_max_bytes and nbytes % 16 == 0:
                algorithm = 'oneshot'
            elif offset is not None and nbytes % 16 == 0:
                algorithm = 'twoshot'
            else:
                algorithm = 'xml'
        self.last_algorithm = algorithm
        if algorithm == 'oneshot':
            # one 16-byte vector per thread
            ctas = int(os.environ.get('MSCCL_ONESHOT_CTAS', '0')) or max(1, min(32, -(-nbytes // (16 * 512))))
            comm.native.oneshot_allreduce(tensor.data_ptr(), tensor.data_ptr(), comm.dev_staging, nbytes,
                                          comm.ll_slot_bytes, code, comm.rank, comm.world, comm.sync_ptr(comm.rank),
                                          comm.timeout_ns, ctas, stream_h)
            self.launches += 1
            return tensor
        if algorithm == 'twoshot':
            if offset is None:
                raise PlanError('two-shot all-reduce needs a tensor from Communicator.symmetric_empty')
            use_nvls = bool(comm.mc_base) and os.environ.get('MSCCL_TWOSHOT_NVLS', '1' if comm.world > 2 else '0') == '1'
            # the switch is the bottleneck of the in-switch reduction: a few CTAs saturate it and more
            # only add contention (measured on 8 GPUs); peer loads want many CTAs in flight
            auto_ctas = 8 if use_nvls else max(1, min(128, nbytes // (32 << 10) or 1))
            ctas = int(os.environ.get('MSCCL_TWOSHOT_CTAS', '0')) or auto_ctas
            comm.native.twoshot_allreduce(comm.dev_heap_bases, comm.mc_base if use_nvls else 0, offset, nbytes, code, comm.rank,
                                          comm.world, comm.dev_syncs, comm.timeout_ns, ctas, stream_h,
                                          pipelined=os.environ.get('MSCCL_TWOSHOT_PIPE', '0') == '1')
            self.launches += 1
            return tensor
        plan = self.select('allreduce', nbytes)
        if plan is None:
            raise PlanError(f'no all-reduce plan registered for {nbytes} bytes')
        flat = tensor.view(-1)
        if plan.algo.inplace:
            self.run(plan, flat, stream=stream)
        else:
            out = self.run(plan, flat, stream=stream)[comm.rank]
            flat.copy_(out[:flat.numel()])
        return tensor

    def _run_registered(self, collective, inp, out, stream):
        nbytes = inp.numel() * inp.element_size()
        plan = self.select(collective, nbytes)
        if plan is None:
            raise PlanError(f'no {collective} plan registered for {nbytes} bytes')
        return self.run(plan, inp.view(-1), out.view(-1) if out is not None else None, stream=stream)[self.comm.rank]

    def _oneshot(self, mode, inp, out, block_bytes, stream):
        """One-shot LL kernel on blocks of ``block_bytes`` (0 all-reduce, 1 all-gather, 2 reduce-scatter, 3 all-to-all)."""
        comm = self.comm
        ctas = int(os.environ.get('MSCCL_ONESHOT_CTAS', '0')) or max(1, min(32, -(-block_bytes // (16 * 512))))
        stream_h = (stream or torch.cuda.current_stream()).cuda_stream
        # all-gather and all-to-all only move bits: any element type goes through the fp32 instance of the kernel
        code = DTYPE_CODES[inp.dtype] if mode in (0, 2) else 0
        comm.native.oneshot(inp.data_ptr(), out.data_ptr(), comm.dev_staging, block_bytes, comm.ll_slot_bytes,
                            code, comm.rank, comm.world, comm.sync_ptr(comm.rank), comm.timeout_ns, ctas, mode,
                            stream_h)
        self.launches += 1
        return out

    def _oneshot_ok(self, block_bytes, inp, out, may_alias, sums=False):
        if self.comm.emulated_mode or block_bytes > self.comm.ll_max_bytes or block_bytes % 16:
            return False
        if inp.dtype != out.dtype or (sums and inp.dtype not in DTYPE_CODES):
            return False
        if inp.data_ptr() % 16 or out.data_ptr() % 16 or not (inp.is_contiguous() and out.is_contiguous()):
            return False
        if not may_alias:
            a0, a1 = inp.data_ptr(), inp.data_ptr() + inp.numel() * inp.element_size()
            b0, b1 = out.data_ptr(), out.data_ptr() + out.numel() * out.element_size()
            if a0 < b1 and b0 < a1:
                return False
        return True

    def _direct_ctas(self, moved_bytes, cap=96):
        # one sweep of a CTA is 64 KB (512 threads x 8 vectors); half of that per CTA keeps mid sizes short
        return int(os.environ.get('MSCCL_DIRECT_CTAS', '0')) or max(1, min(cap, moved_bytes // (32 << 10)))

    def all_gather(self, output, input, stream=None, algorithm='auto'):
        """``output[r * len(input):][:len(input)] = input of rank r``.  With ``output`` from
        ``Communicator.symmetric_empty`` every rank stores its block straight into its peers' outputs
        (``direct``); otherwise the registered MSCCL-IR plan runs (``xml``).  ``input`` may be the
        caller's own block of ``output`` (in place)."""
        comm = self.comm
        nbytes = input.numel() * input.element_size()
        offset = None if comm.emulated_mode else comm.heap_offset_of(output)
        if algorithm == 'auto':
            if self._oneshot_ok(nbytes, input, output, may_alias=True) and output.numel() == input.numel() * comm.world:
                algorithm = 'oneshot'  # latency-bound: flag-in-data packets, no barrier, any memory
            elif offset is not None and nbytes % 16 == 0 and input.data_ptr() % 16 == 0:
                algorithm = 'direct'
            else:
                algorithm = 'xml'
        self.last_algorithm = algorithm
        if algorithm == 'oneshot':
            if not self._oneshot_ok(nbytes, input, output, may_alias=True):
                raise PlanError(f'one-shot all-gather: blocks of at most {comm.ll_max_bytes} bytes, 16-byte aligned')
            return self._oneshot(1, input, output, nbytes, stream)
        if algorithm == 'direct':
            if offset is None:
                raise PlanError('the direct all-gather needs an output from Communicator.symmetric_empty')
            if output.numel() != input.numel() * comm.world:
                raise PlanError('all-gather output must hold one input per rank')
            # one multimem.st per vector instead of n - 1 peer stores: measured on 8 GPUs it is as fast as peer
            # stores up to 16 MB in total (28 us at 4 MB, 50 us at 16 MB) and slower above (414 vs 391 us at 256 MB)
            prefer_switch = comm.world > 2 and nbytes * comm.world <= (16 << 20)
            use_nvls = bool(comm.mc_base) and os.environ.get('MSCCL_PUSH_NVLS', '1' if prefer_switch else '0') == '1'
            stream_h = (stream or torch.cuda.current_stream()).cuda_stream
            comm.native.push_blocks(input.data_ptr(), True, comm.dev_heap_bases, comm.mc_base if use_nvls else 0, offset, nbytes,
                                    comm.rank, comm.world, comm.dev_syncs, comm.timeout_ns,
                                    self._direct_ctas(nbytes * comm.world), stream_h)
            self.launches += 1
            return output
        return self._run_registered('allgather', input, output, stream)

    def reduce_scatter(self, output, input, stream=None, algorithm='auto'):
        """``output = sum over ranks of their input[rank * len(output):][:len(output)]``.  With ``input``
        from ``Communicator.symmetric_empty`` every rank reduces its slice straight out of its peers'
        inputs (``direct``: peer loads in rank order, or the in-switch reduction)."""
        comm = self.comm
        nbytes = input.numel() * input.element_size()
        offset = None if comm.emulated_mode else comm.heap_offset_of(input)
        out_bytes = output.numel() * output.element_size()
        if algorithm == 'auto':
            ok = offset is not None and nbytes % (16 * comm.world) == 0 and output.data_ptr() % 16 == 0
            if self._oneshot_ok(out_bytes, input, output, may_alias=False, sums=True) and out_bytes * comm.world == nbytes:
                algorithm = 'oneshot'
            else:
                algorithm = 'direct' if ok else 'xml'
        self.last_algorithm = algorithm
        if algorithm == 'oneshot':
            if not self._oneshot_ok(out_bytes, input, output, may_alias=False, sums=True) or out_bytes * comm.world != nbytes:
                raise PlanError(f'one-shot reduce-scatter: blocks of at most {comm.ll_max_bytes} bytes, no overlap of input and output')
            return self._oneshot(2, input, output, out_bytes, stream)
        if algorithm == 'direct':
            if offset is None:
                raise PlanError('the direct reduce-scatter needs an input from Communicator.symmetric_empty')
            if output.numel() * comm.world != input.numel() or not output.is_contiguous():
                raise PlanError('reduce-scatter output must hold 1/world of the input')
            use_nvls = bool(comm.mc_base) and os.environ.get('MSCCL_TWOSHOT_NVLS', '1' if comm.world > 2 else '0') == '1'
            ctas = int(os.environ.get('MSCCL_DIRECT_CTAS', '0')) or (8 if use_nvls else self._direct_ctas(nbytes, 128))
            stream_h = (stream or torch.cuda.current_stream()).cuda_stream
            comm.native.twoshot_allreduce(comm.dev_heap_bases, comm.mc_base if use_nvls else 0, offset, nbytes,
                                          DTYPE_CODES[input.dtype], comm.rank, comm.world, comm.dev_syncs, comm.timeout_ns,
                                          ctas, stream_h, output.data_ptr())
            self.launches += 1
            return output
        return self._run_registered('reduce_scatter', input, output, stream)

    def all_to_all(self, output, input, stream=None, algorithm='auto'):
        """``output block s = block `rank` of rank s's input`` (equal blocks).  With ``output`` from
        ``Communicator.symmetric_empty`` every rank stores its blocks straight into its peers' outputs."""
        comm = self.comm
        nbytes = input.numel() * input.element_size()
        offset = None if comm.emulated_mode else comm.heap_offset_of(output)
        if algorithm == 'auto':
            ok = offset is not None and nbytes % (16 * comm.world) == 0 and input.data_ptr() % 16 == 0
            if nbytes % comm.world == 0 and self._oneshot_ok(nbytes // comm.world, input, output, may_alias=False) \
                    and output.numel() == input.numel():
                algorithm = 'oneshot'
            else:
                algorithm = 'direct' if ok else 'xml'
        self.last_algorithm = algorithm
        if algorithm == 'oneshot':
            if nbytes % comm.world or not self._oneshot_ok(nbytes // comm.world, input, output, may_alias=False):
                raise PlanError(f'one-shot all-to-all: blocks of at most {comm.ll_max_bytes} bytes, no overlap of input and output')
            return self._oneshot(3, input, output, nbytes // comm.world, stream)
        if algorithm == 'direct':
            if offset is None:
                raise PlanError('the direct all-to-all needs an output from Communicator.symmetric_empty')
            if output.numel() != input.numel() or not input.is_contiguous():
                raise PlanError('all-to-all input and output must have the same size')
            stream_h = (stream or torch.cuda.current_stream()).cuda_stream
            comm.native.push_blocks(input.data_ptr(), False, comm.dev_heap_bases, 0, offset, nbytes // comm.world,
                                    comm.rank, comm.world, comm.dev_syncs, comm.timeout_ns, self._direct_ctas(nbytes),
                                    stream_h)
            self.launches += 1
            return output
        return self._run_registered('alltoall', input, output, stream)

    def check(self):
        self.comm.check()

    def require_peers(self, max_age=None):
        """Raise ``PeerLostError`` before launching anything if a peer has left the job."""
        self.comm.require_peers(max_age)
