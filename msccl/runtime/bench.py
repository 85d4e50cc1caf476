"""``msccl run`` / ``msccl bench``: execute registered plans (or one XML file) with the native executor
and print one JSON row per size: {collective, algo, nranks, bytes, time_us (max over ranks), algbw, busbw}.

Run under torchrun with one process per GPU, e.g.
``torchrun --nproc-per-node 8 --master-addr 127.0.0.1 -m msccl bench --collective allreduce --nccl``.
"""
import json
import os

import torch

from msccl.utils.sizes import parse_size

_DTYPES = {'bf16': torch.bfloat16, 'fp16': torch.float16, 'fp32': torch.float32}


def _bus_factor(collective, n):
    if n <= 1:
        return 1.0
    return 2.0 * (n - 1) / n if collective == 'allreduce' else (n - 1) / n


def _timed(fn, iters, dist):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) / iters], device='cuda', dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _setup(args, collectives, hi):
    import torch.distributed as dist
    import msccl
    from msccl.runtime import Communicator, Executor
    from msccl.xml import load_xml_file
    if 'RANK' not in os.environ:
        raise SystemExit('msccl run/bench needs one process per GPU: launch it with torchrun '
                         '(--nproc-per-node N --master-addr 127.0.0.1 -m msccl ...)')
    local = int(os.environ.get('LOCAL_RANK', '0'))
    torch.cuda.set_device(local)
    dist.init_process_group('nccl', device_id=torch.device('cuda', local))
    rank, n = dist.get_rank(), dist.get_world_size()
    comm = Communicator.from_process_group(arena_bytes=2 * hi + (96 << 20))
    comm.symmetric_empty(2 * hi + (8 << 20), torch.uint8)      # the two message regions below; what follows is free for plans' scratch
    ex = Executor(comm)
    if args.xml is not None:
        ex.register(load_xml_file(args.xml))
    else:
        machine = 'b200' if n == 8 else f'b200x{n}'
        if rank == 0:
            msccl.init(machine, 1, *[(c, (0, None)) for c in collectives])
            path = [os.environ.get('MSCCL_CONFIG')]
        else:
            path = [None]
        dist.broadcast_object_list(path, src=0)
        if path[0]:
            ex.load_plan_table(path[0])
    return dist, comm, ex, rank, n


_NCCL_TIMES = {}


def _one_size(dist, comm, ex, rank, n, coll, mode, size, dtype, check, nccl, check_only=False):
    """One row (dict) for ``coll`` at ``size`` bytes, or None if nothing can run it.  ``mode``: auto / oneshot / twoshot /
    direct (native kernels), xml (registered plan on ordinary tensors: every tile crosses a FIFO), xmlsym (registered
    plan on tensors from the symmetric arena: stores into the receivers' buffers where the program allows)."""
    esize = torch.empty((), dtype=dtype).element_size()
    unit = n * 16
    registered = mode == 'xmlsym'
    if registered:
        mode = 'xml'
    if mode == 'xml':
        # every chunk of a plan must be a whole number of 16-byte vectors
        probe = ex.select(coll, size if coll != 'allgather' else size // n)
        if probe is not None:
            unit = n * (16 // esize) * max(max(g.i_chunks, g.o_chunks, 1) for g in probe.algo.gpus)
    numel = size // esize // unit * unit
    if numel == 0:
        return None
    nbytes = numel * esize
    gen = torch.Generator(device='cuda').manual_seed(1 + rank)
    plan = None
    if coll == 'allreduce':
        sym = comm.tensor_at(comm.rank, comm.off_arena, numel, dtype)
        src = torch.randn(numel, device='cuda', generator=gen).to(dtype)
        if mode == 'xml':
            work = sym if registered else src.clone()
            fn = lambda: ex.all_reduce(work, algorithm='xml')                          # noqa: E731
            if ex.select('allreduce', nbytes) is None:
                return None
        else:
            fn = lambda: ex.all_reduce(sym, algorithm=mode)                            # noqa: E731
        ref_fn = lambda t: dist.all_reduce(t)                                          # noqa: E731
        algo = mode if mode != 'xml' else ex.select('allreduce', nbytes).algo.name
    else:
        if mode == 'xml':
            plan = ex.select(coll, nbytes if coll != 'allgather' else nbytes // n)
            if plan is None:
                return None
        algo = plan.algo.name if plan is not None else mode
        sym = comm.tensor_at(comm.rank, comm.off_arena, numel, dtype)       # symmetric side of the direct kernels
        if coll == 'allgather':
            src = torch.randn(numel // n, device='cuda', generator=gen).to(dtype)
            out = torch.empty(numel, device='cuda', dtype=dtype)
            ref_fn = lambda t: dist.all_gather_into_tensor(out, t)                    # noqa: E731
            direct = lambda: ex.all_gather(sym, src, algorithm=mode)              # noqa: E731
        elif coll == 'reduce_scatter':
            src = torch.randn(numel, device='cuda', generator=gen).to(dtype)
            out = torch.empty(numel // n, device='cuda', dtype=dtype)
            ref_fn = lambda t: dist.reduce_scatter_tensor(out, t)                     # noqa: E731
            sym.copy_(src)
            direct = lambda: ex.reduce_scatter(mine, sym, algorithm=mode)         # noqa: E731
        else:
            src = torch.randn(numel, device='cuda', generator=gen).to(dtype)
            out = torch.empty(numel, device='cuda', dtype=dtype)
            ref_fn = lambda t: dist.all_to_all_single(out, t)                         # noqa: E731
            direct = lambda: ex.all_to_all(sym, src, algorithm=mode)              # noqa: E731
        mine = torch.empty_like(out)
        if plan is not None and registered:
            # output (and for reduce-scatter the input) inside the arena, at the same offset on every rank
            second = comm.off_arena + ((comm.arena_bytes - (96 << 20)) // 2 + (4 << 20)) // 256 * 256
            if coll == 'reduce_scatter':
                sym.copy_(src)
                src_run, mine = sym, comm.tensor_at(comm.rank, second, out.numel(), dtype)
            else:
                src_run, mine = src, comm.tensor_at(comm.rank, second, out.numel(), dtype)
            fn = lambda: ex.run(plan, src_run, mine)                                   # noqa: E731
        elif plan is not None:
            fn = lambda: ex.run(plan, src, mine)                                       # noqa: E731
        else:
            fn = direct
    row = {'collective': coll, 'algo': algo, 'nranks': n, 'bytes': nbytes, 'memory': 'symmetric' if (registered or mode != 'xml') else 'ordinary'}
    if check:
        if coll == 'allreduce':
            if mode == 'xml':
                work.copy_(src)
                got = work
            else:
                sym.copy_(src)
                got = sym
            fn()
            want = src.clone()
            ref_fn(want)
        else:
            fn()
            ref_fn(src)
            got, want = (mine if plan is not None or coll == 'reduce_scatter' else sym), out
        ex.check()
        # NCCL sums in another order (and with other intermediate precision): allow one rounding per rank
        eps = 2.0 ** -8 if dtype == torch.bfloat16 else (2.0 ** -11 if dtype == torch.float16 else 2.0 ** -23)
        tol = max(3e-2, n * eps) if coll in ('allreduce', 'reduce_scatter') else 0.0
        ok = torch.allclose(got.float(), want.float(), rtol=tol, atol=tol)
        verdict = torch.tensor([1 if ok else 0], device='cuda', dtype=torch.int32)
        dist.all_reduce(verdict, op=dist.ReduceOp.MIN)        # every rank must take the same branch below
        row['matches_nccl'] = bool(verdict.item())
        if not row['matches_nccl'] or check_only:
            return row
    iters = 50 if nbytes <= (1 << 22) else 10
    ms = _timed(fn, iters, dist)
    ex.check()
    if plan is None and mode == 'auto' and ex.last_algorithm:
        row['algo'] = ex.last_algorithm                      # what the size-based dispatch picked
    row.update({'time_us': round(ms * 1e3, 2), 'algbw_gbs': round(nbytes / ms / 1e6, 2),
                'busbw_gbs': round(nbytes * _bus_factor(coll, n) / ms / 1e6, 2)})
    if mode == 'xml':
        row['direct_mask'] = ex.last_direct_mask
    if nccl:
        if (coll, nbytes) not in _NCCL_TIMES:
            t = src.clone()
            _NCCL_TIMES[(coll, nbytes)] = _timed(lambda: ref_fn(t), iters, dist)
        nccl_ms = _NCCL_TIMES[(coll, nbytes)]
        row['nccl_time_us'] = round(nccl_ms * 1e3, 2)
        row['nccl_busbw_gbs'] = round(nbytes * _bus_factor(coll, n) / nccl_ms / 1e6, 2)
    return row


def _sizes(lo, hi):
    size = lo
    while size <= hi:
        yield size
        size *= 4


def main_from_args(args, check=False):
    dtype = _DTYPES[args.dtype]
    lo, hi = parse_size(args.min_bytes), parse_size(args.max_bytes)
    suite = getattr(args, 'suite', False)
    collectives = ['allreduce', 'allgather', 'alltoall', 'reduce_scatter'] if suite else [args.collective]
    dist, comm, ex, rank, n = _setup(args, collectives, hi)
    for coll in collectives:
        mode = getattr(args, 'algo', 'auto')
        if suite:
            modes = ['auto', 'xml', 'xmlsym']
        elif mode == 'auto' and args.xml is not None:
            modes = ['xml']
        else:
            modes = [mode]
        for m in modes:
            for size in _sizes(lo, hi):
                # the suite verifies each (collective, algorithm) once per size before timing it
                row = _one_size(dist, comm, ex, rank, n, coll, m, size, dtype, check or suite,
                                args.nccl and not check, check_only=check)
                if row is not None and rank == 0:
                    print(json.dumps(row), flush=True)
    if suite and n > 2:
        # launch-latency tuning aid: the one-shot kernel with fixed CTA counts
        for size in (16 << 10, 64 << 10, 256 << 10):
            for ctas in (1, 2, 4, 8, 16):
                os.environ['MSCCL_ONESHOT_CTAS'] = str(ctas)
                t = torch.zeros(size // 2, device='cuda', dtype=torch.bfloat16)
                if size <= comm.ll_max_bytes:
                    ms = _timed(lambda: ex.all_reduce(t, algorithm='oneshot'), 50, dist)
                    if rank == 0:
                        print(json.dumps({'tune': 'oneshot_ctas', 'bytes': size, 'ctas': ctas, 'time_us': round(ms * 1e3, 2)}),
                              flush=True)
        os.environ.pop('MSCCL_ONESHOT_CTAS', None)
    comm.close()
    dist.destroy_process_group()


def run_emulated(args):
    """``msccl run --xml FILE --emulate``: all ranks of one program on the current GPU.  Every size is first checked bit
    for bit against the CPU interpreter (up to 1 Mi elements per chunk; larger sizes are timed only), then timed with
    CUDA events.  ``--trace FILE`` dumps the per-step device time stamps of the last size."""
    from msccl.interp import input_chunks_of, run_algorithm
    from msccl.runtime import Communicator, Executor
    from msccl.xml import load_xml_file
    if args.xml is None:
        raise SystemExit('--emulate needs --xml FILE')
    algo = load_xml_file(args.xml)
    dtype = _DTYPES[args.dtype]
    esize = torch.empty((), dtype=dtype).element_size()
    lo, hi = parse_size(args.min_bytes), parse_size(args.max_bytes)
    n = algo.ngpus
    comm = Communicator.emulated(n, fifo_bytes=64 << 20)
    direct = not getattr(args, 'no_direct', False)
    try:
        ex = Executor(comm)
        plan = ex.compile(algo)
        chunks_in = max(input_chunks_of(algo, 0), 1)
        for size in _sizes(lo, hi):
            chunk = max(1, size // esize // chunks_in)
            gen = torch.Generator().manual_seed(1)
            host = [torch.randn(input_chunks_of(algo, r) * chunk, generator=gen).to(dtype) for r in range(n)]

            def place():
                ins, outs = {}, {}
                for r in range(n):
                    if algo.inplace and algo.coll == 'allgather':
                        full = torch.zeros(algo.gpus[r].o_chunks * chunk, dtype=dtype)
                        per = input_chunks_of(algo, r) * chunk
                        full[r * per:(r + 1) * per] = host[r]
                        ins[r] = full.cuda()
                    else:
                        ins[r] = host[r].cuda()
                        if algo.gpus[r].o_chunks > 0 and not algo.inplace:
                            outs[r] = torch.zeros(algo.gpus[r].o_chunks * chunk, dtype=dtype, device='cuda')
                return ins, outs

            ins, outs = place()
            got = ex.run(plan, ins, outs, direct=direct)
            ex.check()
            row = {'algo': algo.name, 'protocol': algo.proto, 'nranks': n, 'chunk_elems': chunk, 'bytes': chunk * chunks_in * esize,
                   'direct_stores': bool(ex.last_direct_mask), 'threadblocks': plan.grid}
            if chunk <= (1 << 20):
                want = run_algorithm(algo, host, chunk, dtype=dtype)
                row['bit_exact'] = all(torch.equal(got[r].cpu()[:want[r].numel()].view(torch.uint8),
                                                   want[r][:got[r].numel()].view(torch.uint8)) for r in range(n))
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            for _ in range(3):
                ex.run(plan, ins, outs, direct=direct)
            torch.cuda.synchronize()
            start.record()
            for _ in range(args.iters):
                ex.run(plan, ins, outs, direct=direct)
            stop.record()
            torch.cuda.synchronize()
            ex.check()
            row['time_us'] = round(start.elapsed_time(stop) / args.iters * 1e3, 2)
            print(json.dumps(row), flush=True)
        if args.trace is not None:
            ex.run(plan, ins, outs, direct=direct, trace=True)
            ex.check()
            from msccl.runtime import trace as step_trace
            rows = ex.last_trace()
            step_trace.write(rows, args.trace, algo.name)
            print(json.dumps({'trace': str(args.trace), 'per_step_type': step_trace.summarize(rows)}), flush=True)
    finally:
        comm.close()
