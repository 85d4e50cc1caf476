"""Time MSCCLang / synthesised / registered programs through the interpreter kernel against NCCL on the same box.

    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 -m msccl.runtime.bench_programs --set all

Sets (one JSON row per program, memory placement and size; times are CUDA events on the launching stream, max over
ranks; every program is first checked bit for bit against the CPU interpreter on a small message):

  allreduce   bf16 all-reduce, 1 KiB .. 1 GiB: the ring, one-shot, two-shot and in-switch MSCCLang programs
  synth       fp16 all-gather synthesised for the fully connected box (steps / rounds bounds) with 1 - 4 chunks per
              rank, 64 KiB .. 256 MiB per rank
  ndv4        the four all-reduce plans the reference registers for one NDv4 box (reference
              ``msccl/autosynth/ndv4_plans.py:14-32``), each inside its registered size range, 8 GPUs only
  registered  every plan ``msccl.init`` selects for this box (machine type ``b200`` / ``b200x4`` / ``b200x2``) in the
              middle of its size range

``memory``: ``ordinary`` - tensors from the caching allocator, every tile crosses a FIFO; ``symmetric`` - tensors from
the communicator's arena at the same offset on every rank, so sends whose receive is ``r`` / ``rcs`` store into the
receiver's slot.
"""
import argparse
import json
import os

import torch

from msccl.utils.sizes import parse_size


def _bus_factor(coll, n):
    return 2.0 * (n - 1) / n if coll == 'allreduce' else (n - 1) / n


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


def _program(name, coll, body, instances=1, **kw):
    from msccl.language import MSCCLProgram
    from msccl.topologies import fully_connected
    from msccl.xml import load_xml
    prog = MSCCLProgram(name, fully_connected(coll.num_ranks), coll, instances, **kw)
    with prog:
        body()
    return load_xml(prog.generate_xml())


def _allreduce_programs(n):
    from msccl.language import ThreadblockPolicy
    from msccl.language.collectives import AllReduce
    from msccl.language.ext_nvls import allreduce_nvls
    from msccl.programs.allreduce import allreduce_one_shot, allreduce_ring, allreduce_two_shot
    from msccl.xml import load_xml
    manual = ThreadblockPolicy.manual
    copies = {2: 128, 4: 32, 8: 16}.get(n, 8)
    ch = min(n, 4)
    return [
        # (program, smallest and largest message in bytes it is timed on)
        (_program(f'ring_{ch}ch_x{max(copies // ch, 1)}', AllReduce(n, n, True), lambda: allreduce_ring(n, ch), max(copies // ch, 1),
                  threadblock_policy=manual), 64 << 10, 1 << 30),
        (_program('ring_ll128', AllReduce(n, n, True), lambda: allreduce_ring(n, ch), 2, threadblock_policy=manual,
                  protocol='LL128'), 1 << 10, 64 << 20),
        (_program('one_shot_ll', AllReduce(n, 1, True), lambda: allreduce_one_shot(n), 1, threadblock_policy=manual,
                  protocol='LL'), 1 << 10, 4 << 20),
        (_program(f'two_shot_x{copies}', AllReduce(n, n, True), lambda: allreduce_two_shot(n), copies, threadblock_policy=manual),
         64 << 10, 1 << 30),
        (_program('two_shot_ll128', AllReduce(n, n, True), lambda: allreduce_two_shot(n), max(copies // 2, 1),
                  threadblock_policy=manual, protocol='LL128'), 1 << 10, 64 << 20),
        (load_xml(allreduce_nvls(n, 8)), 64 << 10, 1 << 30),
    ]


def _synth_programs(n, instances):
    """All-gather on the fully connected box from the SMT synthesiser: least steps at 1 - 4 chunks per rank."""
    from msccl.collectives import allgather
    from msccl.instance import Instance
    from msccl.ncclize import ncclize
    from msccl.path_encoding import PathEncoding
    from msccl.topologies import fully_connected
    from msccl.xml import load_xml
    out = []
    for chunks in (1, 2, 3, 4):
        # one step; a link carries one chunk per round, so c chunks per rank need c rounds
        algo = PathEncoding(fully_connected(n), allgather(n)).solve(Instance(1, extra_rounds=chunks - 1, chunks=chunks))
        if algo is None:
            continue
        ir = load_xml(ncclize(algo, instances=instances, copy_threadblocks=instances))
        ir.name = f'synth_allgather_{chunks}chunk_x{instances}'
        out.append((ir, 64 << 10, 256 << 20))
    return out


def _bit_exact(ex, comm, plan, dist, dtype, rank, n):
    """The program on a small message against the CPU interpreter (every rank checks its own output)."""
    from msccl.interp import input_chunks_of, run_algorithm
    algo = plan.algo
    if plan.nvls_kind is not None:
        return None
    chunk = 1024
    gen = torch.Generator().manual_seed(3)
    host = [torch.randn(input_chunks_of(algo, r) * chunk, generator=gen).to(dtype) for r in range(n)]
    want = run_algorithm(algo, host, chunk, dtype=dtype)[rank]
    if algo.inplace and algo.coll == 'allgather':
        full = torch.zeros(algo.gpus[rank].o_chunks * chunk, dtype=dtype)
        per = input_chunks_of(algo, rank) * chunk
        full[rank * per:(rank + 1) * per] = host[rank]
        got = ex.run(plan, full.cuda())[rank]
    else:
        got = ex.run(plan, host[rank].cuda())[rank]
    ex.check()
    m = min(got.numel(), want.numel())
    ok = torch.equal(got.cpu()[:m].view(torch.uint8), want[:m].view(torch.uint8))
    flag = torch.tensor([1 if ok else 0], device='cuda', dtype=torch.int32)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    return bool(flag.item())


def _sizes(lo, hi, step=4):
    s = lo
    while s <= hi:
        yield s
        s *= step


def _time_program(ex, comm, dist, plan, coll, dtype, lo, hi, rank, n, nccl_cache, out_rows, set_name, regions):
    esize = torch.empty((), dtype=dtype).element_size()
    algo = plan.algo
    sym_a, sym_b = regions
    chunks_in = max(algo.gpus[0].i_chunks, 1) if not (algo.inplace and coll == 'allgather') else max(algo.gpus[0].o_chunks // n, 1)
    exact = _bit_exact(ex, comm, plan, dist, dtype, rank, n)
    for nbytes in _sizes(lo, hi):
        # per-rank message: the all-reduce buffer, or one rank's all-gather contribution
        unit = chunks_in * (16 // esize) * (n if coll == 'allreduce' else 1)
        numel = max(nbytes // esize // unit, 1) * unit
        size = numel * esize
        iters = 20 if size <= (4 << 20) else 5
        for memory in ('ordinary', 'symmetric'):
            if plan.nvls_kind is not None and memory == 'ordinary' and plan.nvls_kind != 'allreduce':
                continue                     # only the in-switch all-reduce stages tensors that are not registered memory
            if coll == 'allreduce':
                t = sym_a[:size].view(dtype) if memory == 'symmetric' else torch.zeros(numel, dtype=dtype, device='cuda')
                fn = lambda: ex.run(plan, t)                                                 # noqa: E731
                ref = lambda: dist.all_reduce(t)                                              # noqa: E731
                moved = size
            else:
                src = sym_a[:size].view(dtype) if memory == 'symmetric' else torch.zeros(numel, dtype=dtype, device='cuda')
                dst = sym_b[:size * n].view(dtype) if memory == 'symmetric' else torch.zeros(numel * n, dtype=dtype, device='cuda')
                fn = lambda: ex.run(plan, src, dst)                                          # noqa: E731
                ref = lambda: dist.all_gather_into_tensor(dst, src)                           # noqa: E731
                moved = size * n
            ms = _timed(fn, iters, dist)
            ex.check()
            key = (coll, size)
            if key not in nccl_cache:
                nccl_cache[key] = _timed(ref, iters, dist)
            row = {'set': set_name, 'program': algo.name, 'protocol': algo.proto, 'collective': coll, 'nranks': n,
                   'threadblocks': plan.grid, 'memory': memory, 'bytes': moved, 'bit_exact_vs_cpu_interpreter': exact,
                   'direct_mask': ex.last_direct_mask, 'time_us': round(ms * 1e3, 2),
                   'busbw_gbs': round(moved * _bus_factor(coll, n) / ms / 1e6, 2),
                   'nccl_time_us': round(nccl_cache[key] * 1e3, 2),
                   'nccl_busbw_gbs': round(moved * _bus_factor(coll, n) / nccl_cache[key] / 1e6, 2)}
            row['speedup_vs_nccl'] = round(nccl_cache[key] / ms, 2)
            out_rows.append(row)
            if rank == 0:
                print(json.dumps(row), flush=True)


def main(argv=None):
    import torch.distributed as dist
    import msccl
    from msccl.runtime import Communicator, Executor
    from msccl.xml.loader import load_plan_table
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument('--set', default='all', help='all, or a comma-separated subset of allreduce, synth, ndv4, registered')
    ap.add_argument('--max-bytes', default='1GB')
    args = ap.parse_args(argv)
    if 'RANK' not in os.environ:
        raise SystemExit('launch with torchrun (--nproc-per-node N --master-addr 127.0.0.1 -m msccl.runtime.bench_programs)')
    local = int(os.environ.get('LOCAL_RANK', '0'))
    torch.cuda.set_device(local)
    dist.init_process_group('nccl', device_id=torch.device('cuda', local))
    rank, n = dist.get_rank(), dist.get_world_size()
    cap = parse_size(args.max_bytes)
    comm = Communicator.from_process_group(arena_bytes=3 * (1 << 30) + (128 << 20), fifo_bytes=256 << 20)
    ex = Executor(comm)
    sym_a = comm.symmetric_empty(1 << 30, torch.uint8)[0]
    sym_b = comm.symmetric_empty(2 << 30, torch.uint8)[0]
    warm = torch.zeros(1024, device='cuda')
    dist.all_reduce(warm)                       # NCCL is up before any environment variable is touched below
    rows, nccl_cache = [], {}
    known = ['allreduce', 'synth', 'ndv4', 'registered']
    sets = known if args.set == 'all' else [v for v in args.set.split(',') if v]
    if any(v not in known for v in sets):
        raise SystemExit(f'--set takes "all" or a comma-separated subset of {", ".join(known)}')

    if 'allreduce' in sets:
        for algo, lo, hi in _allreduce_programs(n):
            plan = ex.compile(algo)
            _time_program(ex, comm, dist, plan, 'allreduce', torch.bfloat16, lo, min(hi, cap), rank, n, nccl_cache, rows,
                          'allreduce', (sym_a, sym_b))
            plan.close()
    if 'synth' in sets:
        for algo, lo, hi in _synth_programs(n, {2: 16, 4: 8, 8: 4}.get(n, 4)):
            plan = ex.compile(algo)
            _time_program(ex, comm, dist, plan, 'allgather', torch.float16, lo, min(hi, cap, (2 << 30) // n), rank, n, nccl_cache,
                          rows, 'synth', (sym_a, sym_b))
            plan.close()

    def plans_of(machine, requests):
        """The plan table msccl.init writes for ``machine`` (the environment is put back afterwards: the NDv4 branch
        of msccl.init exports NCCL and CUDA variables that are not meant for this box)."""
        saved = dict(os.environ)
        path = [None]
        try:
            if rank == 0:
                msccl.init(machine, 1, *requests)
                path = [os.environ.get('MSCCL_CONFIG')]
        finally:
            os.environ.clear()
            os.environ.update(saved)
        dist.broadcast_object_list(path, src=0)
        return load_plan_table(path[0]) if path[0] else []

    if 'ndv4' in sets and n == 8:
        for entry in plans_of('ndv4', [(msccl.Collective.allreduce, (512, 22806528))]):
            plan = ex.compile(entry.algo)
            lo = max(entry.min_bytes, 1 << 10)
            hi = min(int(entry.max_bytes) if entry.max_bytes != float('inf') else cap, cap)
            _time_program(ex, comm, dist, plan, 'allreduce', torch.bfloat16, lo, hi, rank, n, nccl_cache, rows, 'ndv4',
                          (sym_a, sym_b))
            plan.close()
    if 'registered' in sets and n in (2, 4, 8):
        machine = 'b200' if n == 8 else f'b200x{n}'
        for coll in ('allreduce', 'allgather'):
            for entry in plans_of(machine, [(coll, (0, None))]):
                plan = ex.compile(entry.algo)
                lo = max(entry.min_bytes, 4 << 10)
                hi = min(int(entry.max_bytes) if entry.max_bytes != float('inf') else 256 << 20, cap)
                if coll == 'allgather':
                    lo, hi = max(lo // n, 1 << 10), max(hi // n, 1 << 10)
                _time_program(ex, comm, dist, plan, coll, torch.bfloat16, lo, hi, rank, n, nccl_cache, rows, 'registered',
                              (sym_a, sym_b))
                plan.close()
    if rank == 0:
        slower = [r for r in rows if r['speedup_vs_nccl'] < 1.0]
        print(json.dumps({'summary': True, 'rows': len(rows), 'rows_slower_than_nccl': len(slower),
                          'all_bit_exact': all(r['bit_exact_vs_cpu_interpreter'] is not False for r in rows)}), flush=True)
    comm.close()
    dist.destroy_process_group()


if __name__ == '__main__':
    main()
