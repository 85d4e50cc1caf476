#!/usr/bin/env python
"""Headline benchmark: all-reduce bus bandwidth (bf16) through the msccl executor.

    python bench.py --gpus N --steps K --warmup W            (N>1: launched under torchrun)
    python bench.py --impl reference ...                      (unmodified reference + stock NCCL)

One step = one in-place all-reduce of ``--bytes`` (default 1 GiB, larger than the 126 MB L2, so
no cache flush is needed between steps).  busBW = bytes * 2(n-1)/n / time, time measured with
CUDA events on the launching stream, max over ranks.  With one GPU there is no peer: the step is
then the 8-rank ring all-reduce program executed with all eight ranks emulated on the single
GPU (same interpreter kernel, FIFOs in local HBM) on 256 MiB per emulated rank.

The e2e figure repeats the measurement through the public API including, per step, the
host-to-device copy of the step's input from pinned memory and a device-to-host read of a
checksum of the result.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ('index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,'
             'clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,'
             'clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap')

    def __init__(self, device_index):
        self.device_index = device_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(['nvidia-smi', f'--query-gpu={self.QUERY}', '--format=csv,noheader,nounits',
                                          '-lms', '20', '-i', str(self.device_index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(',')])

    def stop(self):
        if self.proc is None:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['nvidia-smi unavailable']}
        time.sleep(0.15)
        self.proc.terminate()
        self.thread.join(timeout=2)
        clocks, reasons, max_mhz = [], set(), None
        names = ['hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap']
        for row in self.rows:
            if len(row) < 9:
                continue
            try:
                clocks.append(float(row[1]))
                max_mhz = float(row[2])
            except ValueError:
                continue
            for name, cell in zip(names, row[5:9]):
                if cell.lower().startswith('active'):
                    reasons.add(name)
        clocks.sort()
        median = clocks[len(clocks) // 2] if clocks else None
        return {'sm_mhz': median, 'sm_max_mhz': max_mhz, 'reasons': sorted(reasons), 'samples': len(clocks)}


def _dist_setup(n):
    import torch
    import torch.distributed as dist
    local = int(os.environ.get('LOCAL_RANK', '0'))
    torch.cuda.set_device(local)
    if n > 1:
        os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
        dist.init_process_group('nccl', device_id=torch.device('cuda', local))
    return local


def _max_over_ranks(value, n):
    import torch
    import torch.distributed as dist
    if n == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device='cuda')
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _timed(n, steps, warmup, step_fn, sync_fn):
    """W warm-up steps, then exactly K steps between barrier+synchronize; returns ms per step (max over ranks)."""
    import torch
    import torch.distributed as dist
    for _ in range(warmup):
        step_fn()
    sync_fn()
    if n > 1:
        dist.barrier()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        step_fn()
    stop.record()
    torch.cuda.synchronize()
    if n > 1:
        dist.barrier()
    torch.cuda.synchronize()
    return _max_over_ranks(start.elapsed_time(stop) / steps, n)


def bus_factor(n):
    return 2.0 * (n - 1) / n if n > 1 else 1.0


def run_ours(args):
    import torch
    sys.path.insert(0, ROOT)
    n = args.gpus
    local = _dist_setup(n)
    rank = int(os.environ.get('RANK', '0'))
    from msccl.runtime import Communicator, Executor
    dtype = torch.bfloat16
    esize = 2
    sampler = ClockSampler(local)
    config = {'model': 'allreduce (MSCCL-IR executor)', 'dtype_bytes': esize, 'l2_policy': 'inputs larger than L2'}
    if n == 1:
        # eight emulated ranks on one GPU, ring program, 256 MiB per rank
        from msccl.language import MSCCLProgram, ThreadblockPolicy
        from msccl.language.collectives import AllReduce
        from msccl.programs.allreduce import allreduce_ring
        from msccl.topologies import fully_connected
        from msccl.xml import load_xml
        world = 8
        nbytes = min(args.bytes, 256 << 20)
        prog = MSCCLProgram('allreduce_ring', fully_connected(world), AllReduce(world, world, True), 4,
                            threadblock_policy=ThreadblockPolicy.manual)
        with prog:
            allreduce_ring(world, 4)
        comm = Communicator.emulated(world, fifo_bytes=256 << 20)
        ex = Executor(comm)
        plan = ex.compile(load_xml(prog.generate_xml()))
        numel = nbytes // esize
        bufs = {r: torch.randn(numel, device='cuda', dtype=torch.float32).to(dtype) for r in range(world)}
        pinned = torch.randn(numel, dtype=torch.float32).to(dtype).pin_memory()
        result_host = torch.empty(1, dtype=torch.float32).pin_memory()

        def step():
            ex.run(plan, bufs)

        # end to end: the step's input arrives from pinned host memory in slices on a copy stream, and the
        # program runs on slice c while slice c + 1 is still crossing PCIe (same public call, on views)
        copy_stream = torch.cuda.Stream()
        pieces = 2          # measured 1 / 2 / 4 / 8 slices: 9.0 / 8.6 / 9.4 / 11.7 ms per step
        piece = numel // pieces // 4096 * 4096
        bounds = [(c * piece, numel if c == pieces - 1 else (c + 1) * piece) for c in range(pieces)]
        arrived = [torch.cuda.Event() for _ in range(pieces)]

        def e2e_step():
            main = torch.cuda.current_stream()
            with torch.cuda.stream(copy_stream):
                for c, (lo, hi) in enumerate(bounds):
                    bufs[0][lo:hi].copy_(pinned[lo:hi], non_blocking=True)
                    arrived[c].record(copy_stream)
            for c, (lo, hi) in enumerate(bounds):
                main.wait_event(arrived[c])
                ex.run(plan, {r: bufs[r][lo:hi] for r in range(world)})
            result_host.copy_(bufs[0][:4096].float().sum().reshape(1), non_blocking=True)
            main.synchronize()

        factor = bus_factor(world)
        config.update({'parallelism': 'emulated 8 ranks on 1 GPU (ring program, 4 instances)', 'ranks': world,
                       'bytes_per_rank': nbytes, 'global_batch': world * nbytes, 'seq_len': None,
                       'algorithm': 'allreduce_ring via interpreter kernel'})
        kernels_per_step = 1
    else:
        world = n
        nbytes = args.bytes
        comm = Communicator.from_process_group(arena_bytes=nbytes + (8 << 20))
        ex = Executor(comm)
        numel = nbytes // esize
        buf, _ = comm.symmetric_empty(numel, dtype)
        buf.copy_(torch.randn(numel, device='cuda', dtype=torch.float32).to(dtype) * 0.01)
        pinned = (torch.randn(numel, dtype=torch.float32) * 0.01).to(dtype).pin_memory()
        result_host = torch.empty(1, dtype=torch.float32).pin_memory()

        def step():
            ex.all_reduce(buf, algorithm='twoshot')

        copy_stream = torch.cuda.Stream()
        pieces = 8
        piece = numel // pieces // 4096 * 4096
        bounds = [(c * piece, numel if c == pieces - 1 else (c + 1) * piece) for c in range(pieces)]
        arrived = [torch.cuda.Event() for _ in range(pieces)]

        def e2e_step():
            # slices of the input cross PCIe on a copy stream while earlier slices are being reduced
            main = torch.cuda.current_stream()
            with torch.cuda.stream(copy_stream):
                for c, (lo, hi) in enumerate(bounds):
                    buf[lo:hi].copy_(pinned[lo:hi], non_blocking=True)
                    arrived[c].record(copy_stream)
            for c, (lo, hi) in enumerate(bounds):
                main.wait_event(arrived[c])
                ex.all_reduce(buf[lo:hi])
            result_host.copy_(buf[:4096].float().sum().reshape(1), non_blocking=True)
            main.synchronize()

        factor = bus_factor(world)
        config.update({'parallelism': f'{n} ranks, one process per GPU', 'ranks': world, 'bytes_per_rank': nbytes,
                       'global_batch': world * nbytes, 'seq_len': None, 'symmetric_memory': comm.mode,
                       'algorithm': 'two-shot ' + ('NVLS multimem' if comm.mc_base else 'peer load/store')})
        kernels_per_step = 1

    sampler.start()
    launches_before = ex.launches
    ms = _timed(n, args.steps, args.warmup, step, ex.check)
    launches = ex.launches - launches_before - 0
    ex.check()
    clocks = sampler.stop()
    e2e_ms = _timed(n, max(2, args.steps // 4), 1, e2e_step, ex.check)
    ex.check()
    value = nbytes * factor / (ms * 1e-3) / 1e9
    e2e_value = nbytes * factor / (e2e_ms * 1e-3) / 1e9
    sweep = None
    if n > 1 and args.sweep:
        sweep = sweep_ours(ex, comm, n, dtype)
    if rank == 0:
        line = {'metric': 'allreduce_busbw', 'value': round(value, 3), 'unit': 'GB/s', 'n_gpus': n,
                'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': round(ms, 5), 'higher_is_better': True,
                'scaling': 'weak', 'vs_baseline': None, 'dtype': 'bf16', 'data': 'synthetic', 'impl': 'msccl-b200',
                'config': config, 'clocks': clocks,
                'e2e': {'value': round(e2e_value, 3), 'unit': 'GB/s', 'ms_per_step': round(e2e_ms, 5),
                        'h2d_bytes_per_step': nbytes, 'd2h_bytes_per_step': 4,
                        'how': f'input in {pieces} slices on a copy stream, each reduced as soon as it has arrived'},
                'gpu_launches': kernels_per_step * args.steps}
        if sweep:
            line['sweep'] = sweep
        print(json.dumps(line), flush=True)
    comm.close()
    if n > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


def sweep_ours(ex, comm, n, dtype, sizes=None):
    """busBW of the auto-dispatched all-reduce for 1 KiB .. 256 MiB (device-timed, max over ranks)."""
    import torch
    rows = []
    sizes = sizes or [1 << s for s in range(10, 29, 2)]
    for nbytes in sizes:
        numel = nbytes // 2
        t = comm.tensor_at(comm.rank, comm.off_arena, numel, dtype)      # symmetric: every path can take it
        iters = 50 if nbytes <= (1 << 20) else 10
        ms = _timed(n, iters, 5, lambda: ex.all_reduce(t), ex.check)
        rows.append({'bytes': nbytes, 'us': round(ms * 1e3, 2), 'busbw_gbs': round(nbytes * bus_factor(n) / (ms * 1e-3) / 1e9, 2)})
    return rows


def run_reference(args):
    """The reference's public path: ``msccl.init(...)`` followed by ordinary ``torch.distributed``
    calls (reference README.md:20-38).  The reference contains no runtime of its own, so the
    collective itself is executed by the stock NCCL that ships with PyTorch."""
    ref = os.path.join(ROOT, 'baseline', '_ref')
    if not os.path.isdir(os.path.join(ref, 'msccl')):
        print(json.dumps({'impl': 'reference', 'unavailable': 'baseline/_ref is not installed on this machine'}))
        return
    sys.path.insert(0, ref)
    sys.path.insert(0, os.path.join(ROOT, 'baseline', 'shims'))
    import torch
    import torch.distributed as dist
    n = args.gpus
    local = _dist_setup(n)
    rank = int(os.environ.get('RANK', '0'))
    if n == 1 and not dist.is_initialized():
        os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
        os.environ.setdefault('MASTER_PORT', '29517')
        dist.init_process_group('nccl', rank=0, world_size=1, device_id=torch.device('cuda', local))
    import msccl as reference_msccl
    assert reference_msccl.__file__.startswith(ref), 'the reference package must be the one that is imported'
    note = 'msccl.init(auto) returned without selecting a plan (SKU not recognised); stock NCCL runs the collective'
    nbytes = args.bytes if n > 1 else min(args.bytes, 256 << 20)
    try:
        reference_msccl.init('auto', 1, (reference_msccl.Collective.allreduce, nbytes))
    except Exception as e:      # noqa: BLE001 - the reference's auto-detection assumes 8 GPUs
        note = f'msccl.init(auto) raised {type(e).__name__}: {e}; stock NCCL runs the collective'
    dtype = torch.bfloat16
    numel = nbytes // 2
    buf = (torch.randn(numel, device='cuda', dtype=torch.float32) * 0.01).to(dtype)
    pinned = (torch.randn(numel, dtype=torch.float32) * 0.01).to(dtype).pin_memory()
    result_host = torch.empty(1, dtype=torch.float32).pin_memory()
    sampler = ClockSampler(local)

    def step():
        dist.all_reduce(buf)

    def e2e_step():
        buf.copy_(pinned, non_blocking=True)
        dist.all_reduce(buf)
        result_host.copy_(buf[:4096].float().sum().reshape(1), non_blocking=True)
        torch.cuda.current_stream().synchronize()

    sampler.start()
    ms = _timed(n, args.steps, args.warmup, step, torch.cuda.synchronize)
    clocks = sampler.stop()
    e2e_ms = _timed(n, max(2, args.steps // 4), 1, e2e_step, torch.cuda.synchronize)
    factor = bus_factor(n)
    sweep = None
    if n > 1 and args.sweep:
        sweep = []
        for size in [1 << s for s in range(10, 29, 2)]:
            t = torch.zeros(size // 2, device='cuda', dtype=dtype)
            iters = 50 if size <= (1 << 20) else 10
            t_ms = _timed(n, iters, 5, lambda: dist.all_reduce(t), torch.cuda.synchronize)
            sweep.append({'bytes': size, 'us': round(t_ms * 1e3, 2),
                          'busbw_gbs': round(size * factor / (t_ms * 1e-3) / 1e9, 2)})
    if n == 1:
        # One GPU: this repo's arm runs an 8-rank program with all ranks emulated on the GPU.  The reference
        # has no way to do that (its runtime is NCCL, which refuses two ranks on one device), and a 1-rank
        # all-reduce moves no data, so there is no reference number for this configuration.  What the
        # reference's path does with one rank is recorded for information only.
        print(json.dumps({'impl': 'reference', 'unavailable': 'the reference runs collectives through NCCL, which cannot '
                          'place the 8 ranks of this configuration on one GPU; its 1-rank all-reduce is an identity that '
                          'moves no data', 'n_gpus': 1,
                          'one_rank_identity': {'bytes': nbytes, 'ms_per_call': round(ms, 5), 'e2e_ms_per_step': round(e2e_ms, 5),
                                                'note': note}, 'clocks': clocks}), flush=True)
        dist.destroy_process_group()
        return
    if rank == 0:
        line = {'metric': 'allreduce_busbw', 'value': round(nbytes * factor / (ms * 1e-3) / 1e9, 3), 'unit': 'GB/s',
                'n_gpus': n, 'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': round(ms, 5),
                'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': 'bf16',
                'data': 'synthetic', 'impl': 'reference',
                'config': {'model': 'allreduce (reference msccl.init + torch.distributed / stock NCCL)',
                           'bytes_per_rank': nbytes, 'global_batch': n * nbytes, 'seq_len': None,
                           'parallelism': f'{n} ranks', 'note': note, 'nccl': '.'.join(map(str, torch.cuda.nccl.version())),
                           'l2_policy': 'inputs larger than L2'},
                'clocks': clocks,
                'e2e': {'value': round(nbytes * factor / (e2e_ms * 1e-3) / 1e9, 3), 'unit': 'GB/s',
                        'ms_per_step': round(e2e_ms, 5), 'h2d_bytes_per_step': nbytes, 'd2h_bytes_per_step': 4},
                'gpu_launches': 0}
        if sweep:
            line['sweep'] = sweep
        print(json.dumps(line), flush=True)
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=5)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--bytes', type=int, default=1 << 30, help='message size per rank')
    ap.add_argument('--sweep', action='store_true', help='also time 1 KiB .. 256 MiB (reported under "sweep")')
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    world = int(os.environ.get('WORLD_SIZE', '1'))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            # convenience: re-launch under torchrun
            cmd = [sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', f'--nproc-per-node={args.gpus}',
                   '--master-addr', '127.0.0.1', '--master-port', os.environ.get('MASTER_PORT', '29533'),
                   os.path.abspath(__file__)] + sys.argv[1:]
            sys.exit(subprocess.call(cmd))
        raise SystemExit(f'--gpus {args.gpus} does not match WORLD_SIZE={world}')
    if args.impl == 'reference':
        run_reference(args)
    else:
        run_ours(args)


if __name__ == '__main__':
    main()
