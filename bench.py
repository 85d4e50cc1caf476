#!/usr/bin/env python
"""Benchmark of the msccl B200 stack against NCCL (+ cuBLAS) on the same box.

    python bench.py --gpus N --steps K --warmup W            (N>1: launched under torchrun)
    python bench.py --impl reference ...                      (unmodified reference + stock NCCL / cuBLAS)

Headline (``value``): bus bandwidth of an in-place bf16 all-reduce of ``--bytes`` (default 1 GiB, larger than the
126 MB L2, so no cache flush is needed between steps) through the public API - ``msccl.init`` registers the plans,
``msccl.torch.all_reduce`` runs the collective on a tensor from ``msccl.torch.symmetric_empty``.  One step = one
all-reduce; busBW = bytes * 2(n-1)/n / time; time from CUDA events on the launching stream, max over ranks, exactly
``--steps`` steps after ``--warmup`` untimed ones.  The result is verified once after the warm-up against the fp32
sum of every rank's input.  ``sustained`` repeats the measurement over at least one second.  ``e2e`` adds, per step,
the host-to-device copy of the step's input from pinned memory and a device-to-host read of a checksum - the same
recipe in both arms.

The same JSON line carries, device-timed and max over ranks (``--sections`` selects them):
  sweep        all-reduce / all-gather / all-to-all, 1 KiB .. 1 GiB, through ``msccl.torch`` (reference arm: NCCL)
  interpreter  registered MSCCL-IR plans through the interpreter kernel, on ordinary and on symmetric tensors
  tp_mlp       Llama-3-8B MLP, 8192 tokens, tensor parallel over all GPUs: fused all-gather->GEMM->SwiGLU and
               GEMM->reduce-scatter kernels (reference arm: NCCL on a side stream overlapping cuBLAS, 4 chunks)
  moe          expert-parallel MoE layer, 4096 tokens per GPU, 8 experts per GPU, top-2, FFN 14336 (reference arm:
               NCCL all-to-all with split sizes exchanged once + cuBLAS grouped GEMMs)

With one GPU there is no peer: the step is then the 8-rank ring all-reduce MSCCLang program executed by the
interpreter kernel with all eight ranks emulated on the single GPU (256 MiB per emulated rank); that line says
``"scaling": "none"`` because it is another workload than the multi-GPU lines.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
SWEEP_SIZES = [1 << s for s in range(10, 31, 2)]          # 1 KiB .. 1 GiB
TP_TOKENS, TP_HIDDEN, TP_FFN = 8192, 4096, 14336          # Llama-3-8B MLP
MOE_TOKENS, MOE_HIDDEN, MOE_FFN, MOE_EXPERTS_PER_GPU, MOE_TOPK = 4096, 4096, 14336, 8, 2


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


def _timed(n, steps, warmup, step_fn, sync_fn=None):
    """W warm-up steps, then exactly K steps between barrier+synchronize; returns ms per step (max over ranks)."""
    import torch
    import torch.distributed as dist
    for _ in range(warmup):
        step_fn()
    if sync_fn is not None:
        sync_fn()
    torch.cuda.synchronize()
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


def _sustained(n, ms_per_step, step_fn, sync_fn=None):
    """The same measurement over at least one second of device time."""
    steps = max(20, int(1100.0 / max(ms_per_step, 1e-3)) + 1)
    ms = _timed(n, steps, 3, step_fn, sync_fn)
    return {'steps': steps, 'ms_per_step': round(ms, 5), 'timed_region_s': round(ms * steps / 1e3, 3)}


def _sustained_sampled(device_index, clocks, *args):
    """_sustained with its own clock sampler: a timed region of a few dozen milliseconds can end before nvidia-smi has
    delivered its first line; the region of at least a second that follows runs the same step under the same load, and
    its samples stand in when the first sampler came back empty."""
    sampler = ClockSampler(device_index)
    sampler.start()
    sustained = _sustained(*args)
    later = sampler.stop()
    if not clocks.get('samples') and later.get('samples'):
        clocks = dict(later, region='sustained region directly after the timed steps (same step function)')
    return sustained, clocks


def bus_factor(n, collective='allreduce'):
    if n <= 1:
        return 1.0
    return 2.0 * (n - 1) / n if collective == 'allreduce' else (n - 1) / n


def _rank_input(rank, numel, dtype):
    """The seeded N(0, 1) * 0.05 input of ``rank`` (every rank can regenerate every other rank's)."""
    import torch
    gen = torch.Generator(device='cuda').manual_seed(1234 + rank)
    return (torch.randn(numel, device='cuda', generator=gen) * 0.05).to(dtype)


def _verify_allreduce(buf, n, numel, dtype, allreduce):
    """Fill ``buf`` with this rank's seeded input, all-reduce it, compare with the fp32 sum over all ranks' inputs."""
    import torch
    import torch.distributed as dist
    rank = dist.get_rank() if n > 1 else 0
    buf.copy_(_rank_input(rank, numel, dtype))
    torch.cuda.synchronize()
    if n > 1:
        dist.barrier()
    allreduce()
    torch.cuda.synchronize()
    want = torch.zeros(numel, device='cuda', dtype=torch.float32)
    for r in range(n):
        want += _rank_input(r, numel, dtype).float()
    # bf16 keeps 8 bits of mantissa; a sum in rank order rounds after every addition, the in-switch sum once
    err = (buf.float() - want).abs()
    tol = 2.0 ** -7 * want.abs() + n * 2.0 ** -9 * 0.05 * 4
    ok = bool((err <= tol).all().item())
    flag = torch.tensor([1 if ok else 0], device='cuda', dtype=torch.int32)
    if n > 1:
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    del want, err, tol
    return bool(flag.item())


# ============================================================================ this repository's arm
def run_ours(args):
    import torch
    sys.path.insert(0, ROOT)
    n = args.gpus
    local = _dist_setup(n)
    rank = int(os.environ.get('RANK', '0'))
    if n == 1:
        return run_ours_one_gpu(args, local)
    import torch.distributed as dist
    import msccl
    import msccl.torch as mt
    dtype = torch.bfloat16
    nbytes = args.bytes
    numel = nbytes // 2
    sections = set(args.sections.split(','))

    # the public path: msccl.init chooses and compiles the registered plans (once, on rank 0; the table travels
    # as a file name), msccl.torch.init builds the communicator and installs them
    machine = 'b200' if n == 8 else f'b200x{n}'
    path = [None]
    if rank == 0:
        msccl.init(machine, 1, *[(c, (0, None)) for c in (msccl.Collective.allreduce, msccl.Collective.allgather,
                                                           msccl.Collective.alltoall, msccl.Collective.reduce_scatter)])
        path = [os.environ.get('MSCCL_CONFIG')]
    dist.broadcast_object_list(path, src=0)
    if path[0]:
        os.environ['MSCCL_CONFIG'] = path[0]
    arena = nbytes + (1 << 30) + (3 << 30) + (64 << 20)      # headline buffer, sweep output, fused TP / MoE buffers
    ex = mt.init(arena_bytes=arena, fifo_bytes=256 << 20, nccl_fallback=False)    # a refused call must fail here, not be timed on NCCL
    comm = mt.communicator()
    buf = mt.symmetric_empty(numel, dtype)
    pinned = (torch.randn(numel, dtype=torch.float32) * 0.01).to(dtype).pin_memory()
    result_host = torch.empty(1, dtype=torch.float32).pin_memory()

    def step():
        mt.all_reduce(buf)

    def e2e_step():
        buf.copy_(pinned, non_blocking=True)
        mt.all_reduce(buf)
        result_host.copy_(buf[:4096].float().sum().reshape(1), non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(2):
        step()
    mt.check()
    verified = _verify_allreduce(buf, n, numel, dtype, step)
    mt.check()
    buf.copy_(_rank_input(rank, numel, dtype) * 0.01)
    sampler = ClockSampler(local)
    sampler.start()
    launches_before = ex.launches
    ms = _timed(n, args.steps, args.warmup, step, mt.check)
    launches = (ex.launches - launches_before) * args.steps // (args.steps + args.warmup)
    algorithm = ex.last_algorithm
    clocks = sampler.stop()
    mt.check()
    sustained, clocks = _sustained_sampled(local, clocks, n, ms, step, mt.check)
    e2e_ms = _timed(n, max(3, min(args.steps, 10)), 3, e2e_step, mt.check)
    mt.check()
    factor = bus_factor(n)
    value = nbytes * factor / (ms * 1e-3) / 1e9
    kind = {'twoshot': 'direct kernel: two-shot all-reduce on symmetric memory, ' +
                       ('in-switch reduction (multimem)' if comm.mc_base and n > 2 else 'peer loads and stores'),
            'oneshot': 'direct kernel: one-shot LL', 'xml': 'registered MSCCL-IR plan on the interpreter kernel'}
    line = {'metric': 'allreduce_busbw', 'value': round(value, 3), 'unit': 'GB/s', 'n_gpus': n,
            'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': round(ms, 5), 'higher_is_better': True,
            'scaling': 'weak', 'vs_baseline': None, 'dtype': 'bf16', 'data': 'synthetic', 'impl': 'msccl-b200',
            'verified': verified,
            'config': {'model': 'all-reduce, in place, through msccl.init + msccl.torch.all_reduce (' +
                                kind.get(algorithm, str(algorithm)) + ')',
                       'algorithm': algorithm, 'dtype_bytes': 2, 'l2_policy': 'inputs larger than L2',
                       'parallelism': f'{n} ranks, one process per GPU', 'ranks': n, 'bytes_per_rank': nbytes,
                       'global_batch': n * nbytes, 'seq_len': None, 'symmetric_memory': comm.mode,
                       'multicast': bool(comm.mc_base), 'machine_type': machine},
            'clocks': clocks,
            'sustained': dict(sustained, value=round(nbytes * factor / (sustained['ms_per_step'] * 1e-3) / 1e9, 3)),
            'e2e': {'value': round(nbytes * factor / (e2e_ms * 1e-3) / 1e9, 3), 'unit': 'GB/s',
                    'ms_per_step': round(e2e_ms, 5), 'h2d_bytes_per_step': nbytes, 'd2h_bytes_per_step': 4,
                    'how': 'one copy of the whole input from pinned memory, the all-reduce, a checksum read back; '
                           'identical in both arms'},
            'gpu_launches': launches}
    if 'sweep' in sections:
        line['sweep'] = sweep_ours(mt, ex, comm, n, dtype, buf)
    if 'interp' in sections:
        line['interpreter'] = interpreter_rows(ex, comm, n, dtype, buf)
    if 'tp' in sections:
        line['tp_mlp'] = tp_ours(comm, n)
    if 'moe' in sections:
        line['moe'] = moe_ours(comm, n)
    if rank == 0:
        print(json.dumps(line), flush=True)
    mt.shutdown()
    dist.destroy_process_group()


def _iters_for(nbytes):
    return 50 if nbytes <= (1 << 20) else (20 if nbytes <= (1 << 26) else 8)


def sweep_ours(mt, ex, comm, n, dtype, buf):
    """busBW of the size-dispatched collectives, 1 KiB .. 1 GiB, on symmetric tensors (device-timed, max over ranks).
    ``bytes`` is the per-rank message: the all-reduce buffer, the gathered all-gather output, the all-to-all input."""
    import torch
    out_sym = mt.symmetric_empty(1 << 29, dtype)                 # 1 GiB: all-gather / all-to-all output
    src = torch.zeros(1 << 29, dtype=dtype, device='cuda')
    rows = {}
    for coll in ('allreduce', 'allgather', 'alltoall'):
        rows[coll] = []
        for nbytes in SWEEP_SIZES:
            numel = nbytes // 2
            if coll == 'allreduce':
                t = buf[:numel]
                fn = lambda: mt.all_reduce(t)                                               # noqa: E731
            elif coll == 'allgather':
                o, i = out_sym[:numel], src[:numel // n]
                fn = lambda: mt.all_gather_into_tensor(o, i)                                # noqa: E731
            else:
                o, i = out_sym[:numel], src[:numel]
                fn = lambda: mt.all_to_all_single(o, i)                                     # noqa: E731
            ms = _timed(n, _iters_for(nbytes), 3, fn, mt.check)
            rows[coll].append({'bytes': nbytes, 'us': round(ms * 1e3, 2), 'algorithm': ex.last_algorithm,
                               'busbw_gbs': round(nbytes * bus_factor(n, coll) / (ms * 1e-3) / 1e9, 2)})
    return rows


def interpreter_rows(ex, comm, n, dtype, buf):
    """Registered MSCCL-IR plans through the interpreter kernel at three sizes, on ordinary tensors (every tile
    crosses a FIFO) and on symmetric tensors (stores into the receivers' buffers where the program allows)."""
    import torch
    rows = []
    out_sym, _ = comm.symmetric_empty(1 << 27, dtype)            # 256 MiB
    for coll in ('allreduce', 'allgather', 'alltoall'):
        for nbytes in (64 << 10, 16 << 20, 256 << 20):
            numel = nbytes // 2
            for memory in ('ordinary', 'symmetric'):
                if coll == 'allreduce':
                    t = buf[:numel] if memory == 'symmetric' else torch.zeros(numel, dtype=dtype, device='cuda')
                    plan = ex.select('allreduce', nbytes)
                    fn = lambda: ex.all_reduce(t, algorithm='xml')                          # noqa: E731
                elif coll == 'allgather':
                    o = out_sym[:numel] if memory == 'symmetric' else torch.zeros(numel, dtype=dtype, device='cuda')
                    i = torch.zeros(numel // n, dtype=dtype, device='cuda')
                    plan = ex.select('allgather', nbytes // n)
                    fn = lambda: ex.all_gather(o, i, algorithm='xml')                       # noqa: E731
                else:
                    o = out_sym[:numel] if memory == 'symmetric' else torch.zeros(numel, dtype=dtype, device='cuda')
                    i = torch.zeros(numel, dtype=dtype, device='cuda')
                    plan = ex.select('alltoall', nbytes)
                    fn = lambda: ex.all_to_all(o, i, algorithm='xml')                       # noqa: E731
                if plan is None:
                    continue
                ms = _timed(n, _iters_for(nbytes), 3, fn, ex.check)
                rows.append({'collective': coll, 'bytes': nbytes, 'memory': memory, 'plan': plan.algo.name,
                             'protocol': plan.algo.proto, 'direct_mask': ex.last_direct_mask, 'us': round(ms * 1e3, 2),
                             'busbw_gbs': round(nbytes * bus_factor(n, coll) / (ms * 1e-3) / 1e9, 2)})
    return rows


def tp_ours(comm, n):
    """Llama-3-8B MLP, 8192 tokens, TP = n: the two fused kernels of msccl.parallel.TensorParallelMLP."""
    import torch
    import torch.distributed as dist
    from msccl.ops import check_gemm_errors
    from msccl.parallel.tensor_parallel import TensorParallelMLP
    rank = comm.rank
    rows, shard = TP_TOKENS // n, TP_FFN // n
    gen = torch.Generator(device='cuda').manual_seed(7 + rank)
    mk = lambda *s: (torch.randn(*s, device='cuda', generator=gen) * 0.02).bfloat16()      # noqa: E731
    w_gate, w_up, w_down = mk(shard, TP_HIDDEN), mk(shard, TP_HIDDEN), mk(TP_HIDDEN, shard)
    mlp = TensorParallelMLP(comm, rows, TP_HIDDEN, TP_FFN, w_gate=w_gate, w_up=w_up, w_down=w_down)
    x = torch.randn(rows, TP_HIDDEN, device='cuda', generator=gen).bfloat16()
    y = torch.empty(rows, TP_HIDDEN, device='cuda', dtype=torch.bfloat16)
    mlp(x, out=y)
    check_gemm_errors()
    # the benchmark's own shape against torch with fp32 accumulation
    full = torch.empty(n * rows, TP_HIDDEN, device='cuda', dtype=torch.bfloat16)
    dist.all_gather_into_tensor(full, x)
    h = torch.nn.functional.silu(full.float() @ w_gate.float().t()) * (full.float() @ w_up.float().t())
    part = h.bfloat16().float() @ w_down.float().t()
    dist.all_reduce(part)
    want = part[rank * rows:(rank + 1) * rows]
    err = (y.float() - want).abs().max().item()
    flag = torch.tensor([1 if err <= 3e-2 * want.abs().max().item() + 1e-3 else 0], device='cuda', dtype=torch.int32)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    ms = _timed(n, 30, 5, lambda: mlp(x, out=y))
    check_gemm_errors()
    result = {'tokens': TP_TOKENS, 'hidden': TP_HIDDEN, 'ffn': TP_FFN, 'tp': n, 'us': round(ms * 1e3, 1),
              'tokens_per_s': round(TP_TOKENS / (ms * 1e-3)), 'verified': bool(flag.item()), 'kernels_per_step': 2}
    # the same layer on block-scaled fp8 operands (weights quantised once, activations per call, inside the step)
    try:
        mlp8 = TensorParallelMLP(comm, rows, TP_HIDDEN, TP_FFN, w_gate=w_gate, w_up=w_up, w_down=w_down, precision='mxfp8')
        y8 = torch.empty_like(y)
        mlp8(x, out=y8)
        check_gemm_errors()
        rel = ((y8.float() - want).norm() / want.norm()).item()          # fp8 operands: a few percent of the norm
        flag8 = torch.tensor([1 if rel < 0.1 else 0], device='cuda', dtype=torch.int32)
        dist.all_reduce(flag8, op=dist.ReduceOp.MIN)
        ms8 = _timed(n, 30, 5, lambda: mlp8(x, out=y8))
        check_gemm_errors()
        result['mxfp8'] = {'us': round(ms8 * 1e3, 1), 'tokens_per_s': round(TP_TOKENS / (ms8 * 1e-3)),
                           'verified': bool(flag8.item()), 'relative_error_vs_fp32': round(rel, 4),
                           'includes': 'quantisation of the token shard and of the SwiGLU output'}
    except Exception as e:      # noqa: BLE001 - reported in the line, the bf16 number stands on its own
        result['mxfp8'] = {'error': f'{type(e).__name__}: {e}'[:200]}
    del full, h, part, want
    return result


def moe_ours(comm, n):
    import torch
    from msccl.ops import check_gemm_errors
    from msccl.parallel.expert_parallel import ExpertParallelMoE
    experts = MOE_EXPERTS_PER_GPU * n
    layer = ExpertParallelMoE(comm, MOE_TOKENS, MOE_HIDDEN, MOE_FFN, experts, MOE_TOPK)
    gen = torch.Generator(device='cuda').manual_seed(99 + comm.rank)
    x = torch.randn(MOE_TOKENS, MOE_HIDDEN, device='cuda', generator=gen).bfloat16()
    logits = torch.randn(MOE_TOKENS, experts, device='cuda', generator=gen)
    y = torch.empty_like(x)
    layer(x, gate_logits=logits, out=y)
    check_gemm_errors()
    ms = _timed(n, 10, 3, lambda: layer(x, gate_logits=logits, out=y))
    check_gemm_errors()
    flops = 2.0 * MOE_TOKENS * MOE_TOPK * 3 * MOE_HIDDEN * MOE_FFN
    return {'tokens_per_gpu': MOE_TOKENS, 'experts': experts, 'topk': MOE_TOPK, 'ffn': MOE_FFN, 'us': round(ms * 1e3, 1),
            'tokens_per_s': round(n * MOE_TOKENS / (ms * 1e-3)), 'tflops_per_gpu': round(flops / (ms * 1e-3) / 1e12, 1),
            'finite': bool(torch.isfinite(y.float()).all().item())}


def run_ours_one_gpu(args, local):
    """One GPU: the 8-rank ring all-reduce program on the interpreter kernel, all ranks emulated on the GPU."""
    import torch
    from msccl.interp import run_algorithm
    from msccl.language import MSCCLProgram, ThreadblockPolicy
    from msccl.language.collectives import AllReduce
    from msccl.programs.allreduce import allreduce_ring
    from msccl.runtime import Communicator, Executor
    from msccl.topologies import fully_connected
    from msccl.xml import load_xml
    dtype, esize, world = torch.bfloat16, 2, 8
    nbytes = min(args.bytes, 256 << 20)
    prog = MSCCLProgram('allreduce_ring', fully_connected(world), AllReduce(world, world, True), 4,
                        threadblock_policy=ThreadblockPolicy.manual)
    with prog:
        allreduce_ring(world, 4)
    algo = load_xml(prog.generate_xml())
    comm = Communicator.emulated(world, fifo_bytes=256 << 20)
    ex = Executor(comm)
    plan = ex.compile(algo)
    numel = nbytes // esize
    # verification on a small case of the same program against the CPU interpreter (bit exact)
    from msccl.interp import input_chunks_of
    gen = torch.Generator().manual_seed(0)
    small_chunk = 4096
    small = [torch.randn(input_chunks_of(algo, r) * small_chunk, generator=gen).to(dtype) for r in range(world)]
    got = ex.run(plan, {r: small[r].cuda() for r in range(world)})
    ex.check()
    want = run_algorithm(algo, small, small_chunk, dtype=dtype)
    verified = all(torch.equal(got[r].cpu().view(torch.int16), want[r].view(torch.int16)) for r in range(world))
    bufs = {r: (torch.randn(numel, device='cuda', dtype=torch.float32) * 0.01).to(dtype) for r in range(world)}
    pinned = (torch.randn(numel, dtype=torch.float32) * 0.01).to(dtype).pin_memory()
    result_host = torch.empty(1, dtype=torch.float32).pin_memory()

    def step():
        ex.run(plan, bufs)

    def e2e_step():
        bufs[0].copy_(pinned, non_blocking=True)
        ex.run(plan, bufs)
        result_host.copy_(bufs[0][:4096].float().sum().reshape(1), non_blocking=True)
        torch.cuda.current_stream().synchronize()

    sampler = ClockSampler(local)
    sampler.start()
    before = ex.launches
    ms = _timed(1, args.steps, args.warmup, step, ex.check)
    launches = (ex.launches - before) * args.steps // (args.steps + args.warmup)
    clocks = sampler.stop()
    ex.check()
    for r in range(world):
        bufs[r].mul_(0)            # the sums of the timed steps have grown; start the next regions from zeros
    sustained, clocks = _sustained_sampled(local, clocks, 1, ms, step, ex.check)
    e2e_ms = _timed(1, max(3, min(args.steps, 10)), 3, e2e_step, ex.check)
    ex.check()
    factor = bus_factor(world)
    line = {'metric': 'allreduce_busbw', 'value': round(nbytes * factor / (ms * 1e-3) / 1e9, 3), 'unit': 'GB/s', 'n_gpus': 1,
            'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': round(ms, 5), 'higher_is_better': True,
            'scaling': 'none', 'vs_baseline': None, 'dtype': 'bf16', 'data': 'synthetic', 'impl': 'msccl-b200',
            'verified': verified,
            'config': {'model': 'all-reduce, MSCCLang ring program on the MSCCL-IR interpreter kernel, 8 ranks emulated on '
                                'one GPU (another workload than the multi-GPU lines: no NVLink is involved)',
                       'algorithm': 'allreduce_ring, 4 channels x 4 instances, Simple protocol, stores into the '
                                    'receiving rank\'s buffer where the program allows',
                       'dtype_bytes': esize, 'l2_policy': 'inputs larger than L2',
                       'parallelism': 'emulated 8 ranks on 1 GPU', 'ranks': world, 'bytes_per_rank': nbytes,
                       'global_batch': world * nbytes, 'seq_len': None,
                       'direct_steps': plan.host.direct_steps, 'threadblocks': plan.grid},
            'clocks': clocks,
            'sustained': dict(sustained, value=round(nbytes * factor / (sustained['ms_per_step'] * 1e-3) / 1e9, 3)),
            'e2e': {'value': round(nbytes * factor / (e2e_ms * 1e-3) / 1e9, 3), 'unit': 'GB/s',
                    'ms_per_step': round(e2e_ms, 5), 'h2d_bytes_per_step': nbytes, 'd2h_bytes_per_step': 4,
                    'how': 'one copy of rank 0\'s input from pinned memory, the program, a checksum read back'},
            'gpu_launches': launches}
    print(json.dumps(line), flush=True)
    comm.close()


# ============================================================================ reference arm
def run_reference(args):
    """The reference's public path: ``msccl.init(...)`` followed by ordinary ``torch.distributed``
    calls (reference README.md:20-38).  The reference contains no runtime of its own, so the
    collective itself is executed by the stock NCCL that ships with PyTorch, and the GEMMs of the
    tensor-parallel and MoE sections by cuBLAS through torch.  Nothing of this repository's package runs here."""
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
    buf = torch.empty(numel, device='cuda', dtype=dtype)
    pinned = (torch.randn(numel, dtype=torch.float32) * 0.01).to(dtype).pin_memory()
    result_host = torch.empty(1, dtype=torch.float32).pin_memory()
    sampler = ClockSampler(local)
    sections = set(args.sections.split(','))

    def step():
        dist.all_reduce(buf)

    def e2e_step():
        buf.copy_(pinned, non_blocking=True)
        dist.all_reduce(buf)
        result_host.copy_(buf[:4096].float().sum().reshape(1), non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(2):
        step()
    verified = _verify_allreduce(buf, n, numel, dtype, step) if n > 1 else None
    buf.copy_(_rank_input(rank, numel, dtype) * 0.01)
    sampler.start()
    ms = _timed(n, args.steps, args.warmup, step)
    clocks = sampler.stop()
    if n == 1:
        # One GPU: this repo's arm runs an 8-rank program with all ranks emulated on the GPU.  The reference
        # has no way to do that (its runtime is NCCL, which refuses two ranks on one device), and a 1-rank
        # all-reduce moves no data, so there is no reference number for this configuration.  What the
        # reference's path does with one rank is recorded for information only.
        print(json.dumps({'impl': 'reference', 'unavailable': 'the reference runs collectives through NCCL, which cannot '
                          'place the 8 ranks of this configuration on one GPU; its 1-rank all-reduce is an identity that '
                          'moves no data', 'n_gpus': 1,
                          'one_rank_identity': {'bytes': nbytes, 'ms_per_call': round(ms, 5), 'note': note},
                          'clocks': clocks}), flush=True)
        dist.destroy_process_group()
        return
    sustained, clocks = _sustained_sampled(local, clocks, n, ms, step)
    e2e_ms = _timed(n, max(3, min(args.steps, 10)), 3, e2e_step)
    factor = bus_factor(n)
    line = {'metric': 'allreduce_busbw', 'value': round(nbytes * factor / (ms * 1e-3) / 1e9, 3), 'unit': 'GB/s',
            'n_gpus': n, 'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': round(ms, 5),
            'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': 'bf16',
            'data': 'synthetic', 'impl': 'reference', 'verified': verified,
            'config': {'model': 'all-reduce, in place (reference msccl.init + torch.distributed / stock NCCL)',
                       'bytes_per_rank': nbytes, 'global_batch': n * nbytes, 'seq_len': None,
                       'parallelism': f'{n} ranks, one process per GPU', 'ranks': n, 'note': note,
                       'nccl': '.'.join(map(str, torch.cuda.nccl.version())), 'dtype_bytes': 2,
                       'l2_policy': 'inputs larger than L2'},
            'clocks': clocks,
            'sustained': dict(sustained, value=round(nbytes * factor / (sustained['ms_per_step'] * 1e-3) / 1e9, 3)),
            'e2e': {'value': round(nbytes * factor / (e2e_ms * 1e-3) / 1e9, 3), 'unit': 'GB/s',
                    'ms_per_step': round(e2e_ms, 5), 'h2d_bytes_per_step': nbytes, 'd2h_bytes_per_step': 4,
                    'how': 'one copy of the whole input from pinned memory, the all-reduce, a checksum read back; '
                           'identical in both arms'},
            'gpu_launches': 0}
    if 'sweep' in sections:
        line['sweep'] = sweep_reference(n, dtype, buf)
    if 'tp' in sections:
        line['tp_mlp'] = tp_reference(n)
    if 'moe' in sections:
        line['moe'] = moe_reference(n)
    if rank == 0:
        print(json.dumps(line), flush=True)
    dist.destroy_process_group()


def sweep_reference(n, dtype, buf):
    import torch
    import torch.distributed as dist
    out = torch.zeros(1 << 29, dtype=dtype, device='cuda')
    src = torch.zeros(1 << 29, dtype=dtype, device='cuda')
    rows = {}
    for coll in ('allreduce', 'allgather', 'alltoall'):
        rows[coll] = []
        for nbytes in SWEEP_SIZES:
            numel = nbytes // 2
            if coll == 'allreduce':
                t = buf[:numel]
                fn = lambda: dist.all_reduce(t)                                             # noqa: E731
            elif coll == 'allgather':
                o, i = out[:numel], src[:numel // n]
                fn = lambda: dist.all_gather_into_tensor(o, i)                              # noqa: E731
            else:
                o, i = out[:numel], src[:numel]
                fn = lambda: dist.all_to_all_single(o, i)                                   # noqa: E731
            ms = _timed(n, _iters_for(nbytes), 3, fn)
            rows[coll].append({'bytes': nbytes, 'us': round(ms * 1e3, 2), 'algorithm': 'nccl',
                               'busbw_gbs': round(nbytes * bus_factor(n, coll) / (ms * 1e-3) / 1e9, 2)})
    return rows


def tp_reference(n, chunks=4):
    """NCCL + cuBLAS pipeline for the same MLP: the all-gather runs in ``chunks`` pieces on a side stream and the
    (gate|up) GEMM of piece c overlaps the gathering of piece c + 1; the down GEMM of piece c overlaps the
    reduce-scatter of piece c - 1."""
    import torch
    import torch.distributed as dist
    rows, shard = TP_TOKENS // n, TP_FFN // n
    piece = rows // chunks
    x = torch.randn(rows, TP_HIDDEN, device='cuda').bfloat16()
    wgu = (torch.randn(2 * shard, TP_HIDDEN, device='cuda') * 0.02).bfloat16()
    wd = (torch.randn(TP_HIDDEN, shard, device='cuda') * 0.02).bfloat16()
    side = torch.cuda.Stream()
    gathered = [torch.empty(n * piece, TP_HIDDEN, device='cuda', dtype=torch.bfloat16) for _ in range(chunks)]
    partial = [torch.empty(n * piece, TP_HIDDEN, device='cuda', dtype=torch.bfloat16) for _ in range(chunks)]
    y = torch.empty(rows, TP_HIDDEN, device='cuda', dtype=torch.bfloat16)
    ready = [torch.cuda.Event() for _ in range(chunks)]
    done = [torch.cuda.Event() for _ in range(chunks)]

    def step():
        main = torch.cuda.current_stream()
        side.wait_stream(main)
        with torch.cuda.stream(side):
            for c in range(chunks):
                dist.all_gather_into_tensor(gathered[c], x[c * piece:(c + 1) * piece])
                ready[c].record(side)
        for c in range(chunks):
            main.wait_event(ready[c])
            gu = gathered[c] @ wgu.t()
            h = torch.nn.functional.silu(gu[:, :shard]) * gu[:, shard:]
            torch.matmul(h, wd.t(), out=partial[c])
            done[c].record(main)
            with torch.cuda.stream(side):
                side.wait_event(done[c])
                dist.reduce_scatter_tensor(y[c * piece:(c + 1) * piece], partial[c])
        main.wait_stream(side)

    def sequential():
        full = torch.empty(n * rows, TP_HIDDEN, device='cuda', dtype=torch.bfloat16)
        dist.all_gather_into_tensor(full, x)
        gu = full @ wgu.t()
        h = torch.nn.functional.silu(gu[:, :shard]) * gu[:, shard:]
        part = h @ wd.t()
        dist.reduce_scatter_tensor(y, part)

    ms = _timed(n, 30, 5, step)
    ms_seq = _timed(n, 30, 5, sequential)
    best = min(ms, ms_seq)
    return {'tokens': TP_TOKENS, 'hidden': TP_HIDDEN, 'ffn': TP_FFN, 'tp': n, 'us': round(best * 1e3, 1),
            'tokens_per_s': round(TP_TOKENS / (best * 1e-3)), 'overlapped_us': round(ms * 1e3, 1),
            'sequential_us': round(ms_seq * 1e3, 1), 'chunks': chunks}


def moe_reference(n):
    """NCCL + cuBLAS MoE layer without host synchronisation inside the step: the routing of the (fixed) input is
    exchanged once before the timed region, which gives ``all_to_all_single`` its split sizes; every step then
    sorts the token copies by expert, dispatches them, runs the experts' GEMMs on their row ranges (one grouped
    GEMM when torch has it, else one cuBLAS call per local expert with sizes known on the host), sends the
    results back and combines them with the routing weights."""
    import torch
    import torch.distributed as dist
    rank = dist.get_rank()
    le, experts = MOE_EXPERTS_PER_GPU, MOE_EXPERTS_PER_GPU * n
    gen = torch.Generator(device='cuda').manual_seed(99 + rank)
    x = torch.randn(MOE_TOKENS, MOE_HIDDEN, device='cuda', generator=gen).bfloat16()
    logits = torch.randn(MOE_TOKENS, experts, device='cuda', generator=gen)
    wgen = torch.Generator(device='cuda').manual_seed(rank)
    w_gu = (torch.randn(le, 2 * MOE_FFN, MOE_HIDDEN, device='cuda', generator=wgen) * 0.02).bfloat16()
    w_dn = (torch.randn(le, MOE_HIDDEN, MOE_FFN, device='cuda', generator=wgen) * 0.02).bfloat16()

    def route():
        probs = torch.softmax(logits.float(), dim=-1)
        wts, ids = torch.topk(probs, MOE_TOPK, dim=-1)
        return ids, wts / wts.sum(dim=-1, keepdim=True)

    # once, outside the timed region: how many copies go to every expert, and what arrives here
    ids, _ = route()
    counts = torch.bincount(ids.reshape(-1), minlength=experts)
    recv_counts = torch.empty_like(counts)
    dist.all_to_all_single(recv_counts, counts)                    # [src rank, local expert]
    send_splits = counts.view(n, le).sum(1).tolist()
    recv_matrix = recv_counts.view(n, le)
    recv_splits = recv_matrix.sum(1).tolist()
    total_recv = sum(recv_splits)
    # received rows are ordered (source rank, expert); the experts want (expert, source rank)
    seg_start = torch.cumsum(recv_matrix.reshape(-1), 0) - recv_matrix.reshape(-1)
    order = []
    for e in range(le):
        for s in range(n):
            k = s * le + e
            order.append(torch.arange(int(seg_start[k]), int(seg_start[k]) + int(recv_matrix[s, e]), device='cuda'))
    to_expert_major = torch.cat(order)
    per_expert = recv_matrix.sum(0).tolist()
    offsets = torch.tensor(per_expert, device='cuda').cumsum(0).to(torch.int32)
    grouped = hasattr(torch, '_grouped_mm')
    recv = torch.empty(total_recv, MOE_HIDDEN, device='cuda', dtype=torch.bfloat16)
    back = torch.empty(MOE_TOKENS * MOE_TOPK, MOE_HIDDEN, device='cuda', dtype=torch.bfloat16)
    y = torch.empty(MOE_TOKENS, MOE_HIDDEN, device='cuda', dtype=torch.bfloat16)

    def experts_fn(rows, use_grouped):
        if use_grouped:
            gu = torch._grouped_mm(rows, w_gu.transpose(1, 2), offs=offsets)
            h = torch.nn.functional.silu(gu[:, :MOE_FFN]) * gu[:, MOE_FFN:]
            return torch._grouped_mm(h, w_dn.transpose(1, 2), offs=offsets)
        out = torch.empty(total_recv, MOE_HIDDEN, device='cuda', dtype=torch.bfloat16)
        lo = 0
        for e in range(le):
            hi = lo + per_expert[e]
            gu = rows[lo:hi] @ w_gu[e].t()
            h = torch.nn.functional.silu(gu[:, :MOE_FFN]) * gu[:, MOE_FFN:]
            torch.matmul(h, w_dn[e].t(), out=out[lo:hi])
            lo = hi
        return out

    state = {'grouped': grouped}

    def step():
        ids, wts = route()
        flat = ids.reshape(-1)
        perm = torch.argsort(flat, stable=True)
        send = x[perm // MOE_TOPK]
        dist.all_to_all_single(recv, send, recv_splits, send_splits)
        out = experts_fn(recv[to_expert_major], state['grouped'])
        unsorted = torch.empty_like(out)
        unsorted[to_expert_major] = out
        dist.all_to_all_single(back, unsorted, send_splits, recv_splits)
        contrib = torch.empty_like(back)
        contrib[perm] = back
        y.copy_((contrib.view(MOE_TOKENS, MOE_TOPK, MOE_HIDDEN).float() * wts.unsqueeze(-1)).sum(1))

    try:
        step()
        torch.cuda.synchronize()
    except Exception:      # noqa: BLE001 - this torch build has no grouped GEMM for these operands
        state['grouped'] = False
        step()
        torch.cuda.synchronize()
    ms = _timed(n, 10, 3, step)
    flops = 2.0 * MOE_TOKENS * MOE_TOPK * 3 * MOE_HIDDEN * MOE_FFN
    return {'tokens_per_gpu': MOE_TOKENS, 'experts': experts, 'topk': MOE_TOPK, 'ffn': MOE_FFN, 'us': round(ms * 1e3, 1),
            'tokens_per_s': round(n * MOE_TOKENS / (ms * 1e-3)), 'tflops_per_gpu': round(flops / (ms * 1e-3) / 1e12, 1),
            'grouped_gemm': state['grouped'], 'finite': bool(torch.isfinite(y.float()).all().item())}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=200)
    ap.add_argument('--warmup', type=int, default=5)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--bytes', type=int, default=1 << 30, help='message size per rank')
    ap.add_argument('--sections', default='sweep,interp,tp,moe',
                    help='comma-separated extra sections of the multi-GPU line: sweep, interp, tp, moe ("" for none)')
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
