"""CPU tests of the host-side helpers of the GPU ops: MX fp8 quantisation and scale packing
(msccl/ops/gemm.py), tile geometry of the interpreter (msccl/runtime/plan.py)."""
import pytest
import torch

from msccl.ops.gemm import dequantize_mxfp8, interleave_gate_up, pack_mx_scales, quantize_mxfp8


def test_mxfp8_quantisation_error_and_scale_choice():
    gen = torch.Generator().manual_seed(0)
    x = torch.randn(64, 256, generator=gen) * torch.exp2(torch.randint(-8, 8, (64, 1), generator=gen).float())
    q, s = quantize_mxfp8(x)
    assert q.dtype == torch.float8_e4m3fn and s.dtype == torch.uint8 and s.shape == (64, 8)
    back = dequantize_mxfp8(q, s)
    # e4m3 has 3 mantissa bits: relative error of a normal value at most 2^-4, measured against the block maximum
    blocks = x.reshape(64, 8, 32)
    err = (back.reshape(64, 8, 32) - blocks).abs().amax(dim=-1)
    assert torch.all(err <= blocks.abs().amax(dim=-1) * 2.0 ** -4 + 1e-30)
    # the scale is the smallest power of two that brings the block maximum into the e4m3 range
    scaled_max = blocks.abs().amax(dim=-1) / torch.exp2(s.float() - 127)
    assert torch.all(scaled_max <= 448.0) and torch.all(scaled_max > 224.0 - 1e-3)


def test_mx_scale_packing_layout():
    rows, kblocks = 300, 8                      # 300 rows -> 3 blocks of 128 (4 when padded to 256), K = 256
    s = (torch.arange(rows * kblocks) % 251).to(torch.uint8).reshape(rows, kblocks)
    for row_multiple, tiles in ((128, 3), (256, 4)):
        p = pack_mx_scales(s, row_multiple)
        assert p.numel() == tiles * (kblocks // 4) * 512
        for r, kb in ((0, 0), (31, 3), (32, 4), (137, 5), (299, 7)):
            tile, rr = divmod(r, 128)
            k128, j = divmod(kb, 4)
            off = (tile * (kblocks // 4) + k128) * 512 + (rr % 32) * 16 + (rr // 32) * 4 + j
            assert p[off].item() == s[r, kb].item(), (r, kb)
        # padding rows carry the scale 1.0
        last = (tiles - 1) * (kblocks // 4) * 512
        pad_row = tiles * 128 - 1 - (tiles - 1) * 128
        assert p[last + (pad_row % 32) * 16 + (pad_row // 32) * 4].item() == 127


def test_interleave_gate_up_groups_rows_per_tile():
    g = torch.arange(256 * 4).float().reshape(256, 4)
    u = -g
    w = interleave_gate_up(g, u)
    assert w.shape == (512, 4)
    assert torch.equal(w[:128], g[:128]) and torch.equal(w[128:256], u[:128])
    assert torch.equal(w[256:384], g[128:]) and torch.equal(w[384:], u[128:])


def test_tile_geometry_pipelines_large_chunks():
    from msccl.language import MSCCLProgram
    from msccl.language.collectives import AllReduce
    from msccl.programs.allreduce import allreduce_ring
    from msccl.runtime.plan import PlanError, compile_plan, tile_geometry
    from msccl.topologies import fully_connected
    from msccl.xml import load_xml
    prog = MSCCLProgram('ring', fully_connected(4), AllReduce(4, 4, True), 1)
    with prog:
        allreduce_ring(4, 1)
    slot = 4 << 20
    plan = compile_plan(load_xml(prog.generate_xml()), [0], slot)
    # small chunk: one iteration
    assert tile_geometry(plan, 1024, 2, slot) == (1024, 1)
    # 8 MB chunk: cut into quarters (2 MB tiles) although a 4 MB slot would take half of it at once
    tile, iters = tile_geometry(plan, 4 << 20, 2, slot)
    assert iters == 4 and tile * 2 == 2 << 20
    # 64 MB chunk: the slot size is the limit
    tile, iters = tile_geometry(plan, 32 << 20, 2, slot)
    assert tile * 2 * plan.max_cnt <= slot and iters * tile >= 32 << 20
    # chunks must be whole 16-byte vectors
    with pytest.raises(PlanError):
        tile_geometry(plan, 500, 2, slot)


def test_flat_gradients_bucket_views_and_reduction():
    # gradients are views into flat buckets; the reduction callback sees whole buckets
    from msccl.parallel.data_parallel import FlatGradients
    model = torch.nn.Sequential(torch.nn.Linear(7, 5), torch.nn.Linear(5, 3))
    allocated = []

    def allocate(numel, dtype):
        allocated.append(torch.full((numel,), 9.0, dtype=dtype))
        return allocated[-1]

    flat = FlatGradients(model.parameters(), allocate, bucket_bytes=200)
    assert len(flat.buckets) >= 2 and all(t.numel() % 4 == 0 for t in allocated)          # 16-byte slots of fp32
    assert all(torch.count_nonzero(t) == 0 for t in allocated)
    model(torch.ones(2, 7)).sum().backward()
    for p in model.parameters():
        assert any(p.grad.data_ptr() >= t.data_ptr() and p.grad.data_ptr() < t.data_ptr() + t.numel() * 4 for t in allocated)
    before = [p.grad.clone() for p in model.parameters()]
    seen = []
    flat.all_reduce_gradients(lambda t: seen.append(t.numel()) or t.mul_(4), world=4)      # "sum" of 4 equal ranks
    assert seen == [t.numel() for t in allocated]
    for p, b in zip(model.parameters(), before):
        assert torch.allclose(p.grad, b)
    model[0].weight.grad = torch.zeros_like(model[0].weight)                               # detached from the bucket
    with pytest.raises(RuntimeError):
        flat.all_reduce_gradients(lambda t: t, world=1)


def test_msccl_torch_needs_init():
    import msccl.torch as mt
    assert not mt.is_initialized()
    with pytest.raises(RuntimeError):
        mt.all_reduce(torch.zeros(4))


def test_msccl_torch_falls_back_to_the_library_when_a_call_is_refused(monkeypatch, capsys):
    # a PlanError comes from host-side checks before any launch; the call then runs on torch.distributed, once announced
    import torch.distributed as dist
    import msccl.torch as mt
    from msccl.runtime.plan import PlanError

    class Refusing:
        def all_reduce(self, t, stream=None):
            raise PlanError('999 input elements are not divisible into 256 chunks')

        def all_gather(self, out, inp, stream=None):
            out.copy_(torch.cat([inp, inp]))                      # a call the executor can run is not redirected

    calls = []
    monkeypatch.setattr(dist, 'all_reduce', lambda t, group=None: calls.append(('all_reduce', t.numel(), group)))
    monkeypatch.setattr(dist, 'all_gather_into_tensor', lambda o, i, group=None: calls.append(('all_gather', o.numel(), group)))
    saved = dict(mt._state)
    try:
        mt._state.update(executor=Refusing(), comm=object(), group='grp', nccl_fallback=True, told=set())
        x = torch.ones(999)
        assert mt.all_reduce(x) is x and mt.all_reduce(x) is x
        out = torch.zeros(8)
        mt.all_gather_into_tensor(out, torch.arange(4.0))
        assert calls == [('all_reduce', 999, 'grp'), ('all_reduce', 999, 'grp')] and out.tolist() == [0, 1, 2, 3, 0, 1, 2, 3]
        said = capsys.readouterr().out
        assert said.count('Falling back to NCCL baseline') == 1 and 'not divisible into 256 chunks' in said
        mt._state.update(nccl_fallback=False)
        with pytest.raises(PlanError):
            mt.all_reduce(x)
    finally:
        mt._state.clear()
        mt._state.update(saved)


def test_route_top_k_renormalises():
    from msccl.ops.moe import route_top_k
    logits = torch.tensor([[0.0, 1.0, 2.0, 3.0], [5.0, 5.0, -9.0, -9.0]])
    experts, weights = route_top_k(logits, topk=2)
    assert experts.tolist()[0] == [3, 2] and sorted(experts.tolist()[1]) == [0, 1]
    assert torch.allclose(weights.sum(dim=-1), torch.ones(2))
    e = torch.exp(torch.tensor([3.0, 2.0]))
    assert torch.allclose(weights[0], e / e.sum())


def test_pipeline_handover_on_gloo_ranks():
    import os
    import socket
    import subprocess
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        port = s.getsockname()[1]
    world = 3
    procs = [subprocess.Popen([sys.executable, os.path.join(here, 'mp_pipeline_worker.py')],
                              env=dict(os.environ, MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port), RANK=str(r),
                                       WORLD_SIZE=str(world), OMP_NUM_THREADS='1'),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outs = []
    for p in procs:
        try:
            outs.append(p.communicate(timeout=120)[0])
        except subprocess.TimeoutExpired:
            p.kill()
            outs.append(p.communicate()[0])
    assert [p.returncode for p in procs] == [0] * world, '\n'.join(outs)
    assert all(f'PIPELINE_OK {r}' in outs[r] for r in range(world))


def test_compiled_plan_tables_are_consistent():
    # the flat arrays the interpreter kernel reads: sizes, FIFO offsets agreed by both ends, dependency indices
    import struct
    from msccl.language import MSCCLProgram, ThreadblockPolicy
    from msccl.language.collectives import AllReduce
    from msccl.programs.allreduce import allreduce_ring
    from msccl.runtime.plan import K_FIFO_SLOTS, K_MAX_RANKS, PlanError, compile_plan
    from msccl.topologies import fully_connected
    from msccl.xml import load_xml
    n, slot = 4, 1 << 16
    prog = MSCCLProgram('ring', fully_connected(n), AllReduce(n, n, True), 2, threadblock_policy=ThreadblockPolicy.manual)
    with prog:
        allreduce_ring(n, 2)
    algo = load_xml(prog.generate_xml())
    plan = compile_plan(algo, list(range(n)), slot)
    tb_fmt, step_fmt = struct.Struct('<4h4i2i2q4i'), struct.Struct('<4B2h3i4Bi2H')       # DevTb, DevStep of the kernel
    assert tb_fmt.size == 64 and step_fmt.size == 32
    tbs = [tb_fmt.unpack_from(plan.tb_bytes, i * 64)[:12] for i in range(len(plan.tb_bytes) // 64)]
    steps = [step_fmt.unpack_from(plan.step_bytes, i * 32)[:9] for i in range(len(plan.step_bytes) // 32)]
    assert len(tbs) == algo.num_threadblocks() == plan.total_tbs() and len(steps) == algo.num_steps()
    send_off, recv_off = {}, {}
    for rank, tb_id, send_peer, recv_peer, chan, nsteps, first, tbs_in_rank, send_conn, recv_conn, s_off, r_off in tbs:
        assert tbs_in_rank == len(algo.gpus[rank].tbs) and first + nsteps <= len(steps)
        if send_peer >= 0:
            assert send_conn == chan * K_MAX_RANKS + send_peer and s_off % (K_FIFO_SLOTS * slot) == 0
            send_off[(rank, send_peer, chan)] = s_off
        if recv_peer >= 0:
            assert recv_conn == chan * K_MAX_RANKS + recv_peer
            recv_off[(recv_peer, rank, chan)] = r_off
        for code, sbuf, dbuf, hasdep, depid, deps, soff, doff, cnt in steps[first:first + nsteps]:
            assert 0 <= code <= 8 and sbuf in (0, 1, 2) and dbuf in (0, 1, 2)
            if depid >= 0:
                assert depid < tbs_in_rank and 0 <= deps
    # sender and receiver of a connection agree on where its slots are in the receiver's FIFO area
    assert send_off == recv_off and len(send_off) > 0
    # no two incoming connections of a rank share slots
    for rank in range(n):
        offs = [off for (src, dst, chan), off in recv_off.items() if dst == rank]
        assert len(offs) == len(set(offs))
    # in place: output chunks are addressed through the input buffer
    assert all(plan.extents[r]['o'] == 0 and plan.extents[r]['i'] == n * 2 for r in range(n))
    # in-switch steps are not for the interpreter kernel
    from msccl.language.ext_nvls import allreduce_nvls
    with pytest.raises(PlanError):
        compile_plan(load_xml(allreduce_nvls(4)), [0], slot)


def test_setup_metadata_and_native_build_step():
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    run = subprocess.run([sys.executable, 'setup.py', '--name', '--version'], cwd=root, capture_output=True, text=True)
    assert run.returncode == 0 and run.stdout.split() == ['msccl-b200', '0.1.0'], run.stderr
    # the build step is the in-tree nvcc build; with an up-to-date module it only reports where it is
    run = subprocess.run([sys.executable, 'setup.py', '-q', 'build_ext', '--inplace'], cwd=root, capture_output=True, text=True)
    assert run.returncode == 0 and 'msccl: native module' in run.stdout, run.stdout + run.stderr


@pytest.mark.parametrize('ranks,blocks', [(2, 3), (8, 8)])
def test_fused_kernel_schedules_are_valid_programs(ranks, blocks):
    # the chunk movement of the fused kernels, stated in the DSL: symbolic check, validator, interpreter
    from msccl.interp import run_reference_check
    from msccl.ops.schedules import all_gather_blocks, dispatch_blocks, reduce_scatter_blocks
    from msccl.xml import load_xml, validate
    for prog, coll in ((all_gather_blocks(ranks, blocks), 'allgather'), (reduce_scatter_blocks(ranks, blocks), 'reduce_scatter'),
                       (dispatch_blocks(ranks), 'alltoall')):
        algo = load_xml(prog.generate_xml())
        assert algo.coll == coll and validate(algo) == []
        assert run_reference_check(algo, 2, race_check=True) == 'pass (race-free)'
    # reduce-scatter: every source visits the owners starting with its right neighbour (no two sources on one owner)
    algo = load_xml(reduce_scatter_blocks(ranks, blocks).generate_xml())
    for g in algo.gpus:
        first_send = min((tb for tb in g.tbs if tb.send != -1 and tb.steps and tb.steps[0].type == 's'),
                         key=lambda tb: tb.steps[0].srcoff, default=None)
        assert first_send is not None


def test_fused_kernel_order_tables_are_lowered_from_the_programs():
    # the tables the fused kernels take as arguments come out of the compiled schedule programs: every row block
    # exactly once, own blocks first for the all-gather, block-major production for the reduce-scatter, and a
    # different program (blocks spread over two channels) gives different tables
    from msccl.ops.schedules import (all_gather_blocks, fused_tp_tables, lower_all_gather, lower_reduce_scatter,
                                     reduce_scatter_blocks)
    from msccl.xml import load_xml
    pairs = lambda flat: [(flat[i], flat[i + 1]) for i in range(0, len(flat), 2)]       # noqa: E731
    n, blocks, rank = 8, 8, 3
    ag, rs, red = fused_tp_tables(n, blocks, rank)
    ag, rs = pairs(ag), pairs(rs)
    everything = sorted((r, b) for r in range(n) for b in range(blocks))
    assert sorted(ag) == everything and sorted(rs) == everything and sorted(red) == list(range(blocks))
    assert ag[:blocks] == [(rank, b) for b in range(blocks)]                 # local blocks need no flag: they lead
    assert [b for _, b in ag[blocks:]] == sorted(b for _, b in ag[blocks:])   # then block 0 of every source, block 1, ...
    assert [b for _, b in rs] == sorted(b for _, b in rs)                     # block 0 for every owner, then block 1, ...
    for b in range(blocks):                                                   # own block last among the block's owners
        assert [o for o, bb in rs if bb == b][-1] == rank
    assert red == list(range(blocks))
    # straight from the MSCCL-IR, another program -> another order
    one = lower_reduce_scatter(load_xml(reduce_scatter_blocks(4, 4, channels=1).generate_xml()), 1)[0]
    two = lower_reduce_scatter(load_xml(reduce_scatter_blocks(4, 4, channels=2).generate_xml()), 1)[0]
    assert sorted(one) == sorted(two) and one != two
    assert [b for _, b in two][:4] == [0, 1, 0, 1]                            # a round now holds two blocks per owner
    g1 = lower_all_gather(load_xml(all_gather_blocks(4, 4, channels=1).generate_xml()), 2)
    g2 = lower_all_gather(load_xml(all_gather_blocks(4, 4, channels=2).generate_xml()), 2)
    assert g1 != g2 and g1[:4] == g2[:4] == [(2, b) for b in range(4)]
    # one rank: nothing moves
    assert fused_tp_tables(1, 4, 0) == ([0, 0, 0, 1, 0, 2, 0, 3], [0, 0, 0, 1, 0, 2, 0, 3], [0, 1, 2, 3])


def test_step_trace_exports(tmp_path):
    # the per-step records of the interpreter kernel as JSON lines, as a Trace Event document, and summed up per step type
    import json
    from msccl.runtime import trace
    rows = [{'rank': 0, 'tb': 0, 'step': 0, 'type': 's', 'start_ns': 0, 'end_ns': 4000, 'wait_ns': 500, 'move_ns': 3000, 'signal_ns': 500},
            {'rank': 0, 'tb': 1, 'step': 0, 'type': 'r', 'start_ns': 100, 'end_ns': 6100, 'wait_ns': 4000, 'move_ns': 2000, 'signal_ns': 0},
            {'rank': 1, 'tb': 0, 'step': 1, 'type': 'r', 'start_ns': 200, 'end_ns': 2200, 'wait_ns': 1000, 'move_ns': 1000, 'signal_ns': 0}]
    doc = trace.to_chrome_trace(rows, 'ring')
    slices = [e for e in doc['traceEvents'] if e['ph'] == 'X']
    names = [e for e in doc['traceEvents'] if e['ph'] == 'M']
    assert len(slices) == 3 and slices[1]['name'] == '0: r' and slices[1]['ts'] == 0.1 and slices[1]['dur'] == 6.0
    assert slices[1]['args'] == {'wait_us': 4.0, 'move_us': 2.0, 'signal_us': 0.0}
    assert {(e['name'], e['pid'], e.get('tid')) for e in names} == {('process_name', 0, None), ('process_name', 1, None),
                                                                    ('thread_name', 0, 0), ('thread_name', 0, 1), ('thread_name', 1, 0)}
    assert trace.summarize(rows) == {'r': {'records': 2, 'wait_us': 2.5, 'move_us': 1.5, 'signal_us': 0.0},
                                     's': {'records': 1, 'wait_us': 0.5, 'move_us': 3.0, 'signal_us': 0.5}}
    trace.write(rows, tmp_path / 't.jsonl')
    assert [json.loads(l) for l in open(tmp_path / 't.jsonl')] == rows
    trace.write(rows, tmp_path / 't.json', 'ring')
    assert json.load(open(tmp_path / 't.json'))['otherData'] == {'program': 'ring'}
