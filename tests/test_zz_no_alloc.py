"""The allocation-free entry point ``msccl_exec_noalloc`` (csrc/no_alloc.h), called through its
exported C symbol, must produce exactly what the ordinary executor produces.

The file name sorts last on purpose: if this addition fails, a run that stops at the first failure
has already exercised everything else.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

FIFO_PER_RANK = 512 * 1024          # MSCCL_NOALLOC_FIFO_PER_RANK
FIFO_SLOTS = 4


def _two_shot_program(n, protocol='Simple'):
    from msccl.language import MSCCLProgram, ThreadblockPolicy
    from msccl.language.collectives import AllReduce
    from msccl.programs.allreduce import allreduce_two_shot
    from msccl.topologies import fully_connected
    from msccl.xml import load_xml
    prog = MSCCLProgram('two_shot', fully_connected(n), AllReduce(n, n, True), 1,
                        threadblock_policy=ThreadblockPolicy.manual, protocol=protocol)
    with prog:
        allreduce_two_shot(n)
    return load_xml(prog.generate_xml())


def _library():
    from msccl.runtime.build import module_path
    lib = ctypes.CDLL(module_path())
    lib.msccl_exec_noalloc.restype = ctypes.c_int
    lib.msccl_exec_noalloc.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                       ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p),
                                       ctypes.POINTER(ctypes.c_int), ctypes.c_longlong, ctypes.c_longlong, ctypes.c_int,
                                       ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.msccl_exec_noalloc_status.restype = ctypes.c_int
    lib.msccl_exec_noalloc_status.argtypes = [ctypes.c_int, ctypes.c_void_p]
    lib.msccl_noalloc_last_error.restype = ctypes.c_char_p
    return lib


def _call(lib, host, algo, tensors, chunk, slot_bytes, dtype_code):
    n = algo.ngpus
    ins = (ctypes.c_void_p * n)(*[t.data_ptr() for t in tensors])
    outs = (ctypes.c_void_p * n)(*[None] * n)          # the program is in place
    scratch = (ctypes.c_int * n)(*[host.extents[r]['s'] for r in range(n)])
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.msccl_exec_noalloc(host.tb_bytes, len(host.tb_bytes) // 64, host.step_bytes, len(host.step_bytes) // 32, n,
                                ins, outs, scratch, chunk, slot_bytes, host.max_cnt, dtype_code, host.proto, stream)
    return rc


@pytest.mark.parametrize('protocol,chunk', [('Simple', 6000), ('LL', 6000), ('LL', 64), ('LL128', 6000)])
@pytest.mark.parametrize('dtype,code', [(torch.float32, 0), (torch.bfloat16, 1)])
def test_matches_the_ordinary_executor_twice_in_a_row(dtype, code, protocol, chunk):
    # 6000-element chunks need several iterations through the small FIFOs; 64-element chunks with the flag-in-data
    # protocol fit one tile per connection, the case in which packets left by the previous call would be taken
    # for new ones if the two calls used the same flags
    from msccl.runtime import Communicator, Executor
    from msccl.runtime.plan import compile_plan, fifo_index_tables
    n = 4
    algo = _two_shot_program(n, protocol)
    conns = max(len(t) for t in fifo_index_tables(algo).values())
    slot_bytes = FIFO_PER_RANK // (conns * FIFO_SLOTS) // 1024 * 1024
    host = compile_plan(algo, range(n), slot_bytes)
    lib = _library()

    comm = Communicator.emulated(n, fifo_bytes=2 << 20)
    try:
        ex = Executor(comm)
        plan = ex.compile(algo)
        gen = torch.Generator().manual_seed(2024)
        for call in range(2):
            data = [torch.randn(n * chunk, generator=gen).to(dtype) for _ in range(n)]
            want = ex.run(plan, {r: data[r].cuda() for r in range(n)})
            ex.check()
            mine = [d.cuda() for d in data]
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info()[0]
            rc = _call(lib, host, algo, mine, chunk, slot_bytes, code)
            assert rc == 0, lib.msccl_noalloc_last_error().decode()
            assert lib.msccl_exec_noalloc_status(n, torch.cuda.current_stream().cuda_stream) == 0
            # The first call on a device makes the driver load the library's device image, fixed array included (CUDA loads
            # modules lazily), so free memory may drop once by the size of that image; no later call may change it.
            if call > 0:
                assert torch.cuda.mem_get_info()[0] == free_before, 'the entry point must not allocate device memory'
            for r in range(n):
                assert torch.equal(mine[r].view(torch.uint8), want[r].view(torch.uint8)), f'call {call}, rank {r}'
    finally:
        comm.close()


def test_rejects_requests_beyond_the_fixed_array():
    from msccl.runtime.plan import compile_plan
    algo = _two_shot_program(4)
    lib = _library()
    tensors = [torch.zeros(4 * 64, device='cuda') for _ in range(4)]
    # FIFO slots larger than the fixed FIFO area
    host = compile_plan(algo, range(4), 1 << 20)
    assert _call(lib, host, algo, tensors, 64, 1 << 20, 0) == 1
    assert b'FIFO' in lib.msccl_noalloc_last_error()
    # scratch larger than the fixed scratch area (3 chunks of 64 Ki floats per rank = 768 KiB)
    host = compile_plan(algo, range(4), 32 * 1024)
    big = [torch.zeros(4 * 65536, device='cuda') for _ in range(4)]
    assert _call(lib, host, algo, big, 65536, 32 * 1024, 0) == 1
    assert b'scratch' in lib.msccl_noalloc_last_error()
    # unknown element type
    assert _call(lib, host, algo, tensors, 64, 32 * 1024, 7) == 2


def test_chunks_of_any_size_run_on_element_wide_accesses():
    from msccl.interp import run_algorithm
    from msccl.runtime.plan import compile_plan
    n, chunk = 4, 333
    algo = _two_shot_program(n)
    host = compile_plan(algo, range(n), 32 * 1024)
    lib = _library()
    gen = torch.Generator().manual_seed(7)
    data = [torch.randn(n * chunk, generator=gen) for _ in range(n)]
    want = run_algorithm(algo, data, chunk, dtype=torch.float32)
    mine = [d.cuda() for d in data]
    assert _call(lib, host, algo, mine, chunk, 32 * 1024, 0) == 0, lib.msccl_noalloc_last_error().decode()
    assert lib.msccl_exec_noalloc_status(n, torch.cuda.current_stream().cuda_stream) == 0
    for r in range(n):
        assert torch.equal(mine[r].cpu(), want[r])
