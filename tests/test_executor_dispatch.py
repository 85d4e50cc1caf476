"""Size- and placement-based dispatch of ``Executor.all_*`` and the hand-over of in-switch programs, checked on
CPU against a recording stand-in for the native module (no kernel runs; the arguments are what is tested)."""
import pytest
import torch

from msccl.runtime.executor import DTYPE_CODES, Executor
from msccl.runtime.plan import PlanError


class FakeNative:
    def __init__(self):
        self.calls = []

    def __getattr__(self, name):
        def record(*args, **kwargs):
            self.calls.append((name, args, kwargs))
        return record


class FakeStream:
    cuda_stream = 77


class FakeComm:
    """Just enough of a Communicator: one process per GPU, a registered arena that is one CPU tensor."""
    emulated_mode = False
    timeout_ns = 5
    dev_heap_bases, dev_syncs, dev_staging = 1001, 1002, 1003
    off_arena = 0

    def __init__(self, world=8, rank=3, multicast=True):
        self.world, self.rank = world, rank
        self.local_ranks = [rank]
        self.native = FakeNative()
        self.mc_base = 5000 if multicast else 0
        self.ll_max_bytes = (2 << 20) if world == 2 else max(256 << 10, (2 << 20) // world)
        self.ll_slot_bytes = 2 * self.ll_max_bytes
        self.arena = torch.zeros(64 << 20, dtype=torch.uint8)

    def sync_ptr(self, r):
        return 2000 + r

    def heap_offset_of(self, t):
        base = self.arena.data_ptr()
        if base <= t.data_ptr() and t.data_ptr() + t.numel() * t.element_size() <= base + self.arena.numel():
            return t.data_ptr() - base
        return None

    def symmetric(self, numel, dtype, at=0):
        esize = torch.empty((), dtype=dtype).element_size()
        return self.arena[at:at + numel * esize].view(dtype)


@pytest.fixture
def ex():
    return Executor(FakeComm())


def last(ex):
    return ex.comm.native.calls[-1]


def test_all_reduce_picks_one_shot_then_two_shot(ex):
    s = FakeStream()
    small = torch.zeros(1024)                                   # 4 KB, ordinary memory
    ex.all_reduce(small, stream=s)
    name, args, _ = last(ex)
    assert name == 'oneshot_allreduce' and ex.last_algorithm == 'oneshot'
    assert args[3] == 4096 and args[5] == DTYPE_CODES[torch.float32] and args[-1] == 77
    big = ex.comm.symmetric(4 << 20, torch.bfloat16)            # 8 MB in the arena
    ex.all_reduce(big, stream=s)
    name, args, _ = last(ex)
    assert name == 'twoshot_allreduce' and ex.last_algorithm == 'twoshot'
    assert args[1] == 5000 and args[2] == 0 and args[3] == 8 << 20 and args[9] == 8      # multicast window, 8 CTAs
    outside = torch.zeros(4 << 20, dtype=torch.bfloat16)        # large but not registered: needs a plan
    with pytest.raises(PlanError):
        ex.all_reduce(outside, stream=s)


def test_gather_type_collectives_by_block_size(ex):
    s, n = FakeStream(), 8
    out = torch.zeros(n * 1024, dtype=torch.int32)              # any element type, ordinary memory
    ex.all_gather(out, torch.zeros(1024, dtype=torch.int32), stream=s)
    name, args, _ = last(ex)
    assert name == 'oneshot' and args[3] == 4096 and args[5] == 0 and args[11] == 1       # bits only: fp32 instance
    ex.all_to_all(out, torch.ones(n * 1024, dtype=torch.int32), stream=s)
    assert last(ex)[0] == 'oneshot' and last(ex)[1][11] == 3 and last(ex)[1][3] == 4096
    red = torch.zeros(1024, dtype=torch.bfloat16)
    ex.reduce_scatter(red, torch.zeros(n * 1024, dtype=torch.bfloat16), stream=s)
    assert last(ex)[0] == 'oneshot' and last(ex)[1][11] == 2 and last(ex)[1][5] == DTYPE_CODES[torch.bfloat16]
    # reduce-scatter must not alias input and output
    buf = torch.zeros(n * 1024, dtype=torch.bfloat16)
    with pytest.raises(PlanError):
        ex.reduce_scatter(buf[:1024], buf, stream=s, algorithm='oneshot')
    # 1 MB blocks: symmetric output -> stores straight into the peers; up to 16 MB in total through the switch
    sym = ex.comm.symmetric(n * (512 << 10), torch.bfloat16)
    ex.all_gather(sym, torch.zeros(512 << 10, dtype=torch.bfloat16), stream=s)
    name, args, _ = last(ex)
    assert name == 'push_blocks' and ex.last_algorithm == 'direct' and args[1] is True and args[3] == 5000
    big = ex.comm.symmetric(n * (2 << 20), torch.bfloat16)      # 32 MB in total: peer stores
    ex.all_gather(big, torch.zeros(2 << 20, dtype=torch.bfloat16), stream=s)
    assert last(ex)[0] == 'push_blocks' and last(ex)[1][3] == 0
    ex.all_to_all(big, torch.zeros(n * (2 << 20), dtype=torch.bfloat16), stream=s)
    name, args, _ = last(ex)
    assert name == 'push_blocks' and args[1] is False and args[5] == 4 << 20              # one block per peer
    ex.reduce_scatter(torch.zeros(2 << 20, dtype=torch.bfloat16), big, stream=s)
    name, args, kwargs = last(ex)
    assert name == 'twoshot_allreduce' and args[1] == 5000 and args[-1] != 0               # result to ordinary memory


def test_in_switch_programs_go_to_the_native_kernels(ex):
    from msccl.language.ext_nvls import allgather_nvls, allreduce_nvls, reduce_scatter_nvls
    s, n, rank = FakeStream(), 8, 3
    t = ex.comm.symmetric(n * 4096, torch.bfloat16, at=1 << 20)
    plan = ex.compile(allreduce_nvls(n, 4))
    assert plan.nvls_kind == 'allreduce' and plan.grid == 0
    assert ex.run(plan, t, stream=s)[rank] is t
    name, args, _ = last(ex)
    assert name == 'twoshot_allreduce' and args[:4] == (1001, 5000, 1 << 20, n * 4096 * 2) and args[9] == 8
    plan = ex.compile(allgather_nvls(n))
    ex.run(plan, t, stream=s)
    name, args, _ = last(ex)
    block = 4096 * 2
    assert name == 'push_blocks' and args[0] == t.data_ptr() + rank * block and args[1] is True and args[3] == 5000
    assert args[4] == 1 << 20 and args[5] == block
    plan = ex.compile(reduce_scatter_nvls(n, 2))
    out = ex.run(plan, t, stream=s)[rank]
    assert out.numel() == 4096 and last(ex)[0] == 'twoshot_allreduce' and last(ex)[1][-1] == out.data_ptr()
    assert ex.last_algorithm == 'in-switch reduce_scatter'
    # gather-type in-switch programs need registered memory (the all-reduce stages ordinary tensors through registered
    # slices, which needs a GPU); every in-switch program needs a multicast window
    with pytest.raises(PlanError):
        ex.run(ex.compile(allgather_nvls(n)), torch.zeros(n * 4096, dtype=torch.bfloat16), stream=s)
    plain = Executor(FakeComm(multicast=False))
    with pytest.raises(PlanError):
        plain.run(plain.compile(allgather_nvls(n)), plain.comm.symmetric(n * 4096, torch.bfloat16), stream=s)
    # the all-reduce program still runs there: the same two-shot kernel on peer loads and stores (no multicast window)
    plain.run(plain.compile(allreduce_nvls(n)), plain.comm.symmetric(n * 4096, torch.bfloat16), stream=s)
    assert last(plain)[0] == 'twoshot_allreduce' and last(plain)[1][1] == 0


def test_two_ranks_prefer_peer_loads_and_large_one_shot_blocks():
    ex = Executor(FakeComm(world=2, rank=1))
    s = FakeStream()
    assert ex.comm.ll_max_bytes == 2 << 20
    t = ex.comm.symmetric(8 << 20, torch.bfloat16)
    ex.all_reduce(t, stream=s)
    assert last(ex)[0] == 'twoshot_allreduce' and last(ex)[1][1] == 0            # peer loads in rank order on 2 GPUs
    out = ex.comm.symmetric(2 * (256 << 10), torch.float32)
    ex.all_gather(out, torch.zeros(256 << 10), stream=s)                         # 1 MB blocks still go one-shot
    assert last(ex)[0] == 'oneshot'
