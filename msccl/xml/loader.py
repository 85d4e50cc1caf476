"""Typed in-memory form of MSCCL-IR XML.

Accepts the files written by both reference writers (MSCCLang ``msccl/language/ir.py:319-391``
and ncclize ``msccl/ncclize.py:658-722``) and by this package.  Schema::

    <algo name proto nchannels nchunksperloop ngpus coll inplace>
      <gpu id i_chunks o_chunks s_chunks>
        <tb id send recv chan>
          <step s type srcbuf srcoff dstbuf dstoff cnt depid deps hasdep/>

For send-type steps ``src`` is a local slot and ``dst`` the slot on the receiving peer; for
receive-type steps ``src`` is the slot on the sending peer and ``dst`` is local.

Also loads the ``<msccl_algos><load path minBytes maxBytes proto/></msccl_algos>`` plan table
that ``msccl.init`` writes (reference ``msccl/autosynth/__init__.py:75-94``).
"""
import math
import xml.etree.ElementTree as ET
from dataclasses import dataclass, field
from typing import List

STEP_TYPES = ('nop', 's', 'r', 'rcs', 'rrs', 'rrc', 'rrcs', 'cpy', 're', 'mmr', 'mmb', 'mmar', 'bar')
SEND_TYPES = frozenset({'s', 'rcs', 'rrs', 'rrcs'})
RECV_TYPES = frozenset({'r', 'rcs', 'rrs', 'rrc', 'rrcs'})
REDUCING_TYPES = frozenset({'rrs', 'rrc', 'rrcs', 're'})
PROTOCOLS = ('Simple', 'LL', 'LL128')


@dataclass
class StepIR:
    s: int
    type: str
    srcbuf: str
    srcoff: int
    dstbuf: str
    dstoff: int
    cnt: int
    depid: int
    deps: int
    hasdep: bool

    def is_send(self):
        return self.type in SEND_TYPES

    def is_recv(self):
        return self.type in RECV_TYPES


@dataclass
class TbIR:
    id: int
    send: int
    recv: int
    chan: int
    steps: List[StepIR] = field(default_factory=list)


@dataclass
class GpuIR:
    id: int
    i_chunks: int
    o_chunks: int
    s_chunks: int
    tbs: List[TbIR] = field(default_factory=list)


@dataclass
class AlgoIR:
    name: str
    proto: str
    nchannels: int
    nchunksperloop: int
    ngpus: int
    coll: str
    inplace: bool
    gpus: List[GpuIR] = field(default_factory=list)

    def num_threadblocks(self):
        return sum(len(g.tbs) for g in self.gpus)

    def num_steps(self):
        return sum(len(tb.steps) for g in self.gpus for tb in g.tbs)

    def max_count(self):
        return max((st.cnt for g in self.gpus for tb in g.tbs for st in tb.steps), default=1)

    def max_tbs_per_gpu(self):
        return max((len(g.tbs) for g in self.gpus), default=0)

    # ---- buffer aliasing of the in-place collectives --------------------------------
    def resolve(self, rank, buf, off):
        """Map (buffer, chunk offset) to the buffer that physically holds it on ``rank``.
        In-place all-reduce: output is input.  In-place all-gather: input chunk k is output chunk
        ``rank*cf + k``.  In-place reduce-scatter: output chunk k is input chunk ``rank*cf + k``."""
        if not self.inplace:
            return buf, off
        if self.coll == 'allreduce' and buf == 'o':
            return 'i', off
        if self.coll == 'allgather' and buf == 'i':
            return 'o', off + rank * (self.gpus[rank].o_chunks // self.ngpus)
        if self.coll == 'reduce_scatter' and buf == 'o':
            return 'i', off + rank * (self.gpus[rank].i_chunks // self.ngpus)
        if self.coll == 'alltoall' and buf == 'o':
            return 'i', off
        return buf, off


def _int(elem, key, default=None):
    raw = elem.get(key)
    if raw is None:
        if default is None:
            raise ValueError(f'<{elem.tag}> lacks attribute {key!r}')
        return default
    return int(raw)


def load_xml(text: str) -> AlgoIR:
    root = ET.fromstring(text)
    if root.tag != 'algo':
        raise ValueError(f'expected <algo>, found <{root.tag}>')
    algo = AlgoIR(name=root.get('name', ''), proto=root.get('proto', 'Simple'),
                  nchannels=_int(root, 'nchannels'), nchunksperloop=_int(root, 'nchunksperloop', 0),
                  ngpus=_int(root, 'ngpus'), coll=root.get('coll', 'custom'),
                  inplace=root.get('inplace', '0') == '1')
    for g in root.findall('gpu'):
        gpu = GpuIR(_int(g, 'id'), _int(g, 'i_chunks'), _int(g, 'o_chunks'), _int(g, 's_chunks'))
        for t in g.findall('tb'):
            tb = TbIR(_int(t, 'id'), _int(t, 'send'), _int(t, 'recv'), _int(t, 'chan'))
            for e in list(t.findall('step')) + list(t.findall('op')):
                tb.steps.append(StepIR(
                    s=_int(e, 's', _int(e, 'step', -1)), type=e.get('type'),
                    srcbuf=e.get('srcbuf', e.get('buf', 'i')), srcoff=_int(e, 'srcoff', _int(e, 'off', -1)),
                    dstbuf=e.get('dstbuf', e.get('buf', 'o')), dstoff=_int(e, 'dstoff', _int(e, 'off', -1)),
                    cnt=_int(e, 'cnt', 1), depid=_int(e, 'depid', -1), deps=_int(e, 'deps', -1),
                    hasdep=e.get('hasdep', '0') == '1'))
            tb.steps.sort(key=lambda st: st.s)
            gpu.tbs.append(tb)
        gpu.tbs.sort(key=lambda tb: tb.id)
        algo.gpus.append(gpu)
    algo.gpus.sort(key=lambda g: g.id)
    return algo


def load_xml_file(path) -> AlgoIR:
    with open(path) as f:
        return load_xml(f.read())


@dataclass
class PlanEntry:
    path: str
    min_bytes: int
    max_bytes: float
    proto: str
    algo: AlgoIR = None


def load_plan_table(path, parse_algorithms=True) -> List[PlanEntry]:
    """Read an ``<msccl_algos>`` file; entries keep file order (first match wins at dispatch)."""
    root = ET.parse(path).getroot()
    if root.tag != 'msccl_algos':
        raise ValueError(f'expected <msccl_algos>, found <{root.tag}>')
    entries = []
    for load in root.findall('load'):
        hi = load.get('maxBytes')
        entry = PlanEntry(load.get('path'), int(load.get('minBytes', '0')),
                          math.inf if hi is None else int(hi), load.get('proto', 'Simple'))
        if parse_algorithms:
            entry.algo = load_xml_file(entry.path)
        entries.append(entry)
    return entries
