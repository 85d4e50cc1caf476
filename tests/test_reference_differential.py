"""Differential test of the MSCCLang compiler against the installed reference (``baseline/_ref``): the same program
sources are compiled by both packages and the MSCCL-IR must agree GPU by GPU, threadblock by threadblock, step by
step in type, buffers, offsets and counts.

Two things are left to the compiler and compared more loosely.  A local copy or reduce has no peer, so it may sit
in any threadblock; where several are equally far along the reference takes whichever its ready queue (a heap
whose ties are unordered) happens to yield, this compiler the first: the communication steps of every threadblock
must match exactly, the local steps as a multiset per GPU.  Likewise a step may wait on any of several equivalent
producers, so dependencies are compared by their number per GPU.  Skipped when the reference is not installed."""
import os
import subprocess
import sys
import xml.etree.ElementTree as ET
from collections import Counter

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, 'baseline', '_ref')
SHIMS = os.path.join(ROOT, 'baseline', 'shims')
HELPER = os.path.join(ROOT, 'tests', 'ref_differential_helper.py')
LOCAL = ('cpy', 're', 'nop')

pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, 'msccl')), reason='the reference is not installed')


def _compile_all(pythonpath, out_dir):
    env = {k: v for k, v in os.environ.items() if k != 'PYTHONPATH'}
    env['PYTHONPATH'] = pythonpath
    os.makedirs(out_dir, exist_ok=True)
    run = subprocess.run([sys.executable, HELPER, str(out_dir)], env=env, capture_output=True, text=True, timeout=1500,
                         cwd=str(out_dir))
    assert run.returncode == 0 and 'DONE' in run.stdout, run.stdout[-2000:] + run.stderr[-3000:]
    return {f[:-4]: open(os.path.join(out_dir, f)).read() for f in sorted(os.listdir(out_dir)) if f.endswith('.xml')}


def _structure(text):
    """(header, per GPU: (buffer sizes, [(tb id, send, recv, chan, [step fields])], multiset of dependency edges))."""
    root = ET.fromstring(text[text.index('<algo'):])
    header = {k: root.get(k) for k in ('name', 'proto', 'nchannels', 'nchunksperloop', 'ngpus', 'coll', 'inplace')}
    gpus = []
    for g in sorted(root.findall('gpu'), key=lambda e: int(e.get('id'))):
        tbs, edges = [], Counter()
        for tb in sorted(g.findall('tb'), key=lambda e: int(e.get('id'))):
            steps = []
            for st in sorted(tb.findall('step'), key=lambda e: int(e.get('s'))):
                steps.append(tuple(st.get(k) for k in ('type', 'srcbuf', 'srcoff', 'dstbuf', 'dstoff', 'cnt')))
                if st.get('depid', '-1') != '-1':
                    edges[(tb.get('id'), st.get('depid'), st.get('deps'))] += 1
            tbs.append((tb.get('id'), tb.get('send'), tb.get('recv'), tb.get('chan'), steps))
        gpus.append(((g.get('i_chunks'), g.get('o_chunks'), g.get('s_chunks')), tbs, edges))
    return header, gpus


def test_same_ir_as_the_reference_compiler(tmp_path):
    mine = _compile_all(ROOT, tmp_path / 'mine')
    theirs = _compile_all(os.pathsep.join([SHIMS, REF]), tmp_path / 'ref')
    assert set(mine) == set(theirs) and len(mine) >= 20
    identical = 0
    for name in sorted(mine):
        head_a, gpus_a = _structure(mine[name])
        head_b, gpus_b = _structure(theirs[name])
        assert head_a == head_b, name
        assert len(gpus_a) == len(gpus_b), name
        for r, (ga, gb) in enumerate(zip(gpus_a, gpus_b)):
            assert ga[0] == gb[0], f'{name}: buffer sizes of GPU {r}'
            assert len(ga[1]) == len(gb[1]), f'{name}: threadblocks of GPU {r}'
            local_a, local_b = Counter(), Counter()
            for ta, tb in zip(ga[1], gb[1]):
                assert ta[:4] == tb[:4], f'{name}: GPU {r} threadblock {ta[0]} (id, send, recv, chan)'
                comm_a = [st for st in ta[4] if st[0] not in LOCAL]
                comm_b = [st for st in tb[4] if st[0] not in LOCAL]
                assert comm_a == comm_b, f'{name}: GPU {r} threadblock {ta[0]} communication steps'
                local_a.update(st for st in ta[4] if st[0] in LOCAL)
                local_b.update(st for st in tb[4] if st[0] in LOCAL)
            assert local_a == local_b, f'{name}: local steps of GPU {r}'
            assert sum(ga[2].values()) == sum(gb[2].values()), f'{name}: dependency edges of GPU {r}'
        identical += mine[name].strip() == theirs[name].strip()
    # many programs come out byte for byte the same (11 of 22 when this test was written); the others differ only in
    # the two respects named in the module docstring
    assert identical >= len(mine) // 3, f'only {identical} of {len(mine)} programs are byte-identical'
