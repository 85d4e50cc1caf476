"""Step traces of the interpreter kernel (``Executor.run(trace=True)`` / ``last_trace()``) in the Trace Event
format that chrome://tracing and Perfetto read: one process per rank, one thread per threadblock, one slice per
step, the time a step spent waiting, moving data and signalling in its arguments.

The reference has no runtime and therefore no step trace; what it offers for looking at a program is the
instruction DAG drawing of ``msccl/language/visualize.py`` (dead code there), which shows order, not time.
"""
import json


def to_chrome_trace(rows, name='msccl program'):
    """``rows``: dicts with rank, tb, step, type, start_ns, end_ns, wait_ns, move_ns, signal_ns (all iterations of a
    step together: first start to last end).  Returns the dict to be dumped as JSON."""
    events = []
    seen_ranks, seen_tbs = set(), set()
    for r in rows:
        rank, tb = int(r['rank']), int(r['tb'])
        if rank not in seen_ranks:
            seen_ranks.add(rank)
            events.append({'ph': 'M', 'name': 'process_name', 'pid': rank, 'args': {'name': f'rank {rank}'}})
        if (rank, tb) not in seen_tbs:
            seen_tbs.add((rank, tb))
            events.append({'ph': 'M', 'name': 'thread_name', 'pid': rank, 'tid': tb, 'args': {'name': f'threadblock {tb}'}})
        start, end = int(r['start_ns']), int(r['end_ns'])
        events.append({'ph': 'X', 'name': f"{r['step']}: {r['type']}", 'cat': r['type'], 'pid': rank, 'tid': tb,
                       'ts': start / 1e3, 'dur': max(end - start, 0) / 1e3,
                       'args': {'wait_us': int(r.get('wait_ns', 0)) / 1e3, 'move_us': int(r.get('move_ns', 0)) / 1e3,
                                'signal_us': int(r.get('signal_ns', 0)) / 1e3}})
    return {'traceEvents': events, 'displayTimeUnit': 'ns', 'otherData': {'program': name}}


def summarize(rows):
    """Per step type: how many (threadblock, step) records, and the mean microseconds spent waiting, moving and
    signalling - the first thing to look at when a program is slower than expected."""
    acc = {}
    for r in rows:
        a = acc.setdefault(r['type'], [0, 0, 0, 0])
        a[0] += 1
        a[1] += int(r.get('wait_ns', 0))
        a[2] += int(r.get('move_ns', 0))
        a[3] += int(r.get('signal_ns', 0))
    return {t: {'records': c, 'wait_us': round(w / c / 1e3, 2), 'move_us': round(m / c / 1e3, 2), 'signal_us': round(s / c / 1e3, 2)}
            for t, (c, w, m, s) in sorted(acc.items())}


def write(rows, path, name='msccl program'):
    """JSON lines (one record per row) unless ``path`` ends in ``.json``: then one Trace Event document."""
    path = str(path)
    with open(path, 'w') as f:
        if path.endswith('.json'):
            json.dump(to_chrome_trace(rows, name), f)
        else:
            for rec in rows:
                f.write(json.dumps(rec) + '\n')
