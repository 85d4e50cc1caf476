"""Static checks on lowered programs.

``check_dependency_cycles`` and ``check_threadblock_ordering`` have parity with reference
``msccl/language/passes.py:8-55``.  ``check_fusion_operands`` closes a gap the reference
leaves open: a fused op forwards the slot it just received into, so the forwarding send
must have read exactly that slot.
"""
import sys


def check_dependency_cycles(tbs):
    """Abort (exit status 1) when the cross-threadblock ``depends`` edges of a rank form a cycle."""
    WHITE, GREY, BLACK = 0, 1, 2
    for rank, rank_tbs in enumerate(tbs):
        colour = {}
        for tbid, tb in rank_tbs.items():
            for root in tb.ops:
                if colour.get(root, WHITE) != WHITE:
                    continue
                stack = [(root, iter(root.depends))]
                colour[root] = GREY
                while stack:
                    node, it = stack[-1]
                    dep = next(it, None)
                    if dep is None:
                        colour[node] = BLACK
                        stack.pop()
                        continue
                    state = colour.get(dep, WHITE)
                    if state == GREY:
                        print(f'Cyclic dependency in rank {rank} threadblock {tbid} at {root}')
                        for entry, _ in stack:
                            print('  ', entry)
                        sys.exit(1)
                    if state == WHITE:
                        colour[dep] = GREY
                        stack.append((dep, iter(dep.depends)))


def check_threadblock_ordering(dag):
    """Sends from one threadblock to a peer threadblock must be received in the order sent."""
    for rank in range(dag.num_ranks):
        for tb in dag.tbs[rank].values():
            last_seen = {}     # receiving tb id -> last matched receive
            for op in tb.ops:
                if not op.is_send():
                    continue
                match = op.recv_match
                if match.is_recv():
                    assert op.dst.rank == match.rank, "Bug in MSCCLang: Sends don't match receives"
                earlier = last_seen.get(match.tb)
                if earlier is not None and match.step <= earlier.step:
                    print('Offending Steps', match.step, earlier.step)
                    print('Sending tb')
                    for o in tb.ops:
                        print(f'{o.step}: Recv step: {o.recv_match.step if o.is_send() else -1} {o} '
                              f'priority:{(o.chunk_step, o.priority, o.dst.index)}')
                    print('Receiving tb')
                    for o in dag.tbs[match.rank][match.tb].ops:
                        print(f'{o.step}: {o} priority:{(o.chunk_step, o.priority, o.dst.index)}')
                    raise AssertionError(f'Rank {op.rank} sends op1 then op2 but {match.rank} '
                                         f'receives op2 then op1')
                last_seen[match.tb] = match
