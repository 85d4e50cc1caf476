"""Instruction fusion: fold a receive and the send that forwards the same data into one op.

    rrc ; send ; (slot later overwritten by a recv)  ->  rrs   (reduced value is only forwarded)
    rrc ; send                                       ->  rrcs
    recv ; send                                      ->  rcs

A pair fuses only when both ops were placed on the same threadblock and channel, move the
same number of chunks, and name the same destination buffer and index.  The fused op keeps
the receive's source and takes over the send's remote destination.

Parity: reference ``msccl/language/rank_dag.py:12-28,209-251``
(expected results pinned by reference ``tests/test_language.py:188-202``).
"""
from msccl.language.mscclir import Instruction, link


def _compatible(first, second):
    return (first.tb == second.tb and first.channel == second.channel
            and first.cnt() == second.cnt()
            and first.dst.buffer == second.dst.buffer and first.dst.index == second.dst.index)


def _splice_out(op):
    """Remove ``op`` from the DAG, connecting its predecessors to its successors."""
    for p in op.prev:
        p.next.remove(op)
    for n in op.next:
        n.prev.remove(op)
    for p in op.prev:
        for n in op.next:
            link(p, n)


def _absorb_send(receiver, send, fused_inst, dag):
    receiver.inst = fused_inst
    receiver.dst = send.dst
    receiver.recv_match = send.recv_match
    send.recv_match.send_match = receiver
    _splice_out(send)
    dag.all_ops.remove(send)


def _try_reduce_forward(op, dag):
    if op.inst != Instruction.recv_reduce_copy or len(op.next) != 1:
        return False
    send = op.next[0]
    if send.inst != Instruction.send or not _compatible(op, send):
        return False
    overwritten = len(send.next) == 1 and send.next[0].inst is Instruction.recv
    _absorb_send(op, send, Instruction.recv_reduce_send if overwritten
                 else Instruction.recv_reduce_copy_send, dag)
    return True


def _try_copy_forward(op, dag):
    if op.inst != Instruction.recv:
        return False
    for send in op.next:
        if send.inst == Instruction.send and _compatible(op, send):
            _absorb_send(op, send, Instruction.recv_copy_send, dag)
            return True
    return False


def fuse_instructions(dag):
    """Run both rewrite families to a fixed point, reductions first."""
    for attempt in (_try_reduce_forward, _try_copy_forward):
        changed = True
        while changed:
            changed = False
            for op in list(dag.all_ops):
                if attempt(op, dag):
                    changed = True
