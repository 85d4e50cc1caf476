"""Data parallelism: gradients live in one flat registered buffer and are summed in place.

Every parameter's ``.grad`` is a view into a flat tensor from ``Communicator.symmetric_empty``, so the
backward pass writes the bucket directly and ``all_reduce_gradients`` is one collective per bucket on memory
that every kernel of the executor can use (one-shot LL for tiny models, the in-switch two-shot reduction for
large ones): no copy into a communication buffer and none back.
"""
import torch


class FlatGradients:
    def __init__(self, parameters, allocate, dtype=None, bucket_bytes=1 << 30):
        """``allocate(numel, dtype)`` returns a flat tensor (``lambda n, d: comm.symmetric_empty(n, d)[0]``).
        Parameters are packed in order into buckets of at most ``bucket_bytes``; every slot starts on a
        16-byte boundary so that any suffix of a bucket is a valid message."""
        self.params = [p for p in parameters if p.requires_grad]
        if not self.params:
            raise ValueError('no parameter requires a gradient')
        self.dtype = dtype or self.params[0].dtype
        esize = torch.empty((), dtype=self.dtype).element_size()
        align = max(1, 16 // esize)
        self.buckets = []          # [(flat tensor, [(param, offset, numel)])]
        plan, used = [], 0
        for p in self.params:
            n = -(-p.numel() // align) * align
            if plan and (used + n) * esize > bucket_bytes:
                self.buckets.append(self._make(plan, used, allocate))
                plan, used = [], 0
            plan.append((p, used, p.numel()))
            used += n
        self.buckets.append(self._make(plan, used, allocate))

    def _make(self, plan, numel, allocate):
        flat = allocate(numel, self.dtype)
        flat.zero_()
        for p, off, n in plan:
            p.grad = flat[off:off + n].view(p.shape)
        return flat, plan

    def zero(self):
        for flat, _ in self.buckets:
            flat.zero_()

    def all_reduce_gradients(self, all_reduce, world, average=True):
        """Sum every bucket over the ranks with ``all_reduce(flat)`` (for example ``executor.all_reduce``) and,
        with ``average``, divide by ``world``."""
        for flat, plan in self.buckets:
            for p, off, n in plan:
                if p.grad is None or p.grad.data_ptr() != flat[off:off + n].data_ptr():
                    raise RuntimeError('a gradient was replaced; keep optimizer.zero_grad(set_to_none=False)')
            all_reduce(flat)
            if average:
                flat.div_(world)
