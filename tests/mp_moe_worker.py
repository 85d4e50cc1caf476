"""Multi-process worker for the fused MoE kernels (run under torchrun): numerics against a plain
PyTorch fp32 reference; with ``--bench`` the 4096-token / 64-expert / top-2 configuration against an
NCCL all_to_all + torch.matmul pipeline."""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from msccl.ops import check_gemm_errors  # noqa: E402
from msccl.ops.moe import FusedMoE, route_top_k  # noqa: E402
from msccl.runtime import Communicator  # noqa: E402


def timed(fn, iters, warmup=2):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) / iters], device='cuda', dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def make_weights(le, ffn, hidden, seed):
    gen = torch.Generator(device='cuda').manual_seed(seed)
    wg = (torch.randn(le, ffn, hidden, device='cuda', generator=gen) * 0.02).bfloat16()
    wu = (torch.randn(le, ffn, hidden, device='cuda', generator=gen) * 0.02).bfloat16()
    wd = (torch.randn(le, hidden, ffn, device='cuda', generator=gen) * 0.02).bfloat16()
    return wg, wu, wd


def check(comm, rank, n, tokens=256, hidden=512, ffn=512, le=2, calls=3, pair=True):
    num_experts = le * n
    moe = FusedMoE(comm, tokens, hidden, ffn, num_experts, topk=2, capacity_factor=3.0, comm_ctas=4)
    assert moe.pair, 'CTA pairs are the default'
    moe.pair = pair
    wg, wu, wd = make_weights(le, ffn, hidden, 10 + rank)
    wgu, wdn = moe.pack_weights(wg, wu, wd)
    all_wg = [torch.empty_like(wg) for _ in range(n)]
    all_wu = [torch.empty_like(wu) for _ in range(n)]
    all_wd = [torch.empty_like(wd) for _ in range(n)]
    dist.all_gather(all_wg, wg), dist.all_gather(all_wu, wu), dist.all_gather(all_wd, wd)
    WG, WU, WD = torch.cat(all_wg).float(), torch.cat(all_wu).float(), torch.cat(all_wd).float()
    gen = torch.Generator(device='cuda').manual_seed(77 + rank)
    for call in range(calls):
        x = torch.randn(tokens, hidden, device='cuda', generator=gen).bfloat16()
        logits = torch.randn(tokens, num_experts, device='cuda', generator=gen)
        experts, weights = route_top_k(logits, 2)
        if call % 2 == 0:
            # routing in this package's own kernel: the same experts in the same order, the same weights
            dev_experts, dev_weights = moe.route(logits)
            assert torch.equal(dev_experts.long(), experts), ('route ids', call)
            assert (dev_weights - weights).abs().max().item() < 1e-5, ('route weights', call)
            y = moe.forward(x, dev_experts, dev_weights, wgu, wdn)
        else:
            y = moe.forward(x, experts, weights, wgu, wdn)
        check_gemm_errors()
        # the sort the dispatch kernel read: stable by expert
        flat = experts.reshape(-1)
        assert torch.equal(moe._sorted.long(), torch.argsort(flat, stable=True)), ('sorted copies', call)
        start = torch.zeros(num_experts + 1, dtype=torch.long, device='cuda')
        start[1:] = torch.cumsum(torch.bincount(flat, minlength=num_experts), 0)
        assert torch.equal(moe._start.long(), start), ('expert prefix', call)
        want = torch.zeros(tokens, hidden, device='cuda')
        xf = x.float()
        for e in range(num_experts):
            for k in range(2):
                sel = (experts[:, k] == e).nonzero().flatten()
                if sel.numel() == 0:
                    continue
                hh = torch.nn.functional.silu(xf[sel] @ WG[e].t()) * (xf[sel] @ WU[e].t())
                want[sel] += weights[sel, k].unsqueeze(1) * (hh.bfloat16().float() @ WD[e].t())
        err = (y.float() - want).abs().max().item()
        assert err <= 3e-2 * want.abs().max().item() + 1e-3, ('moe', call, err, want.abs().max().item())
    dist.barrier()


def bench(comm, rank, n, iters):
    tokens, hidden, ffn, le, topk = 4096, 4096, 14336, 8, 2
    num_experts = le * n
    moe = FusedMoE(comm, tokens, hidden, ffn, num_experts, topk=topk, capacity_factor=1.5)
    wg, wu, wd = make_weights(le, ffn, hidden, 3 + rank)
    wgu, wdn = moe.pack_weights(wg, wu, wd)
    gen = torch.Generator(device='cuda').manual_seed(5 + rank)
    x = torch.randn(tokens, hidden, device='cuda', generator=gen).bfloat16()
    logits = torch.randn(tokens, num_experts, device='cuda', generator=gen)
    experts, weights = route_top_k(logits, topk)
    y = torch.empty_like(x)
    t_fused = timed(lambda: moe.forward(x, experts, weights, wgu, wdn, out=y), iters)
    check_gemm_errors()

    # baseline: NCCL all_to_all_single (variable splits) + per-expert torch.matmul + all_to_all back
    wgu_plain = torch.cat([wg, wu], dim=1)          # [le, 2*ffn, hidden]

    def pipeline():
        flat = experts.reshape(-1)
        order = torch.argsort(flat, stable=True)
        counts = torch.bincount(flat, minlength=num_experts)
        send_rows = x[order // topk]
        in_counts = torch.empty_like(counts)
        dist.all_to_all_single(in_counts, counts)
        send_splits = counts.view(n, le).sum(1).tolist()
        recv_splits = in_counts.view(n, le).sum(1).tolist()
        recv = torch.empty(sum(recv_splits), hidden, device='cuda', dtype=torch.bfloat16)
        dist.all_to_all_single(recv, send_rows, recv_splits, send_splits)
        # rows arrive grouped by source then expert: regroup by expert
        per_src = in_counts.view(n, le)
        expert_of_row = torch.repeat_interleave(torch.arange(le, device='cuda').repeat(n), per_src.reshape(-1))
        perm = torch.argsort(expert_of_row, stable=True)
        grouped = recv[perm]
        out_rows = torch.empty_like(grouped)
        bounds = torch.cumsum(per_src.sum(0), 0).tolist()
        lo = 0
        for e in range(le):
            hi = bounds[e]
            if hi > lo:
                gu = grouped[lo:hi] @ wgu_plain[e].t()
                hh = torch.nn.functional.silu(gu[:, :ffn]) * gu[:, ffn:]
                out_rows[lo:hi] = hh @ wd[e].t()
            lo = hi
        back = torch.empty_like(recv)
        back[perm] = out_rows
        ret = torch.empty_like(send_rows)
        dist.all_to_all_single(ret, back, send_splits, recv_splits)
        res = torch.zeros(tokens * topk, hidden, device='cuda', dtype=torch.bfloat16)
        res[order] = ret
        return (res.view(tokens, topk, hidden).float() * weights.unsqueeze(-1)).sum(1).bfloat16()

    t_pipe = timed(pipeline, max(2, iters // 2))
    want = pipeline()
    err = (y.float() - want.float()).abs().max().item()
    flops = 3 * 2.0 * tokens * topk * hidden * ffn
    if rank == 0:
        print('FUSED_MOE_BENCH ' + json.dumps({
            'n_gpus': n, 'tokens_per_gpu': tokens, 'hidden': hidden, 'ffn': ffn, 'experts': num_experts, 'topk': topk,
            'fused_us': round(t_fused * 1e3, 1), 'nccl_torch_us': round(t_pipe * 1e3, 1),
            'fused_tflops_per_gpu': round(flops / t_fused / 1e9, 1), 'fused_tokens_per_s': round(n * tokens / (t_fused * 1e-3)),
            'pipeline_tokens_per_s': round(n * tokens / (t_pipe * 1e-3)), 'max_abs_diff_vs_pipeline': round(err, 4)}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--bench', action='store_true')
    ap.add_argument('--iters', type=int, default=6)
    args = ap.parse_args()
    local = int(os.environ['LOCAL_RANK'])
    torch.cuda.set_device(local)
    dist.init_process_group('nccl', device_id=torch.device('cuda', local))
    rank, n = dist.get_rank(), dist.get_world_size()
    comm = Communicator.from_process_group(fifo_bytes=16 << 20, arena_bytes=(1024 << 20) if args.bench else (64 << 20))
    check(comm, rank, n)
    check(comm, rank, n, tokens=320, calls=2)                  # an odd number of row tiles per expert: half-empty pairs
    check(comm, rank, n, pair=False, calls=2)                  # the single-CTA kernels
    if rank == 0:
        print('FUSED_MOE_OK', flush=True)
    if args.bench:
        bench(comm, rank, n, args.iters)
    comm.close()
    dist.destroy_process_group()


if __name__ == '__main__':
    main()
