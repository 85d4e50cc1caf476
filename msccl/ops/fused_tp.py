"""Fused tensor-parallel GEMMs: all-gather -> GEMM (optionally with SwiGLU) and GEMM -> reduce-scatter,
each as ONE sm_100a kernel that overlaps NVLink traffic with tcgen05 tiles (``csrc/fused_tp.cu``).

Sequence-parallel convention: activations enter and leave sharded by tokens
(``[tokens_per_rank, hidden]`` per rank); weights are sharded along the FFN dimension.

The chunk movement of both kernels is stated as MSCCLang programs in ``msccl.ops.schedules``
(``all_gather_blocks``, ``reduce_scatter_blocks``: one chunk per 128-row block), where it is checked
symbolically and run on the CPU interpreter.  The compiled programs are lowered into row-block order tables
(``msccl.ops.schedules.fused_tp_tables``) which the kernels take as arguments: the GEMM tiles walk the row
blocks in that order.
"""
import os

import torch

from msccl.ops.gemm import _errors
from msccl.runtime.comm import Communicator


class FusedTensorParallel:
    """Holds the symmetric buffers of the two fused kernels for fixed shapes."""

    def __init__(self, comm: Communicator, tokens_per_rank: int, hidden: int, comm_ctas: int = 8):
        if comm.emulated_mode:
            raise ValueError('the fused kernels need one process per GPU')
        if tokens_per_rank % 128 or hidden % 256:
            raise ValueError('tokens_per_rank must be a multiple of 128 and hidden a multiple of 256')
        self.comm = comm
        self.n = comm.world
        self.rows = tokens_per_rank
        self.hidden = hidden
        self.comm_ctas = int(os.environ.get('MSCCL_COMM_CTAS', comm_ctas))      # CTAs that push the local shard to the peers
        all_rows = self.n * tokens_per_rank
        self.gathered_bytes = all_rows * hidden * 2
        _, self.gathered_off = comm.symmetric_empty(2 * all_rows * hidden, torch.bfloat16)
        _, self.partial_off = comm.symmetric_empty(2 * self.n * tokens_per_rank * hidden, torch.bfloat16)
        self.sms = comm.native.sm_count()
        self.launches = 0
        self.tuning = int(os.environ.get('MSCCL_AG_TUNING', '0'))
        self.grid = int(os.environ.get('MSCCL_AG_GRID', '0'))
        self.reduce_ctas = int(os.environ.get('MSCCL_RS_REDUCE_CTAS', '12'))
        # CTA pairs (tcgen05 cta_group::2, 256 x 256 tiles) whenever the row blocks pair up; MSCCL_FUSED_PAIR=0: single CTAs
        self.pair = (os.environ.get('MSCCL_FUSED_PAIR', '1') != '0' and (self.n * (tokens_per_rank // 128)) % 2 == 0
                     and self.comm_ctas % 2 == 0 and self.reduce_ctas % 2 == 0)
        self.set_schedule()

    def set_schedule(self, ag_channels=1, rs_channels=1):
        """Install the row-block order tables lowered from the schedule programs (``msccl.ops.schedules``); the
        channel counts select among the programs: with c channels a round of the lowering holds c blocks per peer."""
        from msccl.ops.schedules import fused_tp_tables
        ag, rs, red = fused_tp_tables(self.n, self.rows // 128, self.comm.rank, ag_channels, rs_channels)
        dev = f'cuda:{self.comm.device}'
        self.ag_order = torch.tensor(ag, dtype=torch.int32, device=dev)
        self.rs_order = torch.tensor(rs, dtype=torch.int32, device=dev)
        self.reduce_order = torch.tensor(red, dtype=torch.int32, device=dev)

    def all_gather_gemm(self, x_local, weight, epilogue='none', out=None, stream=None):
        """``epilogue(gather(x_local) @ weight.T)``: x_local [rows, hidden], weight [N, hidden] -> [n*rows, N (or N/2)]."""
        c = self.comm
        assert x_local.shape == (self.rows, self.hidden) and x_local.is_contiguous() and x_local.dtype == torch.bfloat16
        n_out, k = weight.shape
        assert k == self.hidden and weight.stride(1) == 1 and n_out % 256 == 0
        swiglu = epilogue == 'swiglu'
        cols = n_out // 2 if swiglu else n_out
        if out is None:
            out = torch.empty(self.n * self.rows, cols, dtype=torch.bfloat16, device=x_local.device)
        stream_h = (stream or torch.cuda.current_stream()).cuda_stream
        c.native.ag_gemm(x_local.data_ptr(), weight.data_ptr(), out.data_ptr(), self.rows, n_out, k, weight.stride(0),
                         out.stride(0), c.rank, self.n, self.comm_ctas, c.dev_heap_bases, list(c.heap_ptrs), c.off_fused,
                         c.mc_base, self.gathered_off, self.gathered_bytes, _errors(x_local.device).data_ptr(),
                         1 if swiglu else 0, self.grid or (0 if self.pair else self.sms), self.tuning, self.ag_order.data_ptr(),
                         stream_h, pair=self.pair)
        self.launches += 1
        return out

    def gemm_reduce_scatter(self, a, weight, out=None, stream=None):
        """``reduce_scatter(a @ weight.T)``: a [n*rows, K_shard], weight [hidden, K_shard] -> this rank's [rows, hidden]."""
        c = self.comm
        m, k = a.shape
        assert m == self.n * self.rows and a.stride(1) == 1 and a.dtype == torch.bfloat16
        assert weight.shape == (self.hidden, k) and weight.stride(1) == 1 and k % 64 == 0
        if out is None:
            out = torch.empty(self.rows, self.hidden, dtype=torch.bfloat16, device=a.device)
        assert out.is_contiguous()
        stream_h = (stream or torch.cuda.current_stream()).cuda_stream
        c.native.gemm_rs(a.data_ptr(), weight.data_ptr(), out.data_ptr(), self.rows, self.hidden, k, a.stride(0),
                         weight.stride(0), c.rank, self.n, c.dev_heap_bases, list(c.heap_ptrs), c.off_fused, self.partial_off,
                         _errors(a.device).data_ptr(), 0 if self.pair else self.sms, self.rs_order.data_ptr(),
                         self.reduce_order.data_ptr(), min(self.reduce_ctas, self.sms - 1), stream_h, pair=self.pair)
        self.launches += 1
        return out

    # ---------------------------------------------------------------- block-scaled fp8 (OCP MX) operands
    @property
    def mx_gate_up_tile(self):
        """Interleave width of gate and up rows the fp8 SwiGLU epilogue expects (``interleave_gate_up(..., tile=...)``):
        256 on CTA pairs (128 gate + 128 up columns per tile), 128 on single CTAs."""
        return 256 if self.pair else 128

    def all_gather_gemm_mxfp8(self, xq_local, sfx_packed, wq, sfw_packed, epilogue='none', out=None, stream=None):
        """The all-gather -> GEMM kernel on MX fp8 operands: ``xq_local`` [rows, hidden] e4m3 with its scales packed by
        ``msccl.ops.gemm.pack_mx_scales(scales, row_multiple=128)``, ``wq`` [N, hidden] e4m3 with packed scales.  What
        crosses NVLink is the fp8 block plus its scale blocks.  Returns bf16 ``[n*rows, N]`` (``N/2`` with ``swiglu``;
        gate and up rows interleaved with ``interleave_gate_up(w_gate, w_up, tile=self.mx_gate_up_tile)``).  Runs on
        CTA pairs (256 x 256 tiles) when the row blocks pair up and N is a multiple of 256."""
        c = self.comm
        k = self.hidden
        assert xq_local.shape == (self.rows, k) and xq_local.is_contiguous() and xq_local.dtype == torch.float8_e4m3fn
        n_out, kw = wq.shape
        assert kw == k and wq.stride(1) == 1 and wq.dtype == torch.float8_e4m3fn and n_out % 128 == 0 and k % 128 == 0
        blocks, k_blocks = self.rows // 128, k // 128
        assert sfx_packed.dtype == torch.uint8 and sfx_packed.numel() == blocks * k_blocks * 512 and sfx_packed.is_contiguous()
        assert sfw_packed.dtype == torch.uint8 and sfw_packed.numel() >= (n_out // 128) * k_blocks * 512
        swiglu = epilogue == 'swiglu'
        cols = n_out // 2 if swiglu else n_out
        if out is None:
            out = torch.empty(self.n * self.rows, cols, dtype=torch.bfloat16, device=xq_local.device)
        per_parity = -(-(self.n * self.rows * k + self.n * blocks * k_blocks * 512) // 1024) * 1024
        assert per_parity <= self.gathered_bytes
        stream_h = (stream or torch.cuda.current_stream()).cuda_stream
        pair = self.pair and n_out % 256 == 0 and self.comm_ctas % 2 == 0
        assert pair or not (swiglu and self.pair), 'with the SwiGLU epilogue on CTA pairs N must be a multiple of 256'
        c.native.ag_gemm_mxfp8(xq_local.data_ptr(), sfx_packed.data_ptr(), wq.data_ptr(), sfw_packed.data_ptr(), out.data_ptr(),
                               self.rows, n_out, k, wq.stride(0), out.stride(0), c.rank, self.n, self.comm_ctas,
                               c.dev_heap_bases, list(c.heap_ptrs), c.off_fused, c.mc_base, self.gathered_off, per_parity,
                               _errors(xq_local.device).data_ptr(), 1 if swiglu else 0, self.grid or (0 if pair else self.sms),
                               self.ag_order.data_ptr(), stream_h, pair)
        self.launches += 1
        return out

    def gemm_reduce_scatter_mxfp8(self, aq, sfa_packed, wq, sfw_packed, out=None, stream=None):
        """The GEMM -> reduce-scatter kernel on MX fp8 operands: ``aq`` [n*rows, K_shard] e4m3 (scales packed with
        ``row_multiple=128``), ``wq`` [hidden, K_shard] e4m3.  The partial sums travel and are added up as bf16, as
        in the bf16 kernel.  Returns this rank's bf16 ``[rows, hidden]``."""
        c = self.comm
        m, k = aq.shape
        assert m == self.n * self.rows and aq.stride(1) == 1 and aq.dtype == torch.float8_e4m3fn and k % 128 == 0
        assert wq.shape == (self.hidden, k) and wq.stride(1) == 1 and wq.dtype == torch.float8_e4m3fn and self.hidden % 128 == 0
        assert sfa_packed.dtype == torch.uint8 and sfa_packed.numel() == (m // 128) * (k // 128) * 512
        assert sfw_packed.dtype == torch.uint8 and sfw_packed.numel() >= (self.hidden // 128) * (k // 128) * 512
        if out is None:
            out = torch.empty(self.rows, self.hidden, dtype=torch.bfloat16, device=aq.device)
        assert out.is_contiguous()
        stream_h = (stream or torch.cuda.current_stream()).cuda_stream
        pair = self.pair and self.hidden % 256 == 0
        c.native.gemm_rs_mxfp8(aq.data_ptr(), sfa_packed.data_ptr(), wq.data_ptr(), sfw_packed.data_ptr(), out.data_ptr(),
                               self.rows, self.hidden, k, aq.stride(0), wq.stride(0), c.rank, self.n, c.dev_heap_bases,
                               list(c.heap_ptrs), c.off_fused, self.partial_off, _errors(aq.device).data_ptr(),
                               0 if pair else self.sms, self.rs_order.data_ptr(), self.reduce_order.data_ptr(),
                               min(self.reduce_ctas, self.sms - 1), stream_h, pair)
        self.launches += 1
        return out
