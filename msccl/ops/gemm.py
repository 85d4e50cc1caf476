"""tcgen05 GEMM for bf16 on sm_100a: ``D = A @ B.T`` with A ``[M, K]`` and B ``[N, K]`` row-major
(both K-major, the layout of activations and ``nn.Linear`` weights), fp32 accumulation in tensor
memory, bf16 result.  ``epilogue='swiglu'`` fuses ``silu(gate) * up`` where each 256-column tile
of B holds 128 gate rows followed by the 128 matching up rows (see ``interleave_gate_up``).
"""
import os

import torch

from msccl.runtime.native import load

_error_words = {}


class GemmKernelError(RuntimeError):
    pass


def _errors(device):
    key = torch.device(device).index or 0
    if key not in _error_words:
        _error_words[key] = torch.zeros(4, dtype=torch.int32, device=f'cuda:{key}')
    return _error_words[key]


def check_gemm_errors(device=None):
    """Synchronise and raise if a GEMM kernel gave up on one of its bounded waits."""
    device = torch.cuda.current_device() if device is None else device
    torch.cuda.synchronize(device)
    words = _errors(device).tolist()
    if words[0] != 0:
        _errors(device).zero_()
        names = {1: 'operands never arrived (TMA)', 2: 'pipeline stage never freed', 3: 'accumulator hand-off',
                 4: 'peer flag'}
        raise GemmKernelError(f'GEMM kernel timeout: {names.get(words[0], words[0])} (block {words[1]}, role {words[2]}, '
                              f'detail {words[3]})')


def interleave_gate_up(w_gate, w_up, tile=256):
    """Stack gate and up projection weights ``[F, K]`` so that every ``tile`` rows hold ``tile/2`` gate
    rows followed by the ``tile/2`` up rows of the same features (what the SwiGLU epilogue expects)."""
    half = tile // 2
    f, k = w_gate.shape
    assert w_up.shape == (f, k) and f % half == 0
    g = w_gate.reshape(f // half, half, k)
    u = w_up.reshape(f // half, half, k)
    return torch.cat([g, u], dim=1).reshape(2 * f, k).contiguous()


def gemm_bf16(a, b, out=None, epilogue='none', bn=256, max_ctas=0, stream=None, pair=None):
    """``a``: [M, K] bf16, ``b``: [N, K] bf16 (row pitch may exceed K).  Returns [M, N] (or [M, N/2] for swiglu).
    ``pair``: run on CTA pairs (``tcgen05 cta_group::2``, 256 x 256 tiles; needs N % 256 == 0); ``None`` takes
    ``MSCCL_GEMM_PAIR`` (default on) whenever the shape allows it and ``bn`` is 256."""
    assert a.is_cuda and b.is_cuda and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    assert a.dim() == 2 and b.dim() == 2 and a.stride(1) == 1 and b.stride(1) == 1
    m, k = a.shape
    n, kb = b.shape
    assert k == kb, 'inner dimensions differ'
    if k % 64 or n % bn:
        raise ValueError(f'K must be a multiple of 64 and N a multiple of {bn} (got K={k}, N={n})')
    swiglu = epilogue == 'swiglu'
    n_out = n // 2 if swiglu else n
    if out is None:
        out = torch.empty(m, n_out, dtype=torch.bfloat16, device=a.device)
    assert out.shape == (m, n_out) and out.stride(1) == 1 and out.dtype == torch.bfloat16
    stream_h = (stream or torch.cuda.current_stream()).cuda_stream
    if pair is None:
        pair = bn == 256 and n % 256 == 0 and os.environ.get('MSCCL_GEMM_PAIR', '1') == '1'
    if pair:
        if n % 256:
            raise ValueError(f'the two-CTA kernel needs N to be a multiple of 256 (got {n})')
        load().gemm_bf16_2cta(a.data_ptr(), b.data_ptr(), out.data_ptr(), m, n, k, a.stride(0), b.stride(0), out.stride(0),
                              1 if swiglu else 0, _errors(a.device).data_ptr(), (max_ctas + 1) // 2, stream_h)
        return out
    load().gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), m, n, k, a.stride(0), b.stride(0), out.stride(0),
                     1 if swiglu else 0, bn, _errors(a.device).data_ptr(), max_ctas, stream_h)
    return out


# ---------------------------------------------------------------------------- block-scaled fp8
MX_BLOCK = 32          # K elements that share one scale
_E4M3_MAX = 448.0


def quantize_mxfp8(x):
    """Quantise ``x`` [R, K] (K % 32 == 0) to the MX fp8 format: e4m3 values plus one UE8M0 scale byte
    (``2 ** (byte - 127)``) per 32 consecutive K elements of a row, chosen as the smallest power of two
    that brings the block's largest magnitude inside the e4m3 range.  Returns ``(q, scales)`` with
    ``q`` [R, K] float8_e4m3fn and ``scales`` [R, K / 32] uint8."""
    r, k = x.shape
    assert k % MX_BLOCK == 0
    blocks = x.float().reshape(r, k // MX_BLOCK, MX_BLOCK)
    amax = blocks.abs().amax(dim=-1).clamp_min(2.0 ** -120)
    exp = torch.ceil(torch.log2(amax / _E4M3_MAX)).clamp(-127, 127)
    q = (blocks / torch.exp2(exp).unsqueeze(-1)).clamp(-_E4M3_MAX, _E4M3_MAX).reshape(r, k).to(torch.float8_e4m3fn)
    return q, (exp + 127).to(torch.uint8)


def quantize_mxfp8_packed(x, out=None, scales_out=None, stream=None):
    """One-pass CUDA quantisation of a bf16 ``x`` [R, K] (K % 128 == 0): returns ``(q, packed_scales)`` - e4m3 values and
    the UE8M0 scales already in the ``pack_mx_scales(..., row_multiple=128)`` arrangement (rows padded with scale 1.0).
    Same scale rule as ``quantize_mxfp8``."""
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1
    r, k = x.shape
    if k % 128:
        raise ValueError(f'K must be a multiple of 128 (got {k})')
    tiles = -(-r // 128)
    if out is None:
        out = torch.empty(r, k, dtype=torch.float8_e4m3fn, device=x.device)
    if scales_out is None:
        scales_out = (torch.empty if r % 128 == 0 else (lambda *a, **kw: torch.full(*a, fill_value=127, **kw)))(
            (tiles * (k // 128) * 512,), dtype=torch.uint8, device=x.device)
    assert out.is_contiguous() and scales_out.numel() == tiles * (k // 128) * 512
    stream_h = (stream or torch.cuda.current_stream()).cuda_stream
    load().quantize_mxfp8(x.data_ptr(), out.data_ptr(), scales_out.data_ptr(), r, k, x.stride(0), stream_h)
    return out, scales_out


def dequantize_mxfp8(q, scales):
    """fp32 values of a ``quantize_mxfp8`` pair."""
    r, k = q.shape
    s = torch.exp2(scales.float() - 127.0).repeat_interleave(MX_BLOCK, dim=1)
    return q.float() * s


def pack_mx_scales(scales, row_multiple=256):
    """Arrange ``scales`` [R, K / 32] (K % 128 == 0) the way the kernel's tensor-memory copy consumes them:
    one 512-byte block per (128 rows, 128 K elements), byte ``(r % 32) * 16 + (r // 32) * 4 + j`` of a block
    = scale of row ``r`` for K elements ``[32 j, 32 j + 32)``.  Rows are padded to a multiple of
    ``row_multiple`` (256: what the CTA-pair kernel reads; 128 is enough for the single-CTA kernel) with
    the scale 1.0.  Returns a flat uint8 tensor."""
    r, kb4 = scales.shape
    assert kb4 % 4 == 0 and scales.dtype == torch.uint8 and row_multiple % 128 == 0
    tiles = -(-r // row_multiple) * (row_multiple // 128)
    padded = torch.full((tiles * 128, kb4), 127, dtype=torch.uint8, device=scales.device)
    padded[:r] = scales
    v = padded.view(tiles, 4, 32, kb4 // 4, 4)            # [tile, r // 32, r % 32, k block, j]
    return v.permute(0, 3, 2, 1, 4).contiguous().view(-1)


def gemm_mxfp8(a, sfa_packed, b, sfb_packed, out=None, max_ctas=0, stream=None, pair=None):
    """``a``: [M, K] e4m3, ``b``: [N, K] e4m3, scales packed by ``pack_mx_scales``.  Returns bf16 [M, N] =
    dequant(a) @ dequant(b).T with the scaling done inside the tensor core (tcgen05 block_scale MMA).
    ``pair``: CTA pairs with 256 x 256 tiles (needs N % 256 == 0 and A scales padded to 256 rows);
    ``None`` uses them whenever the operands allow it (``MSCCL_GEMM_PAIR=0`` turns that off)."""
    assert a.is_cuda and b.is_cuda and a.dtype == torch.float8_e4m3fn and b.dtype == torch.float8_e4m3fn
    assert a.dim() == 2 and b.dim() == 2 and a.stride(1) == 1 and b.stride(1) == 1
    m, k = a.shape
    n, kb = b.shape
    assert k == kb, 'inner dimensions differ'
    if k % 128 or n % 128:
        raise ValueError(f'K and N must be multiples of 128 (got K={k}, N={n})')
    need_a, need_b = -(-m // 128) * (k // 128) * 512, (n // 128) * (k // 128) * 512
    need_a_pair = -(-m // 256) * 2 * (k // 128) * 512
    if sfa_packed.numel() not in (need_a, need_a_pair) or sfb_packed.numel() < need_b:
        raise ValueError(f'packed scales must hold {need_a} (or {need_a_pair}) and {need_b} bytes')
    can_pair = n % 256 == 0 and sfa_packed.numel() == need_a_pair
    if pair is None:
        pair = can_pair and os.environ.get('MSCCL_GEMM_PAIR', '1') == '1'
    if pair and not can_pair:
        raise ValueError('the CTA-pair kernel needs N % 256 == 0 and A scales packed with row_multiple=256')
    assert sfa_packed.dtype == torch.uint8 and sfb_packed.dtype == torch.uint8 and sfa_packed.is_contiguous()
    if out is None:
        out = torch.empty(m, n, dtype=torch.bfloat16, device=a.device)
    assert out.shape == (m, n) and out.stride(1) == 1 and out.dtype == torch.bfloat16
    stream_h = (stream or torch.cuda.current_stream()).cuda_stream
    if pair:
        load().gemm_mxfp8_2cta(a.data_ptr(), sfa_packed.data_ptr(), b.data_ptr(), sfb_packed.data_ptr(), out.data_ptr(), m, n,
                               k, a.stride(0), b.stride(0), out.stride(0), _errors(a.device).data_ptr(), (max_ctas + 1) // 2,
                               stream_h)
        return out
    load().gemm_mxfp8(a.data_ptr(), sfa_packed.data_ptr(), b.data_ptr(), sfb_packed.data_ptr(), out.data_ptr(), m, n, k,
                      a.stride(0), b.stride(0), out.stride(0), _errors(a.device).data_ptr(), max_ctas, stream_h)
    return out
