"""tcgen05 GEMM for bf16 on sm_100a: ``D = A @ B.T`` with A ``[M, K]`` and B ``[N, K]`` row-major
(both K-major, the layout of activations and ``nn.Linear`` weights), fp32 accumulation in tensor
memory, bf16 result.  ``epilogue='swiglu'`` fuses ``silu(gate) * up`` where each 256-column tile
of B holds 128 gate rows followed by the 128 matching up rows (see ``interleave_gate_up``).
"""
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


def gemm_bf16(a, b, out=None, epilogue='none', bn=256, max_ctas=0, stream=None):
    """``a``: [M, K] bf16, ``b``: [N, K] bf16 (row pitch may exceed K).  Returns [M, N] (or [M, N/2] for swiglu)."""
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
    load().gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), m, n, k, a.stride(0), b.stride(0), out.stride(0),
                     1 if swiglu else 0, bn, _errors(a.device).data_ptr(), max_ctas, stream_h)
    return out
