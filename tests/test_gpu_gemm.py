"""tcgen05 GEMM against a plain PyTorch fp32 reference of the same operation."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b):
    return a.float() @ b.float().t()


@pytest.mark.parametrize('m,n,k,bn', [(128, 256, 64, 256), (128, 128, 128, 128), (256, 512, 256, 256),
                                      (1000, 768, 320, 256), (384, 1280, 1024, 128), (4096, 3584, 4096, 256)])
def test_gemm_matches_fp32_reference(m, n, k, bn):
    from msccl.ops import check_gemm_errors, gemm_bf16
    gen = torch.Generator(device='cuda').manual_seed(m + n + k)
    a = torch.randn(m, k, device='cuda', generator=gen).bfloat16()
    b = (torch.randn(n, k, device='cuda', generator=gen) * 0.05).bfloat16()
    d = gemm_bf16(a, b, bn=bn)
    check_gemm_errors()
    want = _ref(a, b)
    err = (d.float() - want).abs().max().item()
    scale = want.abs().max().item()
    assert err <= 1e-2 * scale + 1e-3, (err, scale)


def test_gemm_identity_is_exact():
    # B = identity picks out columns of A: any mistake in swizzle, descriptor or epilogue mapping
    # shows up as a permutation, not as rounding noise
    from msccl.ops import check_gemm_errors, gemm_bf16
    a = torch.randn(256, 256, device='cuda').bfloat16()
    eye = torch.eye(256, device='cuda').bfloat16()
    d = gemm_bf16(a, eye)
    check_gemm_errors()
    assert torch.equal(d, a)


def test_gemm_swiglu_epilogue():
    from msccl.ops import check_gemm_errors, gemm_bf16
    from msccl.ops.gemm import interleave_gate_up
    gen = torch.Generator(device='cuda').manual_seed(3)
    m, k, f = 512, 512, 768
    x = torch.randn(m, k, device='cuda', generator=gen).bfloat16()
    wg = (torch.randn(f, k, device='cuda', generator=gen) * 0.05).bfloat16()
    wu = (torch.randn(f, k, device='cuda', generator=gen) * 0.05).bfloat16()
    h = gemm_bf16(x, interleave_gate_up(wg, wu), epilogue='swiglu')
    check_gemm_errors()
    want = torch.nn.functional.silu(_ref(x, wg)) * _ref(x, wu)
    assert h.shape == (m, f)
    assert (h.float() - want).abs().max().item() <= 2e-2 * want.abs().max().item() + 1e-3


def test_gemm_strided_operands_and_few_ctas():
    from msccl.ops import check_gemm_errors, gemm_bf16
    big_a = torch.randn(300, 512, device='cuda').bfloat16()
    big_b = (torch.randn(512, 512, device='cuda') * 0.1).bfloat16()
    a, b = big_a[:, :256], big_b[:, 128:384]          # row pitch 512, 16-byte aligned starts
    out = torch.zeros(300, 1024, device='cuda', dtype=torch.bfloat16)
    gemm_bf16(a, b, out=out[:, 256:768], max_ctas=3)
    check_gemm_errors()
    want = _ref(a, b)
    assert (out[:, 256:768].float() - want).abs().max().item() <= 1e-2 * want.abs().max().item() + 1e-3
    assert torch.all(out[:, :256] == 0) and torch.all(out[:, 768:] == 0)


@pytest.mark.parametrize('m,n,k', [(128, 128, 128), (256, 256, 512), (300, 384, 1024), (300, 512, 256), (1024, 2048, 2048)])
def test_gemm_mxfp8_block_scaled(m, n, k):
    # block-scaled fp8 (one power-of-two scale per 32 K elements of a row, applied by the tensor core)
    # against the fp32 product of the dequantised operands; rows and K blocks get widely different
    # magnitudes so that a scale landing on the wrong row or block is far outside the tolerance
    from msccl.ops import check_gemm_errors
    from msccl.ops.gemm import dequantize_mxfp8, gemm_mxfp8, pack_mx_scales, quantize_mxfp8
    gen = torch.Generator(device='cuda').manual_seed(m + n + k)

    def operand(rows):
        x = torch.randn(rows, k, device='cuda', generator=gen)
        row_mag = torch.exp2(torch.randint(-4, 5, (rows, 1), device='cuda', generator=gen).float())
        blk_mag = torch.exp2(torch.randint(-3, 4, (rows, k // 32), device='cuda', generator=gen).float())
        return x * row_mag * blk_mag.repeat_interleave(32, dim=1)

    aq, sa = quantize_mxfp8(operand(m))
    bq, sb = quantize_mxfp8(operand(n))
    d = gemm_mxfp8(aq, pack_mx_scales(sa), bq, pack_mx_scales(sb), pair=False)
    check_gemm_errors()
    if n % 256 == 0:
        # CTA pairs (cta_group::2 block-scaled MMA): same products, same order within a tile row
        d2 = gemm_mxfp8(aq, pack_mx_scales(sa), bq, pack_mx_scales(sb), pair=True)
        check_gemm_errors()
        assert torch.equal(d2, d)
    want = dequantize_mxfp8(aq, sa) @ dequantize_mxfp8(bq, sb).t()
    err = (d.float() - want).abs().max().item()
    scale = want.abs().max().item()
    assert err <= 1e-2 * scale + 1e-3, (err, scale)
    # row-wise check as well: a small row must not hide behind a large one
    row_scale = want.abs().amax(dim=1)
    assert torch.all((d.float() - want).abs().amax(dim=1) <= 2e-2 * row_scale + 1e-3)


@pytest.mark.parametrize('m,n,k', [(256, 256, 64), (256, 512, 512), (1000, 768, 1024), (4096, 4096, 2048)])
def test_gemm_cta_pair_matches_reference(m, n, k):
    # tcgen05 cta_group::2: two CTAs share one 256 x 256 tile
    from msccl.ops import check_gemm_errors, gemm_bf16
    gen = torch.Generator(device='cuda').manual_seed(m * 7 + n + k)
    a = torch.randn(m, k, device='cuda', generator=gen).bfloat16()
    b = (torch.randn(n, k, device='cuda', generator=gen) * 0.05).bfloat16()
    d = gemm_bf16(a, b, pair=True)
    check_gemm_errors()
    want = _ref(a, b)
    assert (d.float() - want).abs().max().item() <= 1e-2 * want.abs().max().item() + 1e-3
    # the single-CTA kernel accumulates in the same order: identical bits
    assert torch.equal(d, gemm_bf16(a, b, pair=False))


def test_gemm_cta_pair_identity_and_swiglu():
    from msccl.ops import check_gemm_errors, gemm_bf16
    from msccl.ops.gemm import interleave_gate_up
    a = torch.randn(512, 256, device='cuda').bfloat16()
    eye = torch.eye(256, device='cuda').bfloat16()
    assert torch.equal(gemm_bf16(a, eye, pair=True), a)
    gen = torch.Generator(device='cuda').manual_seed(5)
    x = torch.randn(384, 512, device='cuda', generator=gen).bfloat16()
    wg = (torch.randn(768, 512, device='cuda', generator=gen) * 0.05).bfloat16()
    wu = (torch.randn(768, 512, device='cuda', generator=gen) * 0.05).bfloat16()
    w = interleave_gate_up(wg, wu)
    h = gemm_bf16(x, w, epilogue='swiglu', pair=True)
    check_gemm_errors()
    assert torch.equal(h, gemm_bf16(x, w, epilogue='swiglu', pair=False))


def test_one_pass_mx_quantisation_matches_the_torch_reference():
    """``quantize_mxfp8_packed`` (one CUDA kernel: e4m3 values + packed scale blocks) against ``quantize_mxfp8`` +
    ``pack_mx_scales`` written in torch: the same scale rule, so the bytes agree (a handful of groups whose largest
    magnitude sits exactly on a power-of-two boundary may round the other way in torch's float log2)."""
    from msccl.ops.gemm import pack_mx_scales, quantize_mxfp8, quantize_mxfp8_packed
    gen = torch.Generator(device='cuda').manual_seed(3)
    for rows, k in ((256, 512), (200, 1024), (1024, 1792)):
        x = (torch.randn(rows, k, device='cuda', generator=gen) * torch.rand(rows, 1, device='cuda', generator=gen) * 4).bfloat16()
        x[3, :64] = 0                                   # an all-zero group
        q, packed = quantize_mxfp8_packed(x)
        q_ref, s_ref = quantize_mxfp8(x.float())
        packed_ref = pack_mx_scales(s_ref, row_multiple=128)
        assert packed.shape == packed_ref.shape
        same_scale = (packed == packed_ref).float().mean().item()
        same_value = (q.view(torch.uint8) == q_ref.view(torch.uint8)).float().mean().item()
        assert same_scale > 0.999 and same_value > 0.995, (rows, k, same_scale, same_value)
