"""Parity of the producer-fused forward quantizers (RMSNorm -> Q, SwiGLU -> Q) with the CPU oracle.

The quantizer part is held to the same bar as the plain forward quantizer (codes, scale bytes and mask bits
bit-exact, exceptions counted and explained by a rounding boundary).  The producer part:
* RMSNorm: the row statistic rstd is a sum whose order no two implementations share, so it is checked on its own
  (within 2 fp32 ulp of the float64 value) and then fed to the oracle, after which every remaining step is
  elementwise and the comparison is bit for bit;
* SwiGLU: elementwise throughout; compared with the oracle (torch's CPU silu) and with torch's CUDA kernels followed
  by the plain quantizer.
"""
import pytest
import torch

from oracle import ref_math as rm
from tests import helpers as H

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    import __graft_entry__ as entry

    entry.build()
    from quartet_b200 import ops

    assert torch.cuda.is_available()
    return ops


def _compare(ops, out, a, h):
    """(codes, sf, mask) of the device against the oracle's quantization of the activation `a` (CPU)."""
    codes, sf, mask = out
    rows, cols = a.shape
    ref = rm.quant_fwd(a, h)
    idx, neg = H.unpack_codes(codes)
    e8 = H.unpack_sf(sf, rows, cols)
    n_sf, n_code, bad = H.compare_quantized(idx, neg, e8, ref)
    mask_bad = (H.unpack_mask(mask) != ref.mask) & ~(e8 != ref.e8m0).repeat_interleave(32, dim=1)
    v = (rm.rotate(a, h) / ref.shared.reshape(-1, 1)).abs().reshape(rows, cols)
    assert bool(H.near_threshold(v[bad], H.RTN_THRESHOLDS).all()), "code mismatch away from a rounding boundary"
    assert bool(H.near_threshold(v[mask_bad], torch.tensor([6.0])).all())
    return n_sf, n_code, int(mask_bad.sum())


def _rows(shape, seed, dtype, outliers=False):
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(*shape, generator=gen)
    if outliers:
        x[:, :: 97] *= 20.0
        x[3] = 0.0  # an all-zero row: rstd = rsqrt(eps)
    return x.to(dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(300, 640), (256, 4096), (5, 128)])
def test_rms_stats(ops, shape, dtype):
    x = _rows(shape, 11, dtype, outliers=shape[0] > 5)
    eps = 1e-5
    got = ops.rms_stats(x.cuda(), eps).cpu()
    want = torch.rsqrt(x.double().pow(2).mean(-1) + eps)
    rel = ((got.double() - want) / want).abs().max().item()
    assert rel < 2.5e-7, rel  # 2 ulp of fp32


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(384, 640), (200, 1024), (128, 4096), (256, 2048), (40, 3072), (130, 8192), (5, 128)])
def test_quant_fwd_rmsnorm_matches_oracle(ops, shape, dtype):
    x = _rows(shape, 23, dtype, outliers=True)
    gen = torch.Generator().manual_seed(5)
    w = 1.0 + 0.1 * torch.randn(shape[1], generator=gen)
    eps = 1e-5
    codes, sf, mask, rstd = ops.quant_fwd_rmsnorm(x.cuda(), w.cuda(), eps, had_scale=ops.HAD_SCALE_F32)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert torch.equal(rstd, ops.rms_stats(x.cuda(), eps))
    # the oracle's RMSNorm with the device's row statistic, then the oracle's quantizer (fp32 rotation: the
    # normalised tensor is fp32 whatever the dtype of x, llama.py:73-75)
    a = rm.rmsnorm(x, w, eps, rstd=rstd.cpu())
    assert a.dtype == torch.float32
    n_sf, n_code, n_mask = _compare(ops, (codes, sf, mask), a, rm.hadamard32(torch.float32))
    print(f"rmsnorm {shape} {dtype}: boundary exceptions scale groups {n_sf}, codes {n_code}, mask bits {n_mask}")
    assert n_sf <= 1 and n_code <= 2 and n_mask <= 1
    # and bit for bit what the plain quantizer makes of the same tensor materialised on the device
    xd, wd = x.cuda(), w.cuda()
    a_dev = (xd.float() * rstd.reshape(-1, 1)).type_as(xd) * wd
    c2, s2, m2 = ops.quant_fwd(a_dev.contiguous(), had_scale=ops.HAD_SCALE_F32)
    assert torch.equal(codes, c2) and torch.equal(sf, s2) and torch.equal(mask, m2)  # sf: padding rows of the last block included (zeros)
    # with its own statistic (summed in another order) the oracle's norm differs from the device's by rounding only
    full = rm.rmsnorm(x, w, eps)
    assert torch.allclose(full, a, rtol=1e-6 if dtype == torch.float32 else 1e-2, atol=1e-7)


def test_quant_fwd_rmsnorm_large(ops):
    """132 MB of rows (more than L2 holds), a ragged last band of rows: equal to the plain quantizer on the
    materialised tensor, and a slice of rows quantized alone gives the same rows."""
    rows, cols = 3 * 2688 - 40, 4096
    gen = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(rows, cols, generator=gen, device="cuda")
    w = (1.0 + 0.1 * torch.randn(cols, generator=gen, device="cuda")).contiguous()
    codes, sf, mask, rstd = ops.quant_fwd_rmsnorm(x, w, 1e-6, had_scale=ops.HAD_SCALE_F32)
    a_dev = (x * rstd.reshape(-1, 1)) * w
    c2, s2, m2 = ops.quant_fwd(a_dev, had_scale=ops.HAD_SCALE_F32)
    assert torch.equal(codes, c2) and torch.equal(sf, s2) and torch.equal(mask, m2)
    c3, s3, m3, r3 = ops.quant_fwd_rmsnorm(x[5120:5248].contiguous(), w, 1e-6, had_scale=ops.HAD_SCALE_F32)
    assert torch.equal(c3, codes[5120:5248]) and torch.equal(r3, rstd[5120:5248]) and torch.equal(m3, mask[5120:5248])
    assert ops.device_status() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape", [(384, 1792), (200, 256), (128, 11008)])
def test_quant_fwd_swiglu_matches_oracle(ops, shape, dtype):
    rows, hidden = shape
    gen = torch.Generator().manual_seed(31)
    h = (2.0 * torch.randn(rows, 2 * hidden, generator=gen)).to(dtype)
    h[1, :64] = 0.0
    h[2, :32] = torch.linspace(-30, 30, 32).to(dtype)  # silu's tails
    bf = dtype == torch.bfloat16
    had, hm = (ops.HAD_SCALE_BF16, rm.hadamard32()) if bf else (ops.HAD_SCALE_F32, rm.hadamard32(torch.float32))
    out = ops.quant_fwd_swiglu(h.cuda(), had_scale=had)
    torch.cuda.synchronize()
    # the device's own torch kernels followed by the plain quantizer: the same bits
    hd = h.cuda()
    a_dev = (torch.nn.functional.silu(hd[:, :hidden]) * hd[:, hidden:]).contiguous()
    c2, s2, m2 = ops.quant_fwd(a_dev, had_scale=had)
    diff_groups = int((out[0].reshape(rows, -1, 16) != c2.reshape(rows, -1, 16)).any(-1).sum())
    print(f"swiglu {shape} {dtype}: groups differing from torch's CUDA kernels + plain quantizer: {diff_groups}")
    assert diff_groups == 0 and torch.equal(out[1], s2) and torch.equal(out[2], m2)
    # the oracle (torch's CPU kernels).  Its silu uses another exp, so its activation can differ from the device's in
    # the last place: rarely for bf16 (two roundings hide it), in many values for fp32.  The activations are
    # compared as values; the quantization is then checked on the device's activation, pinned just above.
    a = rm.swiglu(h)
    a_cpu_dev = a_dev.cpu()
    if bf:
        frac = (a != a_cpu_dev).float().mean().item()
        print(f"swiglu {shape} bf16: fraction of activations differing from the CPU's (by one bf16 ulp): {frac:.2e}")
        assert frac < 1e-3 and torch.allclose(a.float(), a_cpu_dev.float(), rtol=2 ** -7, atol=1e-30)
    else:
        assert torch.allclose(a, a_cpu_dev, rtol=5e-7, atol=1e-30)
    same = bool((a == a_cpu_dev).all())
    n_sf, n_code, n_mask = _compare(ops, out, a if same else a_cpu_dev, hm)
    print(f"swiglu {shape} {dtype}: boundary exceptions scale groups {n_sf}, codes {n_code}, mask bits {n_mask}")
    assert n_sf <= 1 and n_code <= 2 and n_mask <= 1


def test_swiglu_values_equal_torch_for_every_bf16_input(ops):
    """The SwiGLU arithmetic of the fused quantizer, read through quartet_swiglu: silu is compared with torch's CUDA
    kernel on ALL 65536 bf16 bit patterns (NaNs aside) and the product on each of them times a spread of gates; then
    the fused quantizer must equal the plain quantizer applied to these values."""
    bits = torch.arange(65536, dtype=torch.int32).to(torch.int16)
    up = bits.view(torch.bfloat16).cuda()
    finite = ~torch.isnan(up.float())
    gates = torch.tensor([1.0, -1.0, 0.3337, 7.25, -1e-3, 3e4, 0.0, 1e-30], dtype=torch.bfloat16, device="cuda")
    h = torch.cat([up.repeat(8, 1), gates.reshape(8, 1).expand(8, 65536)], dim=1).contiguous()  # [8, 2 * 65536]
    got = ops.swiglu(h)
    want = torch.nn.functional.silu(h[:, :65536]) * h[:, 65536:]
    both_nan = torch.isnan(got.float()) & torch.isnan(want.float())  # silu(-inf), inf * 0
    same = (got.view(torch.int16) == want.view(torch.int16)) | both_nan | ~finite
    assert bool(same.all()), f"{int((~same).sum())} of {same.numel()} values differ from torch's"
    hf = h.float()
    assert torch.equal(ops.swiglu(hf).nan_to_num(0.0), (torch.nn.functional.silu(hf[:, :65536]) * hf[:, 65536:]).nan_to_num(0.0))
    # fused quantizer == plain quantizer on these values
    gen = torch.Generator(device="cuda").manual_seed(2)
    h2 = (3.0 * torch.randn(256, 2 * 512, generator=gen, device="cuda")).to(torch.bfloat16)
    a = ops.swiglu(h2)
    f = ops.quant_fwd_swiglu(h2)
    p = ops.quant_fwd(a)
    assert all(torch.equal(x, y) for x, y in zip(f, p))


def test_producer_entries_reject_bad_arguments(ops):
    x = torch.zeros(128, 200, device="cuda")
    with pytest.raises(ValueError):
        ops.quant_fwd_rmsnorm(x, torch.ones(200, device="cuda"), 1e-5)  # width not a multiple of 128
    with pytest.raises(ValueError):
        ops.quant_fwd_rmsnorm(torch.zeros(128, 256, device="cuda"), torch.ones(256, device="cuda", dtype=torch.bfloat16), 1e-5)
    with pytest.raises(ValueError):
        ops.quant_fwd_swiglu(torch.zeros(128, 2 * 200, device="cuda"))
    with pytest.raises(ValueError):
        ops.rms_stats(torch.zeros(4, 12, device="cuda"), 1e-5)
    with pytest.raises(ValueError):
        ops.swiglu(torch.zeros(4, 2 * 12, device="cuda"))
