"""Shared pieces of the parity tests: unpacking device results, boundary accounting."""
from __future__ import annotations

import numpy as np
import torch

from oracle import ref_math as rm

RTN_THRESHOLDS = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])


def bf16r(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.bfloat16).to(torch.float32)


def unpack_codes(codes_u8: torch.Tensor):
    """[rows, cols/2] packed -> (idx int32 [rows, cols], neg bool [rows, cols])"""
    c = codes_u8.cpu()
    lo, hi = c & 0xF, c >> 4
    full = torch.stack([lo, hi], dim=-1).reshape(c.shape[0], -1).to(torch.int32)
    return full & 7, (full & 8) != 0


def unpack_sf(sf_u8: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    return rm.from_blocked(sf_u8.cpu(), rows, cols // 32)


def unpack_mask(mask_u8: torch.Tensor) -> torch.Tensor:
    m = mask_u8.cpu()
    bits = torch.arange(8, dtype=torch.uint8)
    return ((m.unsqueeze(-1) >> bits) & 1).bool().reshape(m.shape[0], -1)


def sign_matters(idx):
    """+0 and -0 are the same value; signs are compared only where the magnitude is non-zero."""
    return idx != 0


def near_threshold(a: torch.Tensor, thresholds: torch.Tensor, ulps: int = 2) -> torch.Tensor:
    """True where |v| lies within `ulps` fp32 ulp of a rounding threshold."""
    a = a.reshape(-1, 1).to(torch.float64)
    t = thresholds.reshape(1, -1).to(torch.float64)
    ulp = torch.tensor(np.spacing(thresholds.numpy().astype(np.float32)), dtype=torch.float64).reshape(1, -1)
    return ((a - t).abs() <= ulps * ulp).any(-1)


def compare_quantized(dev_idx, dev_neg, dev_e8m0, ref: rm.Quantized):
    """Returns (n_scale_mismatch_groups, n_code_mismatch_outside_those_groups, mismatch mask)."""
    rows, cols = ref.rows, ref.cols
    sf_bad = dev_e8m0 != ref.e8m0
    grp_bad = sf_bad.repeat_interleave(32, dim=1)
    code_bad = (dev_idx != ref.idx) | ((dev_neg != ref.neg) & sign_matters(ref.idx) & sign_matters(dev_idx))
    code_bad = code_bad & ~grp_bad
    return int(sf_bad.sum()), int(code_bad.sum()), code_bad


def random_mxfp4(rows: int, cols: int, gen: torch.Generator, e_lo=118, e_hi=130):
    """Random packed codes + logical scales; returns (packed u8, e8m0 u8 [rows, cols/32], values fp32)."""
    codes = torch.randint(0, 16, (rows, cols), generator=gen, dtype=torch.uint8)
    e8 = torch.randint(e_lo, e_hi, (rows, cols // 32), generator=gen, dtype=torch.uint8)
    grid = torch.tensor(rm.E2M1_GRID)
    val = grid[(codes & 7).long()] * torch.where((codes & 8) != 0, -1.0, 1.0)
    val = (val.reshape(rows, -1, 32) * torch.exp2(e8.float() - 127).unsqueeze(-1)).reshape(rows, cols)
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).contiguous()
    return packed, e8, val
