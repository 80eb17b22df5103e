"""Reference and tolerance policy of the kernel tests.

Two regimes, as in the reference's policy (triton_conv3d/reference.py:63-397):

* **Exact**: operands drawn from {-1, 0, +1} (optionally thinned to a density) make every product and
  every partial sum an integer far below 2^24, so an fp32-accumulating tensor-core kernel must reproduce
  the fp64 result *bit for bit* after the final bf16 rounding: any mismatch is an indexing bug, not noise.
* **Bounded**: for real-valued operands the error of a K-term bf16 x bf16 -> fp32 dot product rounded to
  bf16 is bounded by ``8 u32 sqrt(K) rms + 2 r u_out peak`` (``u32 = 2^-24``, ``u_out`` the unit
  round-off of the output type, ``r`` the number of roundings of the result, ``rms`` / ``peak`` of the
  reference); ``assert_close`` applies that bound element-wise.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch

U32 = 2.0 ** -24
UNIT_ROUNDOFF = {torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -11, torch.float32: 2.0 ** -24}


def exact_operand(shape: Sequence[int], generator: Optional[torch.Generator] = None, density: float = 1.0,
                  device="cpu") -> torch.Tensor:
    """fp32 tensor of {-1, 0, +1}; ``density`` is the probability that an entry is non-zero."""
    v = torch.randint(-1, 2, tuple(shape), generator=generator, device=device).float()
    if density < 1.0:
        keep = torch.rand(tuple(shape), generator=generator, device=device) < density
        v = v * keep
    return v


def exact_is_safe(k_terms: int) -> bool:
    """Integer partial sums of ``k_terms`` products in {-1,0,1} stay exact in fp32 below 2^24 and, rounded to
    bf16, exact below 2^8 only if the result fits 8 bits: callers thin the operands so |sum| stays small."""
    return k_terms < 2 ** 24


def conv3d_reference(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, padding: int = 1,
                     stride: int = 1) -> torch.Tensor:
    """fp64 convolution of NCDHW ``x`` (integer-valued references are rounded: some fp64 algorithms leave 1e-14)."""
    y = torch.nn.functional.conv3d(x.double(), w.double(), None if bias is None else bias.double(), stride=stride,
                                   padding=padding)
    return y


def error_bound(reference: torch.Tensor, k_terms: int, out_dtype=torch.bfloat16, roundings: int = 1) -> float:
    """``8 u32 sqrt(K) rms + 2 r u_out peak`` for a K-term reduction accumulated in fp32."""
    ref = reference.double()
    rms = float(ref.pow(2).mean().sqrt())
    peak = float(ref.abs().max())
    return 8.0 * U32 * math.sqrt(max(1, k_terms)) * rms + 2.0 * roundings * UNIT_ROUNDOFF[out_dtype] * peak


def assert_close(got: torch.Tensor, reference: torch.Tensor, k_terms: int, out_dtype=torch.bfloat16,
                 roundings: int = 1, what: str = "") -> None:
    bound = error_bound(reference, k_terms, out_dtype, roundings)
    err = float((got.double() - reference.double()).abs().max())
    if not err <= bound:
        raise AssertionError(f"{what}: max abs error {err:.3e} exceeds the bound {bound:.3e} (K = {k_terms})")


def assert_exact(got: torch.Tensor, reference: torch.Tensor, out_dtype=torch.bfloat16, what: str = "") -> None:
    want = reference.round().to(out_dtype).double()
    if not torch.equal(got.double(), want):
        raise AssertionError(f"{what}: {int((got.double() != want).sum())} elements differ, max abs diff "
                             f"{float((got.double() - want).abs().max())}")
