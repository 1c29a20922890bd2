"""How far apart two correct implementations of one operator may be.

The bound of a comparison follows from the operator's mathematics - its reduction length,
its accumulation type and its output type - never from a measurement of the pair being
compared.  For a sum of ``n`` terms in a type with unit round-off ``u``

    |fl(sum a_i b_i) - sum a_i b_i| <= gamma_n * sum |a_i b_i|,   gamma_n = n u / (1 - n u)

(Higham, *Accuracy and Stability of Numerical Algorithms*, 2nd ed., section 3.1).  Two
implementations differ by at most twice that, and storing the result rounds once more in the
output type.  ``rounding`` is the bound for reductions whose result is a scale of its inputs
(a norm's sum of squares, a softmax denominator); ``dot`` for mixed-sign products (matrix
products, attention scores), where the result can cancel: with independent signs
``|result| ~ sqrt(n) sigma`` against ``sum |a_i b_i| ~ n sigma``, so relative to the output's
largest magnitude the bound is ``2 gamma_n sqrt(n)``; ``exact`` for operators that only move
values.  A comparison is ``|candidate - reference| <= atol + rtol * magnitude`` where the
magnitude is ``|reference|`` or, for a bound that cancels, the output's largest
``|reference|``.

Reference behaviour: crates/ops/src/tolerance.rs:1-60 (reference project path).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

# unit round-off (half the spacing at 1) and smallest normal value per type
_U = {torch.float32: 2.0 ** -24, torch.float16: 2.0 ** -11, torch.bfloat16: 2.0 ** -8,
      torch.float64: 2.0 ** -53, torch.float8_e4m3fn: 2.0 ** -4}
_TINY = {torch.float32: 2.0 ** -126, torch.float16: 2.0 ** -14, torch.bfloat16: 2.0 ** -126,
         torch.float64: 2.0 ** -1022, torch.float8_e4m3fn: 2.0 ** -6}


def unit_roundoff(dtype) -> float:
    return _U[dtype]


def gamma(n: int, u: float) -> float:
    nu = n * u
    assert nu < 1.0, "the reduction is too long for this accumulation type"
    return nu / (1.0 - nu)


@dataclass(frozen=True)
class Tolerance:
    atol: float
    rtol: float
    cancels: bool = False          # rtol applies to the output's largest magnitude

    @staticmethod
    def exact() -> "Tolerance":
        return Tolerance(0.0, 0.0)

    @staticmethod
    def rounding(n: int, accum=torch.float32, out=torch.bfloat16, inputs=None) -> "Tolerance":
        """A reduction of ``n`` same-sign terms accumulated in ``accum``, stored in ``out``;
        ``inputs``: the type the operands were rounded to before the reduction (each operand
        then carries its own relative error ``u_in``, first order in the result)."""
        r = 2.0 * gamma(max(n, 1), _U[accum]) + _U[out]
        if inputs is not None:
            r += 2.0 * _U[inputs]
        return Tolerance(_TINY[out], r)

    @staticmethod
    def dot(n: int, accum=torch.float32, out=torch.bfloat16, inputs=None) -> "Tolerance":
        """A reduction of ``n`` mixed-sign products; relative to the output's largest value."""
        r = 2.0 * gamma(max(n, 1), _U[accum]) * math.sqrt(max(n, 1)) + _U[out]
        if inputs is not None:
            # operands rounded to `inputs` before the product: each product errs by 2 u_in,
            # independent signs over n terms, relative to the output's largest magnitude
            r += 2.0 * _U[inputs]
        return Tolerance(_TINY[out], r, cancels=True)

    def then(self, other: "Tolerance") -> "Tolerance":
        """This operator's output feeding ``other`` (first-order error propagation)."""
        return Tolerance(self.atol + other.atol, self.rtol + other.rtol,
                         self.cancels or other.cancels)

    def scaled(self, k: float) -> "Tolerance":
        return Tolerance(self.atol * k, self.rtol * k, self.cancels)

    # ------------------------------------------------------------------ check --
    def check(self, candidate: torch.Tensor, reference: torch.Tensor, what: str = "") -> None:
        c, r = candidate.detach().double().cpu(), reference.detach().double().cpu()
        assert c.shape == r.shape, f"{what}: shapes {tuple(c.shape)} vs {tuple(r.shape)}"
        if c.numel() == 0:
            return
        mag = r.abs().max() if self.cancels else r.abs()
        excess = (c - r).abs() - (self.atol + self.rtol * mag)
        worst = float(excess.max())
        if not worst <= 0.0:
            i = int(excess.argmax())
            raise AssertionError(
                f"{what}: |candidate - reference| exceeds atol {self.atol:.3g} + rtol "
                f"{self.rtol:.3g} x magnitude by {worst:.3g} at flat index {i} "
                f"(candidate {float(c.flatten()[i]):.6g}, reference {float(r.flatten()[i]):.6g})")
