"""Sub-byte scalar type descriptors with the reference's 64-bit id encoding
(vllm/scalar_type.py:23-164, csrc/core/scalar_type.hpp:17-157).  Only the
weight types the quantized linear path of this package accepts are tabulated."""
from __future__ import annotations

import functools
from dataclasses import dataclass


@dataclass(frozen=True)
class ScalarType:
    exponent: int
    mantissa: int
    signed: bool
    bias: int
    _finite_values_only: bool = False
    nan_repr: int = 1  # IEEE_754; meaningless for integer types

    @functools.cached_property
    def id(self) -> int:
        val, off = 0, 0
        for member, width in ((self.exponent, 8), (self.mantissa, 8), (int(self.signed), 1),
                              (self.bias, 32), (int(self._finite_values_only), 1),
                              (self.nan_repr, 8)):
            val |= (int(member) & ((1 << width) - 1)) << off
            off += width
        return val

    @property
    def size_bits(self) -> int:
        return self.exponent + self.mantissa + int(self.signed)

    def is_integer(self) -> bool:
        return self.exponent == 0

    def is_floating_point(self) -> bool:
        return self.exponent != 0

    def is_signed(self) -> bool:
        return self.signed

    def has_bias(self) -> bool:
        return self.bias != 0

    def min(self) -> int:
        assert self.is_integer()
        raw = -(1 << (self.size_bits - 1)) if self.signed else 0
        return raw - self.bias

    def max(self) -> int:
        assert self.is_integer()
        return (1 << self.mantissa) - 1 - self.bias

    @classmethod
    def uint(cls, size_bits: int, bias: int | None) -> "ScalarType":
        return cls(0, size_bits, False, bias or 0)

    @classmethod
    def float_(cls, exponent: int, mantissa: int, finite_values_only: bool,
               nan_repr: int) -> "ScalarType":
        """Non-IEEE float (vllm/scalar_type.py:308-326); always signed, no bias."""
        return cls(exponent, mantissa, True, 0, finite_values_only, nan_repr)

    @classmethod
    def from_id(cls, type_id: int) -> "ScalarType":
        for t in _ALL:
            if t.id == type_id:
                return t
        raise ValueError(f"unknown ScalarType id {type_id}")

    def __str__(self) -> str:
        if self.is_floating_point():
            # flags (vllm/scalar_type.py:218-246): f = finite values only, n = NaNs in a
            # non-IEEE encoding (nan_repr != NONE = 0)
            return f"float{self.size_bits}_e{self.exponent}m{self.mantissa}" + (
                "f" if self._finite_values_only else "") + ("n" if self.nan_repr != 0 else "")
        s = f"uint{self.size_bits}" if not self.signed else f"int{self.size_bits}"
        return s + (f"b{self.bias}" if self.bias else "")


class scalar_types:
    uint4 = ScalarType.uint(4, None)
    uint8 = ScalarType.uint(8, None)
    uint4b8 = ScalarType.uint(4, 8)
    uint8b128 = ScalarType.uint(8, 128)
    # NanRepr.EXTD_RANGE_MAX_MIN = 2 (vllm/scalar_type.py:14-20,338-340)
    float8_e4m3fn = ScalarType.float_(4, 3, True, 2)
    # NanRepr.NONE = 0 (vllm/scalar_type.py:345): NVFP4 / MXFP4 weight codes
    float4_e2m1f = ScalarType.float_(2, 1, True, 0)


_ALL = (scalar_types.uint4, scalar_types.uint8, scalar_types.uint4b8, scalar_types.uint8b128,
        scalar_types.float8_e4m3fn, scalar_types.float4_e2m1f)
