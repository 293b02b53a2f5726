"""backends.Capabilities of this backend (ref mpsgraph/gomlx/capabilities.go:14-167).

The reference declares 96 op types and 12 dtypes.  Listed here is what this
backend lowers.  Op types of the reference that it does not lower --
convolution, pooling and their gradients (SelectAndScatter) -- are absent, so
GoMLX reports them as not implemented instead of failing late.  Sort is
listed with a limit: its comparator must order by the first input.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict

from .backend import dtypes

OPERATIONS = [
    "Parameter", "Constant", "Identity", "Iota",
    "Abs", "Neg", "Sqrt", "Rsqrt", "Exp", "Expm1", "Log", "Log1p", "Sin", "Cos", "Tanh", "Logistic", "Erf", "Floor", "Ceil",
    "Round", "Sign", "LogicalNot", "BitwiseNot", "IsFinite", "IsNaN",
    "Add", "Sub", "Mul", "Div", "Rem", "Pow", "Max", "Min", "Atan2", "LogicalAnd", "LogicalOr", "LogicalXor", "BitwiseAnd",
    "BitwiseOr", "BitwiseXor", "ShiftLeft", "ShiftRightArithmetic", "ShiftRightLogical",
    "Equal", "NotEqual", "LessThan", "LessOrEqual", "GreaterThan", "GreaterOrEqual",
    "EqualTotalOrder", "NotEqualTotalOrder", "LessThanTotalOrder", "LessOrEqualTotalOrder", "GreaterThanTotalOrder",
    "GreaterOrEqualTotalOrder",
    "Reshape", "Transpose", "ConvertDType", "BroadcastInDim", "Slice", "Concatenate", "Reverse", "Pad", "DynamicSlice", "DynamicUpdateSlice", "Where", "Clamp",
    "DotGeneral", "ReduceSum", "ReduceProduct", "ReduceMax", "ReduceMin", "ReduceLogicalAnd", "ReduceLogicalOr", "ArgMinMax",
    "Gather", "BatchNormForInference",
    "ScatterSum", "ScatterMax", "ScatterMin", "BatchNormForTraining", "BatchNormGradient", "RNGBitGenerator",
    "Call", "While", "If", "Sort",
    "FusedSoftmax", "FusedGelu", "FusedLayerNorm", "FusedDense", "FusedAttentionQKVProjection",
    "FusedScaledDotProductAttention",
]


@dataclass
class Capabilities:
    Functions: bool = True  # closures and named sub-functions for While / If / Sort / Call (ref capabilities.go:17)
    # Weights handed over as graph constants are uploaded to the device once, at compile, and stay resident; as
    # parameters they would be passed (and shape-checked) on every Execute.  Same field as the reference's second
    # backend sets (ref coreml/gomlx/capabilities.go:18-23).
    PreferConstantsForVariables: bool = True
    Operations: Dict[str, bool] = field(default_factory=dict)
    DTypes: Dict[int, bool] = field(default_factory=dict)


def backend_capabilities() -> Capabilities:
    return Capabilities(
        Functions=True,
        PreferConstantsForVariables=True,
        Operations={name: True for name in OPERATIONS},
        DTypes={int(d): True for d in (dtypes.Bool, dtypes.Int8, dtypes.Int16, dtypes.Int32, dtypes.Int64, dtypes.Float16,
                                      dtypes.BFloat16, dtypes.Float32, dtypes.Float64, dtypes.Uint8, dtypes.Uint16,
                                      dtypes.Uint32, dtypes.Uint64)},
    )
