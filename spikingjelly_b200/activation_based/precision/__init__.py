"""Precision policies: fp32 / fp16 / bf16 autocast and fp8 on the package's own tensor-core kernels."""
from .api import PrecisionArtifacts, prepare_model_for_precision, save_precision_reports
from .capability import build_capability_report, validate_capability
from .config import PrecisionConfig
from .convert import ConversionReport, analyze_convertible_modules, convert_model_for_precision
from .float8_attention import TransformerEngineDotProductAttentionAdapter
from .float8_base import Float8LinearStepModule, wrap_float8_linear_module
from .float8_conv import (Float8PointwiseConv1dStepModule, is_supported_pointwise_conv1d, make_linear_from_pointwise_conv1d,
                          wrap_float8_pointwise_conv1d_module)
from .float8_native import (Float8LayerNormLinear, Float8LayerNormMLP, Float8Linear, Float8NativePolicy,
                            Float8TELayerNormLinearModule, Float8TELayerNormMLPModule, Float8TorchAOPolicy,
                            Float8TransformerEnginePolicy)
from .policy import BF16Policy, FP16Policy, FP32Policy, PrecisionPolicy
from .runtime import resolve_precision_policy

__all__ = ["PrecisionArtifacts", "PrecisionConfig", "prepare_model_for_precision", "save_precision_reports",
           "build_capability_report", "validate_capability", "ConversionReport", "analyze_convertible_modules",
           "convert_model_for_precision", "TransformerEngineDotProductAttentionAdapter", "Float8LinearStepModule",
           "wrap_float8_linear_module", "Float8PointwiseConv1dStepModule", "is_supported_pointwise_conv1d",
           "make_linear_from_pointwise_conv1d", "wrap_float8_pointwise_conv1d_module", "Float8TELayerNormLinearModule",
           "Float8TELayerNormMLPModule", "Float8TorchAOPolicy", "Float8TransformerEnginePolicy", "Float8NativePolicy",
           "Float8Linear", "Float8LayerNormLinear", "Float8LayerNormMLP", "PrecisionPolicy", "FP32Policy", "FP16Policy",
           "BF16Policy", "resolve_precision_policy"]
