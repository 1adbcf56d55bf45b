from .base import ConversionRecipe, FXConversionRecipe, ModuleConversionRecipe
from .local_threshold_balancing import LocalThresholdBalancingRecipe
from .qwen2 import Qwen2SNNCalibration, Qwen2SNNConfig, Qwen2SNNModel, Qwen2SNNRecipe, calibrate_qwen2_snn
from .rate_coding import RateCodingRecipe
from .spikezip_qann import SpikeZIPTFQANNRecipe
from .sta_transformer import STATransformerRecipe
from .transformer_td_equivalent import TransformerTDEquivalentRecipe

__all__ = ["ConversionRecipe", "FXConversionRecipe", "ModuleConversionRecipe", "LocalThresholdBalancingRecipe", "RateCodingRecipe", "SpikeZIPTFQANNRecipe",
           "STATransformerRecipe", "TransformerTDEquivalentRecipe", "Qwen2SNNCalibration", "Qwen2SNNConfig", "Qwen2SNNModel",
           "Qwen2SNNRecipe", "calibrate_qwen2_snn"]
