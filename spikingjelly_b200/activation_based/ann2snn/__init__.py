"""ANN-to-SNN conversion: converters, recipes (rate coding, local threshold balancing, exact
temporal-difference conversion of transformers), calibration modules and TD operators."""
from . import operators
from .converter import Converter, FXConverter, ModuleConverter
from .delay import estimate_delay_start
from .factories import NeuronFactory
from .modules import ChannelVoltageScaler, VoltageHook, VoltageScaler
from .qcfs import SignedQCFSSequenceEncoder
from .recipes import (Qwen2SNNCalibration, Qwen2SNNConfig, Qwen2SNNModel, Qwen2SNNRecipe, calibrate_qwen2_snn, ConversionRecipe, FXConversionRecipe, LocalThresholdBalancingRecipe, ModuleConversionRecipe, RateCodingRecipe,
                      STATransformerRecipe, SpikeZIPTFQANNRecipe, TransformerTDEquivalentRecipe)
from .utils import download_url

__all__ = ["Converter", "FXConverter", "ModuleConverter", "ConversionRecipe", "FXConversionRecipe", "ModuleConversionRecipe",
           "RateCodingRecipe", "LocalThresholdBalancingRecipe", "TransformerTDEquivalentRecipe", "STATransformerRecipe", "SpikeZIPTFQANNRecipe", "ChannelVoltageScaler", "VoltageHook",
           "VoltageScaler", "download_url", "NeuronFactory", "operators", "SignedQCFSSequenceEncoder", "estimate_delay_start", "Qwen2SNNCalibration",
           "Qwen2SNNConfig", "Qwen2SNNModel", "Qwen2SNNRecipe", "calibrate_qwen2_snn"]
