"""Memory hierarchy of the NeuroMC-like accelerator model (32 nm): named register files and SRAM macros with their
capacity, word width, port widths and energy per access, plus the switches that decide which traffic a report charges
(``op_counter/neuromc/config.py:1-218`` of the reference).  The numbers are the hardware constants of that model."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Tuple

__all__ = ["MemoryInstanceSpec", "MemoryHierarchyConfig"]


@dataclass(frozen=True)
class MemoryInstanceSpec:
    """One memory: ``size_bits`` capacity, ``datawidth`` bits per word, read / write port widths in bits per access and
    the energy of one access of that width in pJ."""
    name: str
    size_bits: int
    datawidth: int
    r_bw: int
    w_bw: int
    r_cost: float
    w_cost: float


_REG_BIT = 0.00901 / 7.1 * 2            # pJ per register bit access
_REG_16 = 0.14416 / 7.1 * 2
_CONV_SPIKE, _CONV_WORD_S, _CONV_WORD_L = 0.44854798, 5.302477904, 5.792676768
_WIDE, _MASK = 92.68282828, 7.176767677

#: name -> (size_bits, datawidth, port width, read cost, write cost)
_TABLE = {
    "reg_1b": (1, 1, 1, _REG_BIT, _REG_BIT),
    "reg_16b": (16, 16, 16, _REG_16, _REG_16),
    "reg_32b": (32, 32, 32, 2 * _REG_16, 2 * _REG_16),
    # forward core: spikes in, weights in, pre-activations out; soma potentials, spikes, spike masks
    "sram_fp_conv_in_s": (18496, 1, 1, _CONV_SPIKE, _CONV_SPIKE),
    "sram_fp_conv_in_w": (18432, 16, 16, _CONV_WORD_S, _CONV_WORD_S),
    "sram_fp_conv_out_xi": (65536, 16, 16, _CONV_WORD_L, _CONV_WORD_L),
    "sram_fp_soma_u": (1048576, 16, 256, _WIDE, _WIDE),
    "sram_fp_soma_s": (262144, 1, 16, _MASK, _MASK),
    "sram_fp_soma_smask": (65536, 1, 16, _MASK, _MASK),
    # backward core: potential gradients in, weights in, result out; surrogate-gradient operands
    "sram_bp_conv_in_du": (73984, 16, 16, _CONV_WORD_L, _CONV_WORD_L),
    "sram_bp_conv_in_w": (18432, 16, 16, _CONV_WORD_S, _CONV_WORD_S),
    "sram_bp_conv_out_res": (65536, 16, 16, _CONV_WORD_L, _CONV_WORD_L),
    "sram_bp_grad_in_u": (1048576, 16, 256, _WIDE, _WIDE),
    "sram_bp_grad_in_smask": (65536, 1, 16, _MASK, _MASK),
    "sram_bp_grad_in_s": (65536, 1, 16, _MASK, _MASK),
    "sram_bp_grad_out_du": (1048576, 16, 256, _WIDE, _WIDE),
    # weight-gradient core
    "sram_wg_conv_in_s": (4624, 1, 1, _CONV_SPIKE, _CONV_SPIKE),
    "sram_wg_conv_in_du": (65536, 16, 16, _CONV_WORD_L, _CONV_WORD_L),
    "sram_wg_conv_out_dw": (18432, 16, 16, _CONV_WORD_S, _CONV_WORD_S),
    # shared buffers and external memory
    "sram_2MB": (1048576, 16, 256, 46.976, 45.96),
    "sram_6MB": (50331648, 16, 256, 458.1830181, 375.0422185),
    "dram": (134217728 * 64, 16, 64, 1300.0, 1300.0),
}


def _instances() -> Dict[str, MemoryInstanceSpec]:
    return {n: MemoryInstanceSpec(n, size, width, port, port, rc, wc) for n, (size, width, port, rc, wc) in _TABLE.items()}


@dataclass
class MemoryHierarchyConfig:
    """The ``neuromc_like_v1`` preset.  The three ``zero_*`` switches reproduce the accounting of the published energy
    figures: DRAM and network-on-chip traffic are not charged, and of the SRAM traffic only the directions towards the
    compute array (``rh2l``) and back from it (``wl2h``) are."""
    preset_name: str = "neuromc_like_v1"
    technology_nm: int = 32
    level_order: Tuple[str, str, str, str] = ("dram", "sram", "reg", "noc")
    memory_instances: Dict[str, MemoryInstanceSpec] = field(default_factory=_instances)
    zero_dram_in_paper_energy: bool = True
    zero_noc_in_paper_energy: bool = True
    zero_sram_high_directions: bool = True

    @classmethod
    def neuromc_like_v1(cls) -> "MemoryHierarchyConfig":
        return cls()

    def copy(self) -> "MemoryHierarchyConfig":
        return MemoryHierarchyConfig(self.preset_name, self.technology_nm, tuple(self.level_order), dict(self.memory_instances),
                                     self.zero_dram_in_paper_energy, self.zero_noc_in_paper_energy, self.zero_sram_high_directions)

    def validate(self) -> None:
        if self.preset_name != "neuromc_like_v1":
            raise ValueError(f"Only preset_name='neuromc_like_v1' is supported, got {self.preset_name}.")
        if self.technology_nm != 32:
            raise ValueError("Exact NeuroMC v1 only supports 32nm hardware constants.")
        missing = sorted(set(_TABLE) - set(self.memory_instances))
        if missing:
            raise ValueError(f"Missing required NeuroMC memory instances: {missing}.")
