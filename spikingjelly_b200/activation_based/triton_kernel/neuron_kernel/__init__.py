"""Functional multi-step neurons under the reference's names (``triton_kernel/neuron_kernel/{integrate_and_fire,lif,plif,
utils}.py``): ``multistep_if``, ``multistep_lif``, ``multistep_plif`` return ``(spike_seq, v_seq)``; the ``*_mp`` forms take
a storage dtype (fp32 / fp16 / bf16 / fp8 e4m3 / fp8 e5m2), compute dtypes and a spike dtype.  All of them run the CUDA scan
kernels of this package (``ops/neuron_scan.py``): one kernel per direction, only the input kept for backward.

Differences a caller can see: arithmetic is always fp32 in registers (the compute-dtype arguments are validated and kept in
the plan, not used to round); with fp8 storage the spikes and gradients are bf16; ``h_seq`` is never materialised, so the
``*_mp`` functions return ``None`` in its place."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from ... import surrogate as _surrogate
from ..triton_utils import (is_fp8_dtype, normalize_cuda_device, normalize_triton_compute_dtype_name, normalize_triton_storage_dtype,
                            torch_dtype_to_triton_neuron_dtype_id, triton_compute_dtype_name_to_neuron_dtype_id)

__all__ = ["multistep_if", "multistep_lif", "multistep_plif", "multistep_if_mp", "multistep_lif_mp", "multistep_plif_mp",
           "multistep_if_mp_with_plan", "multistep_lif_mp_with_plan", "multistep_plif_mp_with_plan", "multistep_if_inference",
           "multistep_lif_inference", "multistep_plif_inference", "multistep_if_forward", "multistep_lif_forward", "multistep_plif_forward",
           "multistep_if_mp_inference", "multistep_lif_mp_inference", "multistep_plif_mp_inference", "multistep_if_mp_forward",
           "multistep_lif_mp_forward", "multistep_plif_mp_forward", "TritonNeuronExecutionPlan", "prepare_triton_neuron_execution_plan"]


def _spec(kind: str, tau: float, v_threshold: float, v_reset: Optional[float], detach_reset: bool, surrogate_function):
    from ....ops.neuron_scan import KIND, NeuronSpec
    sg = _surrogate.surrogate_spec(surrogate_function)
    if sg is None:
        raise ValueError(f"{type(surrogate_function).__name__} has no kernel descriptor; use one of the table-driven surrogates")
    return NeuronSpec(kind=KIND[kind], v_threshold=float(v_threshold), v_reset=None if v_reset is None else float(v_reset), tau=float(tau), sg=sg,
                      detach_reset=bool(detach_reset))


def _run(x_seq, v_init, spec, r=None, store_v_seq=True, storage_dtype=None):
    from ....ops.neuron_scan import multistep_neuron
    if r is not None and r.dtype != torch.float32:
        r = r.float()                                    # the kernels read the reciprocal time constant as one fp32 value
    s, v_last, v_seq, _ = multistep_neuron(x_seq, v_init, spec, r=r, store_v_seq=store_v_seq, storage_dtype=storage_dtype)
    return s, (v_seq if store_v_seq else v_last.unsqueeze(0))


def multistep_if(x_seq, v_init, v_threshold: float, v_reset: Optional[float], detach_reset: bool, surrogate_function, store_v_seq: bool = True):
    return _run(x_seq, v_init, _spec("if", 2.0, v_threshold, v_reset, detach_reset, surrogate_function), store_v_seq=store_v_seq)


def multistep_lif(x_seq, v_init, decay_input: bool, tau: float, v_threshold: float, v_reset: Optional[float], detach_reset: bool,
                  surrogate_function, store_v_seq: bool = True):
    return _run(x_seq, v_init, _spec("lif_di" if decay_input else "lif_ndi", tau, v_threshold, v_reset, detach_reset, surrogate_function),
                store_v_seq=store_v_seq)


def multistep_plif(x_seq, v_init, r_tau: torch.Tensor, decay_input: bool, v_threshold: float, v_reset: Optional[float], detach_reset: bool,
                   surrogate_function):
    """``r_tau``: the reciprocal time constant ``1 / tau = sigmoid(w)`` as a one-element tensor (learnable)."""
    return _run(x_seq, v_init, _spec("plif_di" if decay_input else "plif_ndi", 2.0, v_threshold, v_reset, detach_reset, surrogate_function), r=r_tau)


@dataclass(frozen=True)
class TritonNeuronExecutionPlan:
    """What a mixed-precision call was asked to do; ``matches`` tells whether a cached plan fits another request."""
    neuron_type: str
    device: torch.device
    storage_dtype: torch.dtype
    forward_compute_dtype_name: str
    backward_compute_dtype_name: str
    spike_dtype: torch.dtype
    storage_dtype_id: int
    forward_compute_dtype_id: int
    backward_compute_dtype_id: int
    spike_dtype_id: int
    save_intermediates: bool

    def matches(self, *, neuron_type, device, storage_dtype, forward_compute_dtype, backward_compute_dtype="fp32", spike_dtype,
                save_intermediates) -> bool:
        try:
            other = prepare_triton_neuron_execution_plan(neuron_type=neuron_type, device=device, storage_dtype=storage_dtype,
                                                         forward_compute_dtype=forward_compute_dtype, backward_compute_dtype=backward_compute_dtype,
                                                         spike_dtype=spike_dtype, save_intermediates=save_intermediates)
        except (ValueError, RuntimeError, TypeError):
            return False
        return other == self


def prepare_triton_neuron_execution_plan(*, neuron_type: str, device, storage_dtype, forward_compute_dtype="fp32", backward_compute_dtype="fp32",
                                         spike_dtype: torch.dtype = torch.float32, save_intermediates: bool = True) -> TritonNeuronExecutionPlan:
    if neuron_type not in ("if", "lif", "plif"):
        raise ValueError(f"neuron_type must be one of 'if', 'lif', or 'plif', but got {neuron_type!r}.")
    storage = normalize_triton_storage_dtype(storage_dtype)
    fwd, bwd = normalize_triton_compute_dtype_name(forward_compute_dtype), normalize_triton_compute_dtype_name(backward_compute_dtype)
    for label, name in (("compute_dtype", fwd), ("backward_compute_dtype", bwd)):
        if name == "fp8" and not is_fp8_dtype(storage):
            raise ValueError(f"{label}='fp8' requires an fp8 storage dtype.")
    if spike_dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise ValueError(f"Unsupported spike dtype {spike_dtype}.")
    return TritonNeuronExecutionPlan(neuron_type, normalize_cuda_device(device), storage, fwd, bwd, spike_dtype,
                                     torch_dtype_to_triton_neuron_dtype_id(storage), triton_compute_dtype_name_to_neuron_dtype_id(fwd, storage),
                                     triton_compute_dtype_name_to_neuron_dtype_id(bwd, storage), torch_dtype_to_triton_neuron_dtype_id(spike_dtype),
                                     bool(save_intermediates))


def _check_plan(x_seq, v_init, plan: "TritonNeuronExecutionPlan", neuron_type: str) -> None:
    if plan.neuron_type != neuron_type:
        raise ValueError(f"{neuron_type.upper()} forward requires a {neuron_type.upper()} plan, got {plan.neuron_type!r}.")
    if not x_seq.is_cuda or x_seq.device != plan.device:
        raise ValueError(f"the plan was prepared for {plan.device}, the input is on {x_seq.device}.")
    if torch.is_tensor(v_init) and v_init.device != x_seq.device:
        raise ValueError("x_seq and v_init must be on the same device.")


def _run_plan(kind: str, x_seq, v_init, plan, tau, v_threshold, v_reset, detach_reset, surrogate_function, r=None):
    sg = surrogate_function if surrogate_function is not None else _surrogate.Sigmoid()
    spec = _spec(kind, tau, v_threshold, v_reset, detach_reset, sg)
    state = torch.bfloat16 if is_fp8_dtype(plan.storage_dtype) else plan.storage_dtype
    v0 = v_init.to(state) if torch.is_tensor(v_init) else v_init
    if is_fp8_dtype(plan.storage_dtype):
        s, v_seq = _run(x_seq, v0, spec, r=r, storage_dtype=plan.storage_dtype)   # the cast happens inside the autograd function
    else:
        s, v_seq = _run(x_seq.to(plan.storage_dtype), v0, spec, r=r)
    return s.to(plan.spike_dtype), v_seq, None


def multistep_if_mp_with_plan(x_seq, v_init, plan: TritonNeuronExecutionPlan, *, v_threshold: float, v_reset: Optional[float],
                              detach_reset: bool = False, surrogate_function=None):
    """The ``*_with_plan`` forms skip the validation and dtype look-ups of ``prepare_triton_neuron_execution_plan``: a module
    prepares the plan once and passes it with every call."""
    _check_plan(x_seq, v_init, plan, "if")
    return _run_plan("if", x_seq, v_init, plan, 2.0, v_threshold, v_reset, detach_reset, surrogate_function)


def multistep_lif_mp_with_plan(x_seq, v_init, plan: TritonNeuronExecutionPlan, *, decay_input: bool, tau: float, v_threshold: float,
                               v_reset: Optional[float], detach_reset: bool = False, surrogate_function=None):
    _check_plan(x_seq, v_init, plan, "lif")
    return _run_plan("lif_di" if decay_input else "lif_ndi", x_seq, v_init, plan, tau, v_threshold, v_reset, detach_reset, surrogate_function)


def multistep_plif_mp_with_plan(x_seq, v_init, r_tau: torch.Tensor, plan: TritonNeuronExecutionPlan, *, decay_input: bool, v_threshold: float,
                                v_reset: Optional[float], detach_reset: bool = False, surrogate_function=None):
    _check_plan(x_seq, v_init, plan, "plif")
    return _run_plan("plif_di" if decay_input else "plif_ndi", x_seq, v_init, plan, 2.0, v_threshold, v_reset, detach_reset, surrogate_function,
                     r=r_tau)


def _plan_for(neuron_type, x_seq, storage_dtype, compute_dtype, backward_compute_dtype, spike_dtype, save_intermediates):
    return prepare_triton_neuron_execution_plan(neuron_type=neuron_type, device=x_seq.device, storage_dtype=storage_dtype,
                                                forward_compute_dtype=compute_dtype, backward_compute_dtype=backward_compute_dtype,
                                                spike_dtype=spike_dtype, save_intermediates=save_intermediates)


def multistep_if_mp(x_seq, v_init, *, v_threshold: float, v_reset: Optional[float], storage_dtype, compute_dtype="fp32",
                    backward_compute_dtype="fp32", spike_dtype: torch.dtype = torch.float32, save_intermediates: bool = True,
                    detach_reset: bool = False, surrogate_function=None) -> Tuple[torch.Tensor, torch.Tensor, None]:
    plan = _plan_for("if", x_seq, storage_dtype, compute_dtype, backward_compute_dtype, spike_dtype, save_intermediates)
    return multistep_if_mp_with_plan(x_seq, v_init, plan, v_threshold=v_threshold, v_reset=v_reset, detach_reset=detach_reset,
                                     surrogate_function=surrogate_function)


def multistep_lif_mp(x_seq, v_init, *, decay_input: bool, tau: float, v_threshold: float, v_reset: Optional[float], storage_dtype,
                     compute_dtype="fp32", backward_compute_dtype="fp32", spike_dtype: torch.dtype = torch.float32,
                     save_intermediates: bool = True, detach_reset: bool = False, surrogate_function=None):
    plan = _plan_for("lif", x_seq, storage_dtype, compute_dtype, backward_compute_dtype, spike_dtype, save_intermediates)
    return multistep_lif_mp_with_plan(x_seq, v_init, plan, decay_input=decay_input, tau=tau, v_threshold=v_threshold, v_reset=v_reset,
                                      detach_reset=detach_reset, surrogate_function=surrogate_function)


def multistep_plif_mp(x_seq, v_init, r_tau: torch.Tensor, *, decay_input: bool, v_threshold: float, v_reset: Optional[float], storage_dtype,
                      compute_dtype="fp32", backward_compute_dtype="fp32", spike_dtype: torch.dtype = torch.float32,
                      save_intermediates: bool = True, detach_reset: bool = False, surrogate_function=None):
    plan = _plan_for("plif", x_seq, storage_dtype, compute_dtype, backward_compute_dtype, spike_dtype, save_intermediates)
    return multistep_plif_mp_with_plan(x_seq, v_init, r_tau, plan, decay_input=decay_input, v_threshold=v_threshold, v_reset=v_reset,
                                       detach_reset=detach_reset, surrogate_function=surrogate_function)


# ------------------------------------------------------------------ gradient-free entry points (positional, as the reference's)
def _inference(kind, x_seq, v_init, tau, v_threshold, v_reset, soft_reset, store_v_seq=True, r=None):
    with torch.no_grad():
        return _run(x_seq, v_init, _spec(kind, tau, v_threshold, None if soft_reset else v_reset, False, _surrogate.Sigmoid()), r=r,
                    store_v_seq=store_v_seq)


def multistep_if_inference(x_seq, v_init, v_threshold: float, v_reset: float, soft_reset: bool, store_v_seq: bool = True):
    return _inference("if", x_seq, v_init, 2.0, v_threshold, v_reset, soft_reset, store_v_seq)


def multistep_lif_inference(x_seq, v_init, decay_input: bool, tau: float, v_threshold: float, v_reset: float, soft_reset: bool,
                            store_v_seq: bool = True):
    return _inference("lif_di" if decay_input else "lif_ndi", x_seq, v_init, tau, v_threshold, v_reset, soft_reset, store_v_seq)


def multistep_plif_inference(x_seq, v_init, r_tau: torch.Tensor, decay_input: bool, v_threshold: float, v_reset: float, soft_reset: bool):
    return _inference("plif_di" if decay_input else "plif_ndi", x_seq, v_init, 2.0, v_threshold, v_reset, soft_reset, True, r=r_tau)


# ------------------------------------------------------------------ positional forms (the reference's custom-op signatures)
# A surrogate is given as (sg_triton_id, sg_alpha) in the reference's numbering (triton_kernel/surrogate_kernel.py); dtypes as the
# integer ids of triton_utils.  Every form returns (spike_seq, v_seq, h_seq) with h_seq = None: it is never materialised here.
def _sg_from_id(sg_triton_id: int, sg_alpha: float):
    from ..surrogate_kernel import _BY_ID
    if sg_triton_id not in _BY_ID:
        raise ValueError(f"unknown surrogate id {sg_triton_id}")
    return _BY_ID[sg_triton_id](alpha=float(sg_alpha))


def _reset(v_reset, soft_reset):
    return None if soft_reset else v_reset


def multistep_if_forward(x_seq, v_init, v_threshold: float, v_reset: float, soft_reset: bool, detach_reset: bool, sg_triton_id: int,
                         sg_alpha: float, store_v_seq: bool = True):
    return (*multistep_if(x_seq, v_init, v_threshold, _reset(v_reset, soft_reset), detach_reset, _sg_from_id(sg_triton_id, sg_alpha), store_v_seq), None)


def multistep_lif_forward(x_seq, v_init, decay_input: bool, tau: float, v_threshold: float, v_reset: float, soft_reset: bool,
                          detach_reset: bool, sg_triton_id: int, sg_alpha: float, store_v_seq: bool = True):
    return (*multistep_lif(x_seq, v_init, decay_input, tau, v_threshold, _reset(v_reset, soft_reset), detach_reset,
                           _sg_from_id(sg_triton_id, sg_alpha), store_v_seq), None)


def multistep_plif_forward(x_seq, v_init, r_tau: torch.Tensor, decay_input: bool, v_threshold: float, v_reset: float, soft_reset: bool,
                           detach_reset: bool, sg_triton_id: int, sg_alpha: float):
    return (*multistep_plif(x_seq, v_init, r_tau, decay_input, v_threshold, _reset(v_reset, soft_reset), detach_reset,
                            _sg_from_id(sg_triton_id, sg_alpha)), None)


def _plan_from_ids(neuron_type, x_seq, storage_dtype_id, forward_compute_dtype_id, backward_compute_dtype_id, spike_dtype_id, save_intermediates):
    from ..triton_utils import triton_neuron_dtype_id_to_torch_dtype as to_dtype
    names = {torch.float32: "fp32", torch.float16: "fp16", torch.bfloat16: "bf16"}
    comp = lambda i: names.get(to_dtype(i), "fp8")          # noqa: E731
    return prepare_triton_neuron_execution_plan(neuron_type=neuron_type, device=x_seq.device, storage_dtype=to_dtype(storage_dtype_id),
                                                forward_compute_dtype=comp(forward_compute_dtype_id),
                                                backward_compute_dtype=comp(backward_compute_dtype_id), spike_dtype=to_dtype(spike_dtype_id),
                                                save_intermediates=save_intermediates)


def multistep_if_mp_inference(x_seq, v_init, v_threshold: float, v_reset: float, soft_reset: bool, storage_dtype_id: int,
                              forward_compute_dtype_id: int, spike_dtype_id: int, save_intermediates: bool = False):
    plan = _plan_from_ids("if", x_seq, storage_dtype_id, forward_compute_dtype_id, 0, spike_dtype_id, save_intermediates)
    with torch.no_grad():
        return multistep_if_mp_with_plan(x_seq, v_init, plan, v_threshold=v_threshold, v_reset=_reset(v_reset, soft_reset))


def multistep_lif_mp_inference(x_seq, v_init, decay_input: bool, tau: float, v_threshold: float, v_reset: float, soft_reset: bool,
                               storage_dtype_id: int, forward_compute_dtype_id: int, spike_dtype_id: int, save_intermediates: bool = False):
    plan = _plan_from_ids("lif", x_seq, storage_dtype_id, forward_compute_dtype_id, 0, spike_dtype_id, save_intermediates)
    with torch.no_grad():
        return multistep_lif_mp_with_plan(x_seq, v_init, plan, decay_input=decay_input, tau=tau, v_threshold=v_threshold,
                                          v_reset=_reset(v_reset, soft_reset))


def multistep_plif_mp_inference(x_seq, v_init, r_tau: torch.Tensor, decay_input: bool, v_threshold: float, v_reset: float, soft_reset: bool,
                                storage_dtype_id: int, forward_compute_dtype_id: int, spike_dtype_id: int, save_intermediates: bool = False):
    plan = _plan_from_ids("plif", x_seq, storage_dtype_id, forward_compute_dtype_id, 0, spike_dtype_id, save_intermediates)
    with torch.no_grad():
        return multistep_plif_mp_with_plan(x_seq, v_init, r_tau, plan, decay_input=decay_input, v_threshold=v_threshold,
                                           v_reset=_reset(v_reset, soft_reset))


def multistep_if_mp_forward(x_seq, v_init, v_threshold: float, v_reset: float, soft_reset: bool, detach_reset: bool, sg_triton_id: int,
                            sg_alpha: float, storage_dtype_id: int, forward_compute_dtype_id: int, backward_compute_dtype_id: int,
                            spike_dtype_id: int):
    plan = _plan_from_ids("if", x_seq, storage_dtype_id, forward_compute_dtype_id, backward_compute_dtype_id, spike_dtype_id, True)
    return multistep_if_mp_with_plan(x_seq, v_init, plan, v_threshold=v_threshold, v_reset=_reset(v_reset, soft_reset), detach_reset=detach_reset,
                                     surrogate_function=_sg_from_id(sg_triton_id, sg_alpha))


def multistep_lif_mp_forward(x_seq, v_init, decay_input: bool, tau: float, v_threshold: float, v_reset: float, soft_reset: bool,
                             detach_reset: bool, sg_triton_id: int, sg_alpha: float, storage_dtype_id: int, forward_compute_dtype_id: int,
                             backward_compute_dtype_id: int, spike_dtype_id: int):
    plan = _plan_from_ids("lif", x_seq, storage_dtype_id, forward_compute_dtype_id, backward_compute_dtype_id, spike_dtype_id, True)
    return multistep_lif_mp_with_plan(x_seq, v_init, plan, decay_input=decay_input, tau=tau, v_threshold=v_threshold,
                                      v_reset=_reset(v_reset, soft_reset), detach_reset=detach_reset,
                                      surrogate_function=_sg_from_id(sg_triton_id, sg_alpha))


def multistep_plif_mp_forward(x_seq, v_init, r_tau: torch.Tensor, decay_input: bool, v_threshold: float, v_reset: float, soft_reset: bool,
                              detach_reset: bool, sg_triton_id: int, sg_alpha: float, storage_dtype_id: int, forward_compute_dtype_id: int,
                              backward_compute_dtype_id: int, spike_dtype_id: int):
    plan = _plan_from_ids("plif", x_seq, storage_dtype_id, forward_compute_dtype_id, backward_compute_dtype_id, spike_dtype_id, True)
    return multistep_plif_mp_with_plan(x_seq, v_init, r_tau, plan, decay_input=decay_input, v_threshold=v_threshold,
                                       v_reset=_reset(v_reset, soft_reset), detach_reset=detach_reset,
                                       surrogate_function=_sg_from_id(sg_triton_id, sg_alpha))


# longer names of the mixed-precision forms, and the debugging slots the reference's kernels fill with the loop style they
# chose ("static" / "dynamic"); the CUDA kernels have one loop style, so the slots stay empty
multistep_if_mixed_precision_forward, multistep_if_mixed_precision_forward_with_plan = multistep_if_mp, multistep_if_mp_with_plan
multistep_lif_mixed_precision_forward, multistep_lif_mixed_precision_forward_with_plan = multistep_lif_mp, multistep_lif_mp_with_plan
multistep_plif_mixed_precision_forward, multistep_plif_mixed_precision_forward_with_plan = multistep_plif_mp, multistep_plif_mp_with_plan
LAST_FORWARD_LOOP_MODE = LAST_BACKWARD_LOOP_MODE = None
