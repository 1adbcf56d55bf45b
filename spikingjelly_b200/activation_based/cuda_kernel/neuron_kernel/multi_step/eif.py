"""Exponential IF neuron on the native scan kernel (``cuda_kernel/neuron_kernel/multi_step/eif.py`` of the reference)."""
from .... import functional

__all__ = ["eif_multi_step", "cupy_multistep_eif_forward"]


def eif_multi_step(x_seq, v_init, tau, v_threshold, v_reset, v_rest, theta_rh, delta_T, detach_reset, surrogate_function):
    """``(spike_seq, v_seq)``."""
    s, _, v_seq = functional.neuron.eif_multi_step_cuda(x_seq, v_init, tau, v_threshold, v_reset, v_rest, theta_rh, delta_T, surrogate_function,
                                                        detach_reset, store_v_seq=True)
    return s, v_seq


def cupy_multistep_eif_forward(x_seq, v_init, tau, v_threshold, v_reset, v_rest, theta_rh, delta_T, detach_reset, surrogate_function,
                               capture_context=False):
    s, v_seq = eif_multi_step(x_seq, v_init, tau, v_threshold, v_reset, v_rest, theta_rh, delta_T, detach_reset, surrogate_function)
    return s, v_seq, None
