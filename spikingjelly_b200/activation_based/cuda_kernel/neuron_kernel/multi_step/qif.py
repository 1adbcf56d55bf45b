"""Quadratic IF neuron on the native scan kernel (``cuda_kernel/neuron_kernel/multi_step/qif.py`` of the reference)."""
from .... import functional

__all__ = ["qif_multi_step", "cupy_multistep_qif_forward"]


def qif_multi_step(x_seq, v_init, tau, v_threshold, v_reset, v_rest, v_c, a0, detach_reset, surrogate_function):
    """``(spike_seq, v_seq)``."""
    s, _, v_seq = functional.neuron.qif_multi_step_cuda(x_seq, v_init, tau, v_c, a0, v_threshold, v_rest, v_reset, surrogate_function, detach_reset,
                                                        store_v_seq=True)
    return s, v_seq


def cupy_multistep_qif_forward(x_seq, v_init, tau, v_threshold, v_reset, v_rest, v_c, a0, detach_reset, surrogate_function, capture_context=False):
    """Same computation with the reference operator's argument order (the surrogate object stands where its id stood)."""
    s, v_seq = qif_multi_step(x_seq, v_init, tau, v_threshold, v_reset, v_rest, v_c, a0, detach_reset, surrogate_function)
    return s, v_seq, None
