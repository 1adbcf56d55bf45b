"""Process-wide knobs.  Change them as attributes of this module
(``spikingjelly_b200.configure.cuda_threads = 256``); a ``from … import`` copy
does not propagate.  Parity: ``spikingjelly/configure.py:14-85``.
"""

# dataset preprocessing (event file -> numpy, events -> frames) worker threads
max_threads_number_for_datasets_preprocess = 16
# store converted datasets as compressed ``npz``
save_datasets_compressed = True

# Threads per CTA of the element-wise neuron kernels.  The native scan kernels
# process several neurons per thread with 128-bit accesses; 256 threads gives
# 8 resident CTAs per SM on B200 at the kernels' register budget.
cuda_threads = 256
# Kept for source compatibility with scripts that set them; the native kernels
# are compiled ahead of time for sm_100a and ignore both.
cuda_compiler_options = ("-use_fast_math",)
cuda_compiler_backend = "nvcc"

# Spikes saved for backward by spike_linear / spike_conv are stored
#   level 0: one byte per spike (bool);  level 1: bit-packed, 32 spikes per word.
save_spike_as_bool_in_neuron_kernel = False
save_bool_spike_level = 0

# Largest T for which the scan kernels are fully unrolled in registers; longer
# sequences are processed in register-resident chunks of this many steps with the
# membrane potential carried between chunks.
scan_kernel_chunk_T = 8
# Accepted for compatibility (the reference's Triton path switches loop style here).
triton_neuron_kernel_static_range_max_T = 64

# Name used when a user asks for one of the reference's GPU backends
# ("cupy", "triton", "inductor"): all of them resolve to the native kernels.
native_backend_name = "cuda"

# ``layer.Linear`` (and everything built on it) runs forward, dgrad and wgrad on the tcgen05 GEMM kernel when its input
# is a CUDA tensor computed in bf16 / fp16 (under autocast, or with 16-bit parameters) and the feature sizes are multiples
# of 8.  False: always ``torch.nn.functional.linear`` (cuBLAS).
native_linear = True
