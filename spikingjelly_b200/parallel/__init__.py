"""Scale-out: data / tensor / pipeline parallelism and the in-kernel collectives."""
