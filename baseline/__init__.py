"""The reference's own CUDA kernels, compiled unchanged, as a second oracle and a timed baseline."""
