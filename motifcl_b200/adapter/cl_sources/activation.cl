/* Stand-in for MotifCL kernels/activation.cl: the CUDA OpenCL seam dispatches kernels by name and ignores program text. */
