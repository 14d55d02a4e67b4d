/* Stand-in for MotifCL kernels/attention.cl: the CUDA OpenCL seam dispatches kernels by name and ignores program text. */
