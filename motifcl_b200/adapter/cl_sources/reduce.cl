/* Stand-in for MotifCL kernels/reduce.cl: the CUDA OpenCL seam dispatches kernels by name and ignores program text. */
