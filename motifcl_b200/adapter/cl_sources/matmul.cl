/* Stand-in for MotifCL kernels/matmul.cl: the CUDA OpenCL seam dispatches kernels by name and ignores program text. */
