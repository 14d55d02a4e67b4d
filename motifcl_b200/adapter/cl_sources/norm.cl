/* Stand-in for MotifCL kernels/norm.cl: the CUDA OpenCL seam dispatches kernels by name and ignores program text. */
