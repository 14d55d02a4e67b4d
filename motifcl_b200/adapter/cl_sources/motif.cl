/* Stand-in for MotifCL kernels/motif.cl: the CUDA OpenCL seam dispatches kernels by name and ignores program text. */
