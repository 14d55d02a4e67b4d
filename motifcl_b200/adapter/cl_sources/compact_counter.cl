/* Stand-in for MotifCL kernels/compact_counter.cl: the CUDA OpenCL seam dispatches kernels by name and ignores program text. */
