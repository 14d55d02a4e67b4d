/* Stand-in for MotifCL kernels/embedding.cl: the CUDA OpenCL seam dispatches kernels by name and ignores program text. */
