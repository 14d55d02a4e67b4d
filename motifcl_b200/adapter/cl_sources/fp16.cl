/* Stand-in for MotifCL kernels/fp16.cl: the CUDA OpenCL seam dispatches kernels by name and ignores program text. */
