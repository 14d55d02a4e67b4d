/* Stand-in for MotifCL kernels/loss.cl: the CUDA OpenCL seam dispatches kernels by name and ignores program text. */
