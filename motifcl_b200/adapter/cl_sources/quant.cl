/* Stand-in for MotifCL kernels/quant.cl: the CUDA OpenCL seam dispatches kernels by name and ignores program text. */
