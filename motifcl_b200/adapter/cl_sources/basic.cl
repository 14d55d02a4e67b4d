/* Stand-in for MotifCL kernels/basic.cl: the CUDA OpenCL seam dispatches kernels by name and ignores program text. */
