/* Stand-in for MotifCL kernels/optim.cl: the CUDA OpenCL seam dispatches kernels by name and ignores program text. */
