"""Test infrastructure: the CPU restatement of the reference's hot path (ref_ops), the recipe that compiles the
reference's own kernels from its sources (build_ref) and the loader that runs them on the GPU (ref_cuda). Nothing in
the product path imports this package."""
