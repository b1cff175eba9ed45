"""CUDA kernels of the engine: build, bindings, and the dispatch of matrix products and attention."""
