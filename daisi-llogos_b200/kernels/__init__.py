"""The CUDA kernels' Python face (``ops``) and the matrix-product dispatch (``linear``)."""
