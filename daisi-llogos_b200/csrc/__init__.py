"""CUDA sources and their build (``build.py``)."""
