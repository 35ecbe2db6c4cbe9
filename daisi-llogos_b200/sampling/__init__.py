"""Sampling parameters, the device sampler and the generation loop."""
