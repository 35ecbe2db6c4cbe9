"""Typed configurations and the registry of architectures."""
from .dense import ConfigError, DenseDecoderConfig, RopeScaling, read_config_json
from .registry import (Architecture, architecture_of, dense_decoder_spec, known_architectures,
                       register_architecture)

__all__ = ["ConfigError", "DenseDecoderConfig", "RopeScaling", "read_config_json", "Architecture",
           "architecture_of", "dense_decoder_spec", "known_architectures", "register_architecture"]
