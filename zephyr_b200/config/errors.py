"""Exceptions of the configuration and weight layers.

Mirrors the split of the reference's exception hierarchy
(src/include/common/exception.hpp:11-87): a configuration problem is not an
invalid argument of a call.
"""


class ZephyrError(Exception):
    """Base of every error this package raises on purpose."""


class ConfigError(ZephyrError):
    """config.json is missing a key, has a wrong type, or asks for an unsupported feature."""


class WeightError(ZephyrError):
    """A checkpoint is malformed, or its tensors do not match what the model reads."""


class InvalidArgumentError(ZephyrError, ValueError):
    """A call was given an argument outside its contract."""


class OutOfPagesError(ZephyrError):
    """The cache pool cannot hold what a step asks of it."""
