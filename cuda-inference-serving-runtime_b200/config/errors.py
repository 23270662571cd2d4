"""The error every configuration class and the registry raise."""


class ConfigError(ValueError):
    """config.json asks for something this engine does not compute, or names nothing it knows."""
