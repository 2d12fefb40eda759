class ConfigError(ValueError):
    """A config.json that is missing a required key, holds a wrong type, or asks for
    something this engine does not implement."""
