"""Error classes of the engine, the same five as the reference's (src/core/error.h:12-44)."""


class TieError(Exception):
    """Base of every error the engine raises on purpose."""


class LoadError(TieError):
    """A model folder, config.json or a weight file is missing, malformed or inconsistent."""


class UnsupportedError(TieError):
    """The model asks for something this engine does not compute."""


class CapacityError(TieError):
    """A request or a step does not fit the cache, the context or the step limits."""


class InvalidArgument(TieError):
    """A caller passed a value that can never be valid."""
