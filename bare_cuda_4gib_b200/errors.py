"""Exception types of the engine.  Every failure is an exception with a message that names the
thing that is wrong (cuongvng/bare-cuda-4gib raises one `llm::Error` for everything:
engine/include/llm/error.h:10-19)."""


class EngineError(RuntimeError):
    """Base class: anything the engine refuses or fails at."""


class ConfigError(EngineError):
    """config.json is missing a key, has a value out of range, or names an unknown architecture."""


class WeightError(EngineError):
    """The weight file is malformed or does not match the model (missing, unexpected, wrong shape)."""


class KernelBuildError(EngineError):
    """A CUDA source could not be compiled or loaded; there is no fallback path."""


class KernelLaunchError(EngineError):
    """A kernel launcher refused its arguments or CUDA reported an error."""


class CacheError(EngineError):
    """The cache manager was misused (page freed twice, unknown slot) or ran out of pages."""


class OutOfPages(CacheError):
    """No free page is left in a pool."""
