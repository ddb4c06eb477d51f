"""Error types of the library.

The reference reports failures as an error code plus a message kept per thread
(src/libllm/llm.h:42-47, src/lutil/error.h:34-77).  Here each code is an exception
class; ``code`` carries the reference's number so that a C-style front end can
return it."""


class LlmError(Exception):
    """Base of every error this library raises on purpose."""
    code = 0x0102  # LLM_ERROR_ABORTED


class InvalidArgError(LlmError):
    """An argument, option or configuration value is not acceptable."""
    code = 0x0100  # LLM_ERROR_INVALID_ARG


class ConfigError(InvalidArgError):
    """config.json is missing a key or holds a value the architecture does not allow."""


class WeightsError(LlmError):
    """The weight files do not fit the model: carries the full lists."""

    def __init__(self, message, missing=(), unexpected=(), wrong_shape=()):
        super().__init__(message)
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)


class CacheError(LlmError):
    """The cache cannot serve a request: no free slot or page, a slot freed twice."""


class UnsupportedError(LlmError):
    """A size or option that a kernel of this library refuses instead of computing a
    wrong result."""


class ExtensionError(LlmError):
    """The CUDA extension is missing, cannot be built or reported a launch failure."""


class EndOfSequence(LlmError):
    """A completion has ended (the reference's LLM_ERROR_EOF)."""
    code = 0x0103  # LLM_ERROR_EOF
