"""Typed errors a caller can match on.

Counterpart of the reference's error enum (llmoxide/src/error.rs:9-45:
UnsupportedArch, Unsupported, ContextOverflow, NoDevice, Gguf, Other), with
the checkpoint errors split by what went wrong.
"""

from __future__ import annotations


class LlmoxideError(Exception):
    """Base of every error this package raises on purpose."""


class ConfigError(LlmoxideError):
    """config.json is missing a key, or a value is inconsistent or unsupported."""


class UnsupportedArch(LlmoxideError):
    """config.json names an architecture that is not registered."""

    def __init__(self, name, known):
        self.name, self.known = name, sorted(known)
        super().__init__(f"unsupported architecture {name!r}; registered: {', '.join(self.known) or 'none'}")


class Unsupported(LlmoxideError):
    """A size or option that a kernel or part refuses rather than miscompute."""


class WeightsError(LlmoxideError):
    """The checkpoint does not fit the configuration.  One error lists every
    missing tensor, every unexpected tensor and every wrong shape or dtype."""

    def __init__(self, missing=(), unexpected=(), wrong=(), where=""):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong = list(wrong)  # (name, problem) pairs
        lines = [f"checkpoint {where} does not fit the configuration:".replace("  ", " ")]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong:
            lines.append(f"  wrong shape or dtype ({len(self.wrong)}):")
            lines += [f"    {name}: {problem}" for name, problem in self.wrong]
        super().__init__("\n".join(lines))


class CheckpointFormatError(LlmoxideError):
    """A safetensors file is truncated or its header is malformed."""


class ContextOverflow(LlmoxideError):
    """A request needs more positions than the cache or the model allows
    (llmoxide/src/error.rs ContextOverflow{tokens, context})."""

    def __init__(self, tokens, context, what="context"):
        self.tokens, self.context = tokens, context
        super().__init__(f"{tokens} tokens do not fit the {what} of {context}")


class CacheExhausted(LlmoxideError):
    """No free slot or page is left for the live requests."""


class CacheMisuse(LlmoxideError):
    """A slot was freed twice, used after being freed, or never acquired."""


class ExtensionMissing(LlmoxideError):
    """The CUDA extension could not be built or loaded, or there is no GPU.
    There is no CPU fallback: the engine stops here."""


class KernelError(LlmoxideError):
    """A kernel launch failed, or a kernel reported a failure in its library's status word (a bounded
    wait that ran out, a request it could not serve); ``kernels.check_status`` raises it when the host
    has waited for the step."""
