"""A string that does not print itself.

Tokens (Hugging Face, API keys) are wrapped so that ``repr``, ``str``, f-strings, logging, ``dataclasses.asdict`` dumps,
JSON and pickling of a config never contain the value; code that needs it calls :meth:`expose_secret`.
Behaviour parity: crates/pmetal-core/src/secrets.rs (``[REDACTED]`` in Debug / Display, explicit accessor)."""
from __future__ import annotations

from typing import Optional

REDACTED = "[REDACTED]"


class SecretString:
    __slots__ = ("_value",)

    def __init__(self, secret: str = ""):
        if isinstance(secret, SecretString):
            secret = secret.expose_secret()
        object.__setattr__(self, "_value", str(secret))

    @classmethod
    def from_option(cls, secret: Optional[str]) -> Optional["SecretString"]:
        return None if secret is None else cls(secret)

    def expose_secret(self) -> str:
        return self._value

    def is_empty(self) -> bool:
        return not self._value

    def __len__(self) -> int:
        return len(self._value)

    def __bool__(self) -> bool:
        return bool(self._value)

    def __repr__(self) -> str:
        return f"SecretString({REDACTED})"

    def __str__(self) -> str:
        return REDACTED

    def __format__(self, spec: str) -> str:
        return format(REDACTED, spec)

    def __eq__(self, other) -> bool:
        import hmac
        if isinstance(other, SecretString):
            other = other._value
        return isinstance(other, str) and hmac.compare_digest(self._value.encode(), other.encode())

    def __hash__(self) -> int:
        return hash(("SecretString", self._value))

    def __setattr__(self, name, value):
        raise AttributeError("SecretString is immutable")

    def __deepcopy__(self, memo) -> "SecretString":      # dataclasses.asdict deep-copies leaves: keep the wrapper
        return self

    def __reduce__(self):
        raise TypeError("SecretString is not picklable; pass the token through the environment instead")


def expose(value) -> Optional[str]:
    """Plain string of a ``SecretString`` / ``str`` / ``None``."""
    if value is None:
        return None
    return value.expose_secret() if isinstance(value, SecretString) else str(value)
