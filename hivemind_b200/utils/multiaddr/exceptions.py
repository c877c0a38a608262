"""Errors of the multiaddr package (names as in hivemind/utils/multiaddr/exceptions.py, which vendors py-multiaddr)."""
from typing import Any, Optional


class Error(Exception):
    """Base class of everything this package raises on its own account."""


class LookupError(LookupError, Error):  # noqa: A001 (the name is part of the API)
    """A lookup inside an address failed."""


class ProtocolLookupError(LookupError):
    """An address has no component of the requested protocol."""

    def __init__(self, proto: Any, string: str):
        self.proto, self.string = proto, string
        super().__init__(f"MultiAddr {string!r} does not contain protocol {proto}")


class ParseError(ValueError, Error):
    """An address could not be parsed."""


class StringParseError(ParseError):
    """The text form of an address is malformed."""

    def __init__(self, message: str, string: str, protocol: Optional[str] = None, original: Optional[BaseException] = None):
        self.message, self.string, self.protocol, self.original = message, string, protocol, original
        where = f" (component {protocol})" if protocol is not None else ""
        super().__init__(f"Invalid MultiAddr {string!r}{where}: {message}")


class BinaryParseError(ParseError):
    """The binary form of an address is malformed."""

    def __init__(self, message: str, binary: bytes, protocol: Any, original: Optional[BaseException] = None):
        self.message, self.binary, self.protocol, self.original = message, binary, protocol, original
        super().__init__(f"Invalid binary MultiAddr (component {protocol}): {message}")


class ProtocolRegistryError(Error):
    """A protocol registry was used wrongly."""


ProtocolManagerError = ProtocolRegistryError  # older spelling


class ProtocolRegistryLocked(Error):
    """A locked registry was asked to change."""

    def __init__(self):
        super().__init__("Protocol registry is locked and does not accept any new values")


class ProtocolExistsError(ProtocolRegistryError):
    """A protocol of this name or code is registered already."""

    def __init__(self, proto: Any, kind: str = "name"):
        self.proto, self.kind = proto, kind
        super().__init__(f"Protocol with {kind} {getattr(proto, kind)!r} already exists")


class ProtocolNotFoundError(ProtocolRegistryError):
    """No protocol of this name or code is registered."""

    def __init__(self, value: Any, kind: str = "name"):
        self.value, self.kind = value, kind
        super().__init__(f"No protocol with {kind} {value!r} found")
