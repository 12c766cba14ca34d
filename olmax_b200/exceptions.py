"""
Error hierarchy.  Mirrors the reference's names (``olmax/exceptions.py:1-18``) so that callers can keep their
``except`` clauses, and adds :class:`OLMaxKernelError` for device-side failures reported through a status word.
"""

__all__ = [
    "OLMaxError",
    "CallbackExistsError",
    "OLMaxEnvironmentError",
    "OLMaxNetworkError",
    "OLMaxUploadError",
    "OLMaxConfigurationError",
    "OLMaxKernelError",
]


class OLMaxError(Exception):
    """Base class of every error this framework raises on purpose."""


class CallbackExistsError(OLMaxError):
    """A callback with the same name is already attached to the trainer."""


class OLMaxEnvironmentError(OLMaxError):
    """A required environment variable, credential or optional dependency is missing."""


class OLMaxNetworkError(OLMaxError):
    """A remote file-system request failed after retries."""


class OLMaxUploadError(OLMaxError):
    """An upload to remote storage failed."""


class OLMaxConfigurationError(OLMaxError):
    """A configuration value (mesh degrees, shapes, ...) is invalid."""


class OLMaxKernelError(OLMaxError):
    """A CUDA kernel gave up on a bounded wait or rejected its arguments."""
