"""One-line precondition helper.  Parity: ``unirl/config/require.py``."""


def require(condition: bool, message: str) -> None:
    """Raise ``ValueError(message)`` unless ``condition`` holds."""
    if not condition:
        raise ValueError(message)


__all__ = ["require"]
