"""Version string and the "previous minor version" helper used for hidden metrics.

Parity: vllm_metax/version.py:5-39 (``__version__``, ``_prev_minor_version_was``).
"""

__version__ = "0.1.0"
__version_tuple__ = (0, 1, 0)


def _prev_minor_version_was(version_str: str) -> bool:
    """True when ``version_str`` ("X.Y") names the minor release before this one.

    Used to decide whether metrics hidden in the previous release may still be
    re-enabled with ``--show-hidden-metrics-for-version``.
    """
    major, minor = __version_tuple__[:2]
    if minor == 0:
        return False
    return version_str == f"{major}.{minor - 1}"


def _prev_minor_version() -> str:
    major, minor = __version_tuple__[:2]
    return f"{major}.{max(minor - 1, 0)}"
