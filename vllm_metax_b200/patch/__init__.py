"""Runtime patches applied to upstream vLLM when this package runs as a platform plugin.

Importing this package applies every enabled patch (each ``@patch`` acts at import).  The three
groups follow vllm_metax/patch/{bugfix,enhancement,performance}/__init__.py.
"""
from . import bugfix, enhancement, performance  # noqa: F401
from .utils import applied, patch, revert_all  # noqa: F401
