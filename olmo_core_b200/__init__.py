"""
B200-native LLM training framework with the public API of OLMo-core: PyTorch framework layer, hand-written
sm_100a CUDA kernels for the hot ops (``olmo_core_b200.ops``), a sharded-parameter / tensor / context / expert
parallel runtime over NVLink (``olmo_core_b200.parallel``).
"""

from .version import VERSION as __version__  # noqa: F401

try:  # install the ``olmo_core`` import alias when the alias package is importable
    import olmo_core  # noqa: F401
except Exception:  # pragma: no cover
    pass
