"""Abstract sequence mixer and its config (names of src/olmo_core/nn/attention/base.py:20-80)."""

from . import SequenceMixer, SequenceMixerConfig

__all__ = ["SequenceMixer", "SequenceMixerConfig"]
