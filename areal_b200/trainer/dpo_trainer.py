"""Entry point kept for source compatibility with the reference's module layout."""
from .sl_trainer import DPOTrainer  # noqa: F401

__all__ = ["DPOTrainer"]
